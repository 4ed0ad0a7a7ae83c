"""Python faces of the CUDA kernels.

Every function here checks what it is given (device, dtype, contiguity, sizes),
passes raw pointers and the current stream to the `extern "C"` function of the
same purpose, and raises `KernelError` with the kernel's own message when that
refuses.  Nothing here computes: if the compiled library is missing and cannot be
built, loading it raises `ExtensionMissingError`.
"""
from __future__ import annotations

import ctypes
import os
import re
from dataclasses import dataclass
from typing import List, Optional

import torch

from .csrc import build
from .errors import KernelError

F32, BF16 = 0, 1
PAGE_TOKENS = 64
EPI_NONE, EPI_SOFTCAP, EPI_GATED = 0, 1, 2
ACT_GELU_TANH, ACT_SILU, ACT_CLAMPED_SWISH = 0, 1, 2
ACTIVATIONS = {"gelu_tanh": ACT_GELU_TANH, "silu": ACT_SILU}
# the clamped form as the products' gated epilogues know it: g logistic(SWISH_ALPHA g) (u + SWISH_SHIFT), the limit a parameter
SWISH_ALPHA, SWISH_SHIFT = 1.702, 1.0
ROPE_STYLES = {"rotate_half": 0, "interleaved": 1}

_p, _i, _f, _l = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong

_CT = {"p": _p, "i": _i, "f": _f, "l": _l}
_EXPORT = re.compile(r'extern\s+"C"\s+int\s+(\w+)\s*\(([^)]*)\)', re.S)


def _parse_signatures(sources) -> dict:
    """Argument types of every `extern "C" int f(...)` in the given .cu files, read
    from the sources themselves so that the Python side cannot drift from them."""
    sigs = {}
    for src in sources:
        with open(os.path.join(build.HERE, src)) as fh:
            text = fh.read()
        for name, args in _EXPORT.findall(text):
            sig = ""
            for a in args.split(","):
                a = a.strip()
                if not a:
                    continue
                if "*" in a or "cudaStream_t" in a:
                    sig += "p"
                elif "long long" in a:
                    sig += "l"
                elif a.startswith("float") or a.startswith("const float"):
                    sig += "f"
                else:
                    sig += "i"
            sigs[name] = sig
    return sigs


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"no kernel takes dtype {dt}")


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_device_index: Optional[int] = None


def _stream():
    """The current CUDA stream as a raw handle.  Asked for at every launch, so it goes the
    short way: one call into torch's C layer instead of building a Stream object."""
    global _device_index
    if _raw_stream is None:
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if _device_index is None:
        _device_index = torch.cuda.current_device()
    return ctypes.c_void_p(_raw_stream(_device_index))


class Library:
    """A loaded CUDA library with typed entry points."""

    def __init__(self, name: str):
        self.name = name
        self.lib = build.load(name)
        self._signatures = _parse_signatures(build.library_spec(name)[0])
        self._fns = {}
        self._last_error = None
        if hasattr(self.lib, "hos_last_error"):
            self._last_error = self.lib.hos_last_error
            self._last_error.restype = ctypes.c_char_p
            self._last_error.argtypes = []
        # kernels whose bounded waits run out say so in one word of pinned host memory (check_errors)
        for setter in _ERROR_WORD_SETTERS:
            f = getattr(self.lib, setter, None)
            if f is not None and torch.cuda.is_available():
                f.restype, f.argtypes = ctypes.c_int, [ctypes.c_void_p]
                f(ctypes.c_void_p(_error_word().data_ptr()))
        self._set_pdl = getattr(self.lib, "hos_set_pdl", None)
        if self._set_pdl is not None:
            self._set_pdl.restype, self._set_pdl.argtypes = None, [ctypes.c_int]
            self._set_pdl(1 if _launch_ahead else 0)
        _libraries.append(self)

    def fn(self, name: str, signature: Optional[str] = None):
        f = self._fns.get(name)
        if f is None:
            try:
                f = getattr(self.lib, name)
            except AttributeError as e:
                raise KernelError(f"library {self.name} has no function {name}") from e
            sig = signature or self._signatures[name]
            f.argtypes = [_CT[c] for c in sig]
            f.restype = ctypes.c_int
            self._fns[name] = f
        return f

    def call(self, name: str, *args, signature: Optional[str] = None) -> None:
        global launch_count
        launch_count += 1
        if _call_times is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = self.fn(name, signature)(*args)
            e1.record()
            _call_times.append((name, e0, e1))
        else:
            rc = self.fn(name, signature)(*args)
        if rc != 0:
            msg = self._last_error() if self._last_error else b""
            raise KernelError((msg or b"").decode(errors="replace") or f"{name} failed with code {rc}")


_libraries: List["Library"] = []
_call_times: Optional[list] = None


def time_calls(on: bool) -> None:
    """Measurement aid: while on, every call into a CUDA library is bracketed by two events on the launching
    stream (not inside a graph capture); `call_times()` adds them up by function."""
    global _call_times
    _call_times = [] if on else None


def call_times() -> dict:
    """{function: (calls, milliseconds in all)} of the calls made since time_calls(True); waits for them."""
    torch.cuda.synchronize()
    out = {}
    for name, e0, e1 in _call_times or []:
        n, ms = out.get(name, (0, 0.0))
        out[name] = (n + 1, ms + e0.elapsed_time(e1))
    if _call_times is not None:
        _call_times.clear()
    return out
_launch_ahead = False

_ERROR_WORD_SETTERS = ("hos_gemm_tc_set_error_word", "hos_attn_decode_set_error_word",
                       "hos_attn_prefill_tc_set_error_word")
GIVE_UP_CODES = {1: "the tcgen05 matrix product", 2: "the decode attention", 3: "the tcgen05 prompt attention"}
_error_word_tensor: Optional[torch.Tensor] = None
_after_give_up = []        # callables that put shared scratch state right after a kernel gave up


def _error_word() -> torch.Tensor:
    """One int32 in pinned host memory (the same address on the device): 0, or the code of the
    kernel whose bounded wait ran out last."""
    global _error_word_tensor
    if _error_word_tensor is None:
        _error_word_tensor = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _error_word_tensor


def on_give_up(fn) -> None:
    """Register what has to be put right when a kernel gave up (counters it left behind)."""
    _after_give_up.append(fn)


def check_errors() -> None:
    """Call after a synchronisation, before a step's result is used: raises KernelError if a kernel of
    the steps that are complete by now gave up a bounded wait (its results are then not to be trusted).
    Costs a read of host memory."""
    w = _error_word_tensor
    if w is None:
        return
    code = int(w[0])
    if code == 0:
        return
    w[0] = 0
    for fn in _after_give_up:
        fn()
    raise KernelError(f"{GIVE_UP_CODES.get(code, 'a kernel')} gave up a wait that should have ended (about a second); "
                      f"the results of the steps since the last check are not valid")


_room_left = False


def note_room_left(left: bool) -> None:
    """A launcher's word about the kernel it has just launched: it leaves at least half of the SMs free (the decode
    attention of one sequence does: 64 CTAs).  The launcher of the next kernel may then place that kernel beside it,
    ahead of its end (`take_room_left`); with the SMs full, kernels that wait on them cost more than they hide."""
    global _room_left
    _room_left = bool(left)


def take_room_left() -> bool:
    """What the last launcher said (see note_room_left); the word holds for one launch."""
    global _room_left
    left, _room_left = _room_left, False
    return left


def set_launch_ahead(on: bool) -> None:
    """Whether kernels are launched so that they may be set up while the kernel before them still
    runs (programmatic dependent launch).  It pays for steps of many tokens, whose kernels are
    launched one by one, and costs for single-token steps; the runner switches it per step."""
    global _launch_ahead
    if on == _launch_ahead:
        return
    _launch_ahead = on
    for lib in _libraries:
        if lib._set_pdl is not None:
            lib._set_pdl(1 if on else 0)


_sm_count: Optional[int] = None


def sm_count() -> int:
    """Streaming multiprocessors of the current device (asked once).  Without a device, as the
    host-side choices are also exercised where there is none, the B200's 148."""
    global _sm_count
    if _sm_count is None:
        _sm_count = (torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
                     if torch.cuda.is_available() else 148)
    return _sm_count


_core: Optional[Library] = None
launch_count = 0        # calls into the CUDA libraries so far (each launches one kernel or more)


def core() -> Library:
    global _core
    if _core is None:
        _core = Library("core")
    return _core


def _check(t: torch.Tensor, what: str, dtype=None, dim=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{what} must be on the GPU")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, found {t.dtype}")
    if dim is not None and t.dim() != dim:
        raise KernelError(f"{what} must have {dim} dimensions, found {t.dim()}")
    if not t.is_contiguous():
        raise KernelError(f"{what} must be contiguous")


@dataclass
class PagedKVArgs:
    """One call's view of the paged cache, as the kernels take it."""
    k_pages: torch.Tensor        # [n_pages, n_kv_heads, 64, head_dim]
    v_pages: torch.Tensor
    page_table: torch.Tensor     # int32 [n_slots, table_stride]
    ring_pages: int              # 0: all keys kept; > 0: ring of that many pages
    n_kv_heads: int
    head_dim: int
    v_head_dim: int = 0          # 0: values are as wide as keys

    @property
    def table_stride(self) -> int:
        return self.page_table.shape[1]

    @property
    def v_dim(self) -> int:
        return self.v_head_dim or self.head_dim


# ---- element-wise and norms ------------------------------------------------------------

def embed(tokens: torch.Tensor, table: torch.Tensor, scale: float, out: torch.Tensor) -> None:
    _check(tokens, "tokens", torch.int32, 1)
    _check(table, "embedding table", None, 2)
    _check(out, "embedding output", torch.float32, 2)
    n, d = out.shape
    if tokens.shape[0] != n or table.shape[1] != d:
        raise KernelError("embed: sizes of tokens, table and output disagree")
    core().call("hos_embed", _ptr(tokens), _ptr(table), dtype_code(table.dtype), float(scale),
                _ptr(out), n, d, _stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, add_one: bool, out: torch.Tensor) -> None:
    _check(x, "norm input", None, 2)
    _check(w, "norm weight", torch.float32, 1)
    _check(out, "norm output", None, 2)
    n, d = x.shape
    if out.shape != x.shape or w.shape[0] != d:
        raise KernelError("rmsnorm: sizes of input, weight and output disagree")
    core().call("hos_rmsnorm", _ptr(x), dtype_code(x.dtype), _ptr(w), float(eps), int(add_one),
                _ptr(out), dtype_code(out.dtype), n, d, _stream())


def norm_add_norm(y: torch.Tensor, w_post: torch.Tensor, eps_post: float, add_one_post: bool,
                  x: torch.Tensor, w_next: Optional[torch.Tensor] = None, eps_next: float = 0.0,
                  add_one_next: bool = False, h: Optional[torch.Tensor] = None) -> None:
    """x += RMSNorm(y; w_post); if h is given, h = RMSNorm(x; w_next).  y is [N, D], or
    [parts, N, D] float32 partial sums (of a matrix product that split K), added here."""
    _check(y, "norm input")
    _check(x, "residual stream", torch.float32, 2)
    _check(w_post, "norm weight", torch.float32, 1)
    n_parts = y.shape[0] if y.dim() == 3 else 1
    n, d = x.shape
    if tuple(y.shape[-2:]) != (n, d) or w_post.shape[0] != d or y.dim() not in (2, 3):
        raise KernelError("norm_add_norm: sizes disagree")
    if h is not None:
        _check(h, "next norm output", None, 2)
        _check(w_next, "next norm weight", torch.float32, 1)
        if h.shape != x.shape or w_next.shape[0] != d:
            raise KernelError("norm_add_norm: sizes of the next norm disagree")
    core().call("hos_norm_add_norm", _ptr(y), dtype_code(y.dtype), n_parts, _ptr(w_post), float(eps_post),
                int(add_one_post), _ptr(x), _ptr(w_next), float(eps_next), int(add_one_next),
                _ptr(h), dtype_code(h.dtype) if h is not None else 0, n, d, _stream())


def rope_table(token_pos: torch.Tensor, inv_freq: torch.Tensor) -> torch.Tensor:
    """float32 [N, len(inv_freq), 2]: (cos, sin) of position * inv_freq, taken in 32-bit."""
    _check(token_pos, "positions", torch.int32, 1)
    _check(inv_freq, "inverse frequencies", torch.float32, 1)
    out = torch.empty((token_pos.shape[0], inv_freq.shape[0], 2), dtype=torch.float32, device=token_pos.device)
    core().call("hos_rope_table", _ptr(token_pos), _ptr(inv_freq), _ptr(out), token_pos.shape[0], inv_freq.shape[0],
                _stream())
    return out


def residual_add(y: torch.Tensor, x: torch.Tensor) -> None:
    _check(y, "branch output")
    _check(x, "residual stream", torch.float32)
    if y.shape != x.shape:
        raise KernelError("residual_add: sizes disagree")
    core().call("hos_residual_add", _ptr(y), dtype_code(y.dtype), _ptr(x), x.numel(), _stream())


def rope_kv_write(qkv: torch.Tensor, n_heads: int, token_pos, token_seq, seq_slot, seq_len_after,
                  inv_freq: Optional[torch.Tensor], rotary_dim: int, style: int,
                  cache: Optional[PagedKVArgs], n_kv_heads: int, head_dim: int,
                  partials: Optional[torch.Tensor] = None) -> None:
    """Rotate the q and k heads of the fused projection rows `qkv` in place; if `cache` is
    given, store the rotated keys and the values at the tokens' places.  With `partials`
    ([parts, N, width] float32 partial sums of the projection) the rows are first formed from
    them and written to `qkv`."""
    _check(qkv, "qkv rows", None, 2)
    n, stride = qkv.shape
    if stride != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError("rope: row width does not match the head counts")
    if inv_freq is None:
        rotary_dim = 0
    else:
        _check(inv_freq, "inverse frequencies", torch.float32, 1)
        if inv_freq.shape[0] * 2 != rotary_dim:
            raise KernelError("rope: one inverse frequency per rotated pair is needed")
    if cache is not None and cache.k_pages.dtype != qkv.dtype:
        raise KernelError("rope: cache and activations differ in dtype")
    src, n_parts = qkv, 1
    if partials is not None:
        _check(partials, "partial sums", torch.float32, 3)
        if tuple(partials.shape[1:]) != (n, stride):
            raise KernelError("rope: partial sums and rows differ in size")
        src, n_parts = partials, partials.shape[0]
    core().call("hos_rope_kv_write", _ptr(src), dtype_code(src.dtype), n_parts, _ptr(qkv), dtype_code(qkv.dtype),
                stride, n_heads,
                _ptr(token_pos), _ptr(token_seq), _ptr(seq_slot), _ptr(seq_len_after),
                _ptr(inv_freq), rotary_dim, style,
                _ptr(cache.k_pages) if cache else None, _ptr(cache.v_pages) if cache else None,
                _ptr(cache.page_table) if cache else None, cache.table_stride if cache else 0,
                cache.ring_pages if cache else 0, n_kv_heads, head_dim, 1 if cache else 0, n,
                _stream())


def gated_act(gu: torch.Tensor, out: torch.Tensor, act: int) -> None:
    _check(gu, "gate|up rows", None, 2)
    _check(out, "activation output", gu.dtype, 2)
    n, f = out.shape
    if gu.shape != (n, 2 * f):
        raise KernelError("gated_act: sizes disagree")
    core().call("hos_gated_act", _ptr(gu), _ptr(out), dtype_code(gu.dtype), n, f, act, _stream())


def clamped_gated_act(gu: torch.Tensor, out: torch.Tensor, limit: float, alpha: float, shift: float) -> None:
    """out = g logistic(alpha g) (u + shift) with g = min(gate, limit), u = clamp(up, -limit, limit) (limit 0: no clamp);
    gu: float32 [N, 2F] gate then up; out: [N, F] in the products' type."""
    _check(gu, "gate|up rows", torch.float32, 2)
    n, f = out.shape
    if gu.shape != (n, 2 * f):
        raise KernelError("clamped_gated_act: sizes disagree")
    core().call("hos_clamped_gated_act", _ptr(gu), _ptr(out), dtype_code(out.dtype), n, f, float(limit), float(alpha),
                float(shift), _stream())


def gather_rows(x: torch.Tensor, idx: torch.Tensor, out: torch.Tensor) -> None:
    _check(x, "rows", torch.float32, 2)
    _check(idx, "row indices", torch.int32, 1)
    _check(out, "gathered rows", torch.float32, 2)
    if out.shape != (idx.shape[0], x.shape[1]):
        raise KernelError("gather_rows: sizes disagree")
    core().call("hos_gather_rows", _ptr(x), _ptr(idx), _ptr(out), idx.shape[0], x.shape[1], _stream())


# ---- matrix product (plain) --------------------------------------------------------------

def gemm_plain(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_NONE,
               cap: float = 0.0, act: int = 0) -> None:
    """out[M, N] = a[M, K] . w[N, K]^T with 32-bit accumulation on the CUDA cores.
    Gated epilogue: w has 2N rows (gate rows, then up rows), out = act(gate) * up."""
    _check(a, "left operand", None, 2)
    _check(w, "weight", None, 2)
    _check(out, "product", None, 2)
    m, k = a.shape
    n = out.shape[1]
    want_rows = 2 * n if epilogue == EPI_GATED else n
    if out.shape[0] != m or w.shape != (want_rows, k):
        raise KernelError(f"gemm: sizes disagree: a {tuple(a.shape)} w {tuple(w.shape)} out {tuple(out.shape)}")
    core().call("hos_gemm_plain", _ptr(a), dtype_code(a.dtype), _ptr(w), dtype_code(w.dtype),
                _ptr(out), dtype_code(out.dtype), m, n, k, k, k, n, epilogue, float(cap), act,
                _stream())


# ---- attention (plain) -------------------------------------------------------------------

def attn_plain(q: torch.Tensor, q_stride: int, out: torch.Tensor, token_pos, token_seq, n_tokens: int,
               n_heads: int, n_kv_heads: int, head_dim: int, scale: float, cap: float,
               window: Optional[int], *, k_rows=None, v_rows=None, kv_stride: int = 0,
               cu_seqlens=None, seq_slot=None, cache: Optional[PagedKVArgs] = None) -> None:
    """Either (k_rows, v_rows, cu_seqlens): keys of this step's own rows, sequences
    from position 0; or (cache, seq_slot): keys from the paged cache."""
    paged = cache is not None
    _check(out, "attention output", q.dtype, 2)
    core().call("hos_attn_plain", dtype_code(q.dtype), int(paged), _ptr(q), q_stride,
                _ptr(k_rows), _ptr(v_rows), kv_stride, _ptr(out), out.shape[1],
                _ptr(token_pos), _ptr(token_seq), _ptr(cu_seqlens), _ptr(seq_slot),
                _ptr(cache.k_pages) if paged else None, _ptr(cache.v_pages) if paged else None,
                _ptr(cache.page_table) if paged else None, cache.table_stride if paged else 0,
                cache.ring_pages if paged else 0, n_tokens, n_heads, n_kv_heads, head_dim,
                float(scale), float(cap), int(window) if window else 0, _stream())


# ---- sampling ----------------------------------------------------------------------------

_argmax_state = {}


def argmax(logits: torch.Tensor, out: torch.Tensor, rep_penalty: float = 1.0,
           recent: Optional[torch.Tensor] = None, recent_len: Optional[torch.Tensor] = None) -> None:
    """out[b] = the first maximum of row b.  With `recent` ([B, n] token ids, recent_len[b] of them
    valid) and a penalty other than 1 the sampler's repetition penalty is applied on the fly."""
    _check(logits, "logits", torch.float32, 2)
    _check(out, "tokens", torch.int32, 1)
    b, v = logits.shape
    stride = 0
    if recent is not None:
        _check(recent, "recent tokens", torch.int32, 2)
        _check(recent_len, "recent counts", torch.int32, 1)
        if recent.shape[0] != b or recent_len.shape[0] != b:
            raise KernelError("argmax: one row of recent tokens per row of logits is needed")
        stride = recent.shape[1]
    lib = core()
    f = lib.lib.hos_argmax_chunks
    f.restype, f.argtypes = ctypes.c_int, [ctypes.c_int]
    chunks = f(v)
    key = (logits.device, b, chunks)
    st = _argmax_state.get(key)
    if st is None:       # partial maxima and ids, and the tickets (zero between launches)
        st = _argmax_state[key] = (torch.empty(2 * b * chunks, dtype=torch.float32, device=logits.device),
                                   torch.zeros(b, dtype=torch.int32, device=logits.device))
    lib.call("hos_argmax", _ptr(logits), v, b, v, _ptr(out), _ptr(st[0]), _ptr(st[1]), _ptr(recent), stride,
             _ptr(recent_len), float(rep_penalty), _stream())


def sample(logits: torch.Tensor, uniforms: torch.Tensor, out: torch.Tensor, temp: float, top_k: int,
           top_p: float, rep_penalty: float = 1.0, recent: Optional[torch.Tensor] = None,
           recent_len: Optional[torch.Tensor] = None) -> None:
    _check(logits, "logits", torch.float32, 2)
    _check(uniforms, "uniform draws", torch.float32, 1)
    _check(out, "tokens", torch.int32, 1)
    b, v = logits.shape
    if recent is not None:
        _check(recent, "recent tokens", torch.int32, 2)
        _check(recent_len, "recent lengths", torch.int32, 1)
    core().call("hos_sample", _ptr(logits), v, b, v, _ptr(uniforms), _ptr(recent),
                recent.shape[1] if recent is not None else 0, _ptr(recent_len), float(temp),
                int(top_k), float(top_p), float(rep_penalty), _ptr(out), _stream())


# ---- the per-slot record (csrc/slot_state.cu) ----------------------------------------------
SLOT_WORDS, RECENT_MAX, MAX_STOPS = 8, 256, 16
SLOT_POS, SLOT_LAST, SLOT_FLAGS, SLOT_COUNT, SLOT_RNG_LO, SLOT_RNG_HI, SLOT_LIMIT = range(7)
BEGIN_ADVANCE, BEGIN_TOKEN_FROM_RECORD, BEGIN_UNIFORM, BEGIN_RECENT, BEGIN_SKIP_FINISHED = 1, 2, 4, 8, 16


def slot_begin(record, ring, slots, meta, b: int, flags: int, tokens, pos, after, seq, cu, uniforms=None,
               recent=None, recent_len=None) -> None:
    """The start of a single-token step of up to b rows (meta[0] of them live): row i belongs to slot
    slots[i]; positions come from the record and move on by one; the input token comes from the
    record (or stays the caller's); for sampling, the next draw of each sequence's generator and its
    recent tokens."""
    core().call("hos_slot_begin", _ptr(record), _ptr(ring), _ptr(slots), _ptr(meta), int(b), int(flags), _ptr(tokens),
                _ptr(pos), _ptr(after), _ptr(seq), _ptr(cu), _ptr(uniforms), _ptr(recent), _ptr(recent_len),
                recent.shape[1] if recent is not None else 0, _stream())


def slot_end(record, ring, slots, meta, b: int, sampled) -> None:
    """After sampling: the tokens go into the records (last token, recent tokens, count, finished)."""
    core().call("hos_slot_end", _ptr(record), _ptr(ring), _ptr(slots), _ptr(meta), int(b), _ptr(sampled), _stream())


def slot_set_pos(record, seq_slot, seq_len_after, cu_seqlens, n_seqs: int) -> None:
    core().call("hos_slot_set_pos", _ptr(record), _ptr(seq_slot), _ptr(seq_len_after), _ptr(cu_seqlens), int(n_seqs),
                _stream())


def slot_write(record, slots, values, word_mask: int) -> None:
    """record[slots[i]][w] = values[i][w] for the words w whose bit is set in word_mask."""
    _check(values, "record values", torch.int32, 2)
    core().call("hos_slot_write", _ptr(record), _ptr(slots), _ptr(values), int(word_mask), values.shape[0], _stream())


def decode_advance(tokens, token_pos, seq_len_after, token_seq, sampled) -> None:
    core().call("hos_decode_advance", _ptr(tokens), _ptr(token_pos), _ptr(seq_len_after), _ptr(token_seq),
                _ptr(sampled), tokens.shape[0], _stream())


# ---- the other kinds of block (csrc/embed_pair.cu, latent_attention.cu, wkv.cu, moe.cu) ------
_blocks: Optional[Library] = None


def blocks() -> Library:
    """Attention over a latent cache and the matrix-state recurrence with its token shift."""
    global _blocks
    if _blocks is None:
        _blocks = Library("blocks")
    return _blocks


_rows_lib: Optional[Library] = None
_experts: Optional[Library] = None
_gated_attn_lib: Optional[Library] = None


def rows_lib() -> Library:
    """The hashed token-pair embedding, the parallel block's add-and-norms, the norm without statistics."""
    global _rows_lib
    if _rows_lib is None:
        _rows_lib = Library("rows")
    return _rows_lib


def experts() -> Library:
    """The routed feed-forward."""
    global _experts
    if _experts is None:
        _experts = Library("experts")
    return _experts


def gated_attn_lib() -> Library:
    """Attention with a gate per head, a sink, chunks or a window, keys and values of unequal sizes."""
    global _gated_attn_lib
    if _gated_attn_lib is None:
        _gated_attn_lib = Library("gated_attn")
    return _gated_attn_lib


def embed_pair(step, prev_token: torch.Tensor, table: torch.Tensor, pair_table: torch.Tensor, buckets: int,
               mul_prev: int, mul_cur: int, out: torch.Tensor) -> None:
    """out[n] = table[token] + pair_table[(previous * mul_prev + token * mul_cur) % buckets], row `buckets`
    for a sequence's first token; the previous token of a continuing sequence's first row is
    prev_token[slot].  `step`: a StepInfo (device arrays)."""
    _check(out, "embedding output", torch.float32, 2)
    _check(prev_token, "previous tokens", torch.int32, 1)
    n, d = out.shape
    if table.dtype != pair_table.dtype or table.shape[1] != d or pair_table.shape != (buckets + 1, d):
        raise KernelError("embed_pair: the tables do not fit each other or the output")
    rows_lib().call("hos_embed_pair", _ptr(step.tokens), _ptr(step.token_pos), _ptr(step.token_seq),
                  _ptr(step.cu_seqlens), _ptr(step.seq_slot), _ptr(prev_token), _ptr(table), _ptr(pair_table),
                  dtype_code(table.dtype), int(buckets), int(mul_prev), int(mul_cur), _ptr(out), n, d, _stream())


def keep_last_token(step, prev_token: torch.Tensor) -> None:
    rows_lib().call("hos_keep_last_token", _ptr(step.tokens), _ptr(step.token_seq), _ptr(step.cu_seqlens),
                  _ptr(step.seq_slot), _ptr(prev_token), int(step.n_seqs), _stream())


def scaled_add_norms(a: Optional[torch.Tensor], f: Optional[torch.Tensor], mult: float, x: torch.Tensor,
                     w1: Optional[torch.Tensor] = None, eps1: float = 0.0, h1: Optional[torch.Tensor] = None,
                     w2: Optional[torch.Tensor] = None, eps2: float = 0.0, h2: Optional[torch.Tensor] = None) -> None:
    """x += mult * (a + f) (either may be absent); then h1 = RMSNorm(x; w1, eps1), h2 = RMSNorm(x; w2, eps2)
    for those that are given."""
    _check(x, "residual stream", torch.float32, 2)
    n, d = x.shape
    for t, what in ((a, "mixer output"), (f, "feed-forward output"), (h1, "first norm output"), (h2, "second norm output")):
        if t is not None:
            _check(t, what, None, 2)
            if t.shape != x.shape:
                raise KernelError(f"scaled_add_norms: {what} and the residual stream differ in size")
    if h1 is not None and h2 is not None and h1.dtype != h2.dtype:
        raise KernelError("scaled_add_norms: the two norm outputs differ in dtype")
    h = h1 if h1 is not None else h2
    rows_lib().call("hos_scaled_add_norms", _ptr(a), dtype_code(a.dtype) if a is not None else 0,
                  _ptr(f), dtype_code(f.dtype) if f is not None else 0, float(mult), _ptr(x),
                  _ptr(w1), float(eps1), _ptr(h1), _ptr(w2), float(eps2), _ptr(h2),
                  dtype_code(h.dtype) if h is not None else 0, n, d, _stream())


def latent_prep(proj: torch.Tensor, n_heads: int, dq: int, rank: int, rot: int, w_norm: Optional[torch.Tensor], eps: float,
                inv_freq: Optional[torch.Tensor], rot_dims: int, step, kc: Optional[torch.Tensor], q_lat: torch.Tensor,
                cache: Optional[PagedKVArgs]) -> None:
    """kc None: the rows hold queries only (a call that reads another call's cache): the queries' rotated parts are
    written and nothing is normed or stored."""
    _check(proj, "projection rows", None, 2)
    _check(q_lat, "latent queries", torch.float32, 3)
    n = proj.shape[0]
    if kc is None:
        if proj.shape[1] != n_heads * (dq + rot) or q_lat.shape != (n, n_heads, rank + rot):
            raise KernelError("latent_prep: sizes disagree")
        cache = None
    else:
        _check(kc, "latent rows", proj.dtype, 2)
        if proj.shape[1] != n_heads * (dq + rot) + rank + rot or kc.shape != (n, rank + rot) \
                or q_lat.shape != (n, n_heads, rank + rot) or w_norm is None:
            raise KernelError("latent_prep: sizes disagree")
    if cache is not None and (cache.k_pages.dtype != proj.dtype or cache.head_dim != rank + rot or cache.n_kv_heads != 1):
        raise KernelError("latent_prep: the cache does not fit the latent rows")
    blocks().call("hos_latent_prep", _ptr(proj), dtype_code(proj.dtype), proj.shape[1], n_heads, dq, rank, rot,
                  _ptr(w_norm), float(eps), _ptr(inv_freq), int(rot_dims) if inv_freq is not None else 0,
                  _ptr(step.token_pos), _ptr(step.token_seq), _ptr(step.seq_slot), _ptr(step.seq_len_after),
                  _ptr(kc), _ptr(q_lat), _ptr(cache.k_pages) if cache else None,
                  _ptr(cache.page_table) if cache else None, cache.table_stride if cache else 0,
                  cache.ring_pages if cache else 0, n, _stream())


def latent_attn(q_lat: torch.Tensor, kc: Optional[torch.Tensor], cache: Optional[PagedKVArgs], sink: Optional[torch.Tensor],
                o_lat: torch.Tensor, step, row0: int, rows: int, rank: int, scale: float, window: Optional[int],
                paged: bool, n_splits: int = 1, rows_per_block: int = 1, tensor_cores: bool = True) -> None:
    """Rows row0 .. row0+rows-1 of the step: keys from `kc` (the step's own rows; sequences from position 0)
    or from the paged cache.  `n_splits` > 1: every row's keys are cut into that many shares that run side by side
    and are merged (few rows: decoding); `rows_per_block` > 1: neighbouring rows share the keys they read (prompts)."""
    _check(q_lat, "latent queries", torch.float32, 3)
    _check(o_lat, "latent outputs", (cache.k_pages if paged else kc).dtype, 3)
    n, heads, d = q_lat.shape
    if o_lat.shape != (n, heads, rank):
        raise KernelError("latent_attn: sizes disagree")
    src = cache.k_pages if paged else kc
    part_acc = part_ml = None
    if n_splits > 1:
        part_acc = torch.empty((n, heads, n_splits, rank), dtype=torch.float32, device=q_lat.device)
        part_ml = torch.empty((n, heads, n_splits, 2), dtype=torch.float32, device=q_lat.device)
    blocks().call("hos_latent_attn", dtype_code(src.dtype), int(paged), _ptr(q_lat), _ptr(kc),
                  _ptr(cache.k_pages) if paged else None, _ptr(cache.page_table) if paged else None,
                  cache.table_stride if paged else 0, cache.ring_pages if paged else 0, _ptr(sink), _ptr(o_lat),
                  _ptr(part_acc), _ptr(part_ml), int(n_splits), int(rows_per_block),
                  _ptr(step.token_pos), _ptr(step.token_seq), _ptr(step.cu_seqlens), _ptr(step.seq_slot),
                  int(row0), int(rows), heads, rank, d, float(scale), int(window) if window else 0,
                  1 if tensor_cores else 0, _stream())


def heads_product(x: torch.Tensor, x_off: int, lda: int, a_head: int, w: torch.Tensor, out: torch.Tensor, out_off: int,
                  ldo: int, o_head: int, m: int) -> None:
    """out[r, h, :] = w[h] . x[r, h, :] for all heads in one launch; w: [heads, N, K]; x and out are given with
    an element offset, a row stride and a head stride (in elements)."""
    heads, n, k = w.shape
    blocks().call("hos_heads_product", ctypes.c_void_p(x.data_ptr() + x_off * x.element_size()), dtype_code(x.dtype),
                  _ptr(w), dtype_code(w.dtype), ctypes.c_void_p(out.data_ptr() + out_off * out.element_size()),
                  dtype_code(out.dtype), int(m), n, k, heads, int(lda), int(a_head), int(ldo), int(o_head), _stream())


def token_shift(h: torch.Tensor, kept: torch.Tensor, mu: torch.Tensor, step) -> List[torch.Tensor]:
    """The mixes h + (previous row - h) * mu[s], one [N, D] tensor per row of mu (each 16-byte aligned)."""
    _check(h, "rows", None, 2)
    _check(mu, "mixing weights", torch.float32, 2)
    n, d = h.shape
    if mu.shape[1] != d or kept.shape[1] != d:
        raise KernelError("token_shift: sizes disagree")
    plane = (n * d + 15) // 16 * 16
    out = torch.empty(mu.shape[0] * plane, dtype=h.dtype, device=h.device)
    blocks().call("hos_token_shift", _ptr(h), dtype_code(h.dtype), _ptr(kept), _ptr(mu), mu.shape[0],
                  _ptr(step.token_pos), _ptr(step.token_seq), _ptr(step.cu_seqlens), _ptr(step.seq_slot), _ptr(out),
                  plane, n, d, _stream())
    return [out[s * plane: s * plane + n * d].view(n, d) for s in range(mu.shape[0])]


def tanh_rows(x: torch.Tensor, out: torch.Tensor) -> None:
    _check(x, "rows", torch.float32)
    _check(out, "tanh output")
    blocks().call("hos_tanh_rows", _ptr(x), _ptr(out), dtype_code(out.dtype), x.numel(), _stream())


def wkv_scan(r, k, v, wx, g, w0, u, norm_w, eps: float, state: torch.Tensor, kept: torch.Tensor, h: torch.Tensor,
             step, out: torch.Tensor, heads: int, dim: int) -> None:
    for t in (r, k, v, wx, g):
        _check(t, "recurrence input", torch.float32, 2)
        if t.shape != (h.shape[0], heads * dim):
            raise KernelError("wkv_scan: sizes disagree")
    _check(state, "recurrent state", torch.float32, 4)
    _check(out, "recurrence output", h.dtype, 2)
    blocks().call("hos_wkv_scan", _ptr(r), _ptr(k), _ptr(v), _ptr(wx), _ptr(g), _ptr(w0), _ptr(u), _ptr(norm_w),
                  float(eps), _ptr(state), _ptr(kept), _ptr(h), dtype_code(h.dtype), h.shape[1], _ptr(step.token_pos),
                  _ptr(step.token_seq), _ptr(step.cu_seqlens), _ptr(step.seq_slot), _ptr(out), int(step.n_seqs),
                  heads, dim, _stream())


_moe_tile: Optional[int] = None


def moe_tile_rows() -> int:
    global _moe_tile
    if _moe_tile is None:
        f = experts().lib.hos_moe_tile_rows
        f.restype, f.argtypes = ctypes.c_int, []
        _moe_tile = int(f())
    return _moe_tile


MOE_SCORING = {"softmax": 0, "logistic": 1}


def moe_route(h, router, correction, token_seq, choice, weight, top: int, scoring: int = 0,
              renormalise: Optional[float] = None, weight_scale: float = 1.0) -> None:
    """renormalise (a number >= 0): the chosen scores are divided by their sum plus that number; weight_scale: a constant
    on every weight after that."""
    _check(h, "rows", None, 2)
    _check(router, "router", torch.float32, 2)
    n, d = h.shape
    # few rows and many router outputs: the outputs are cut over blocks, which leave their logits here for a second launch
    logits = torch.empty((n, router.shape[0]), dtype=torch.float32, device=h.device) if router.shape[0] > 8 and n < 2048 else None
    experts().call("hos_moe_route", _ptr(h), dtype_code(h.dtype), _ptr(router), _ptr(correction), _ptr(token_seq),
                  _ptr(choice), _ptr(weight), n, d, router.shape[0], int(top), int(scoring), _ptr(logits),
                  -1.0 if renormalise is None else float(renormalise), float(weight_scale), _stream())


def moe_align(choice, n_experts: int, listed, tile_expert) -> None:
    experts().call("hos_moe_align", _ptr(choice), choice.numel(), int(n_experts), _ptr(listed), listed.numel(),
                  _ptr(tile_expert), tile_expert.numel(), _stream())


def moe_gate_up(h, w, listed, tile_expert, y, top: int, limit: float, alpha: float, up_shift: float = 1.0,
                in_weight: Optional[torch.Tensor] = None) -> None:
    """in_weight ([pairs] float32): the pair's weight multiplies the expert's input (then `moe_down` takes none)."""
    _check(w, "expert gate/up weights", h.dtype, 3)
    experts().call("hos_moe_gate_up", _ptr(h), _ptr(w), dtype_code(h.dtype), _ptr(listed), _ptr(tile_expert), _ptr(y),
                  tile_expert.numel(), h.shape[1], w.shape[1] // 2, int(top), float(limit), float(alpha), float(up_shift),
                  _ptr(in_weight), _stream())


def moe_down(y, w, listed, tile_expert, weight, pair_out) -> None:
    _check(w, "expert down weights", y.dtype, 3)
    experts().call("hos_moe_down", _ptr(y), _ptr(w), dtype_code(y.dtype), _ptr(listed), _ptr(tile_expert), _ptr(weight),
                  _ptr(pair_out), tile_expert.numel(), w.shape[1], w.shape[2], _stream())


def moe_few(h, w_gate_up, w_down, choice, weight, y, pair_out, top: int, n_experts: int, limit: float, alpha: float,
            up_shift: float = 1.0, weight_on_input: bool = False) -> bool:
    """Both expert products for a handful of (row, choice) pairs, without lists or tiles (decoding at small batch):
    y [pairs, F] and pair_out [pairs, D] by pair id.  False: the sizes are not these kernels' and nothing ran."""
    lib = experts()
    global launch_count
    pairs, d, f = choice.numel(), h.shape[1], w_down.shape[2]

    def timed(name, *args):                 # these calls may answer 1 (not their sizes), so they do not go through call()
        if _call_times is None:
            return lib.fn(name)(*args)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = lib.fn(name)(*args)
        e1.record()
        if rc == 0:
            _call_times.append((name, e0, e1))
        return rc

    rc = timed("hos_moe_gate_up_few", _ptr(h), _ptr(w_gate_up), _ptr(choice), _ptr(y), pairs, d, f, int(top), int(n_experts),
               float(limit), float(alpha), float(up_shift), _ptr(weight) if weight_on_input else None, _stream())
    if rc == 1:
        return False
    if rc == 0:
        rc = timed("hos_moe_down_few", _ptr(y), _ptr(w_down), _ptr(choice), None if weight_on_input else _ptr(weight),
                   _ptr(pair_out), pairs, d, f, int(n_experts), _stream())
    launch_count += 2
    if rc != 0:
        msg = lib._last_error() if lib._last_error else b""
        raise KernelError((msg or b"").decode(errors="replace") or "the few-rows expert products failed")
    return True


def moe_combine(pair_out, choice, weight, h, out, top: int, n_experts: int, extra: Optional[torch.Tensor] = None) -> None:
    """extra ([N, D] of h's type): added to every row (an expert that all rows use)."""
    n, d = h.shape
    if extra is not None:
        _check(extra, "the shared expert's output", h.dtype, 2)
        if extra.shape != h.shape:
            raise KernelError("moe_combine: the shared expert's output and the rows differ in size")
    experts().call("hos_moe_combine", _ptr(pair_out), _ptr(choice), _ptr(weight), _ptr(h), dtype_code(h.dtype), _ptr(out),
                  n, d, int(top), int(n_experts), _ptr(extra), _stream())


def add_dyt(a: Optional[torch.Tensor], f: Optional[torch.Tensor], mult: float, x: torch.Tensor, alpha: float,
            w: Optional[torch.Tensor], b: Optional[torch.Tensor], h: Optional[torch.Tensor]) -> None:
    """x += mult * (a + f) (either may be absent; each [N, D] of any type or [parts, N, D] float32 partial sums); then,
    if h is given, h = tanh(alpha * x) * w + b (h may be x itself)."""
    _check(x, "residual stream", torch.float32, 2)
    n, d = x.shape
    parts = []
    for t, what in ((a, "mixer output"), (f, "feed-forward output")):
        if t is None:
            parts.append(0)
            continue
        _check(t, what)
        if t.dim() not in (2, 3) or tuple(t.shape[-2:]) != (n, d):
            raise KernelError(f"add_dyt: {what} and the residual stream differ in size")
        parts.append(t.shape[0] if t.dim() == 3 else 1)
    if h is not None:
        _check(h, "norm output", None, 2)
        _check(w, "norm weight", torch.float32, 1)
        _check(b, "norm bias", torch.float32, 1)
        if h.shape != x.shape or w.shape[0] != d or b.shape[0] != d:
            raise KernelError("add_dyt: sizes of the norm disagree")
    rows_lib().call("hos_add_dyt", _ptr(a), dtype_code(a.dtype) if a is not None else 0, parts[0],
                  _ptr(f), dtype_code(f.dtype) if f is not None else 0, parts[1], float(mult), _ptr(x), float(alpha),
                  _ptr(w), _ptr(b), _ptr(h), dtype_code(h.dtype) if h is not None else 0, n, d, _stream())


# ---- a norm after the sum, gated attention with a sink, matrix-state scans (csrc/postnorm.cu, gated_attention.cu,
# ---- state_scan.cu) ----------------------------------------------------------------------------------------------
_mixers: Optional[Library] = None
ACT_LOGISTIC, ACT_X_LOGISTIC = 0, 1


def mixers() -> Library:
    global _mixers
    if _mixers is None:
        _mixers = Library("mixers")
    return _mixers


def scale_add_norm(y: torch.Tensor, alpha: float, x: torch.Tensor, w: torch.Tensor, eps: float,
                   h: Optional[torch.Tensor] = None, w_next: Optional[torch.Tensor] = None, eps_next: float = 0.0) -> None:
    """x <- RMSNorm(alpha * x + y; w, eps).  y: [N, D], or [parts, N, D] float32 partial sums.  With `h`: h = the new x
    in h's type, or, with `w_next`, RMSNorm(x; w_next, eps_next)."""
    _check(x, "residual stream", torch.float32, 2)
    _check(y, "branch output")
    _check(w, "norm weight", torch.float32, 1)
    n, d = x.shape
    if y.dim() not in (2, 3) or tuple(y.shape[-2:]) != (n, d) or w.shape[0] != d:
        raise KernelError("scale_add_norm: sizes disagree")
    if h is not None:
        _check(h, "next input", None, 2)
        if h.shape != x.shape or (w_next is not None and w_next.shape[0] != d):
            raise KernelError("scale_add_norm: sizes of the next input disagree")
    mixers().call("hos_scale_add_norm", _ptr(y), dtype_code(y.dtype), y.shape[0] if y.dim() == 3 else 1, float(alpha),
                  _ptr(x), _ptr(w), float(eps), _ptr(h), dtype_code(h.dtype) if h is not None else 0, _ptr(w_next),
                  float(eps_next), n, d, _stream())


def cast_rows(x: torch.Tensor, h: torch.Tensor) -> None:
    _check(x, "rows", torch.float32)
    _check(h, "rows in the products' type")
    if h.shape != x.shape:
        raise KernelError("cast_rows: sizes disagree")
    mixers().call("hos_cast_rows", _ptr(x), _ptr(h), dtype_code(h.dtype), x.numel(), _stream())


def group_norm_gate(o: torch.Tensor, w: torch.Tensor, gate: torch.Tensor, gate_col: int, act: int, token_seq,
                    out: torch.Tensor, eps: float, groups: int, group_size: int) -> None:
    """out[n, g, :] = o[n, g, :] / rms * w * act(gate[n, gate_col + g * group_size + :]); w: [group_size] (shared by
    the groups) or [groups * group_size]."""
    _check(o, "mixer output", torch.float32, 2)
    _check(gate, "gate rows", torch.float32, 2)
    _check(w, "norm weight", torch.float32, 1)
    n = o.shape[0]
    if o.shape[1] != groups * group_size or out.shape != o.shape or w.shape[0] not in (group_size, groups * group_size) \
            or gate.shape[0] != n or gate_col + groups * group_size > gate.shape[1]:
        raise KernelError("group_norm_gate: sizes disagree")
    shared = 1 if (w.shape[0] == group_size and groups > 1) else 0
    mixers().call("hos_group_norm_gate", _ptr(o), _ptr(w), shared,
                  ctypes.c_void_p(gate.data_ptr() + gate_col * 4), gate.shape[1], int(act), _ptr(token_seq), _ptr(out),
                  dtype_code(out.dtype), float(eps), n, int(groups), int(group_size), _stream())


def qk_prep(proj: torch.Tensor, bias: Optional[torch.Tensor], q_norm: Optional[torch.Tensor], k_norm: Optional[torch.Tensor],
            eps: float, freq: Optional[torch.Tensor], rot_dims: int, magnitude: float, step, q_out: torch.Tensor,
            cache: PagedKVArgs, n_heads: int, n_kv: int, kd: int, vd: int, norm_whole: bool = False,
            v_first: Optional[torch.Tensor] = None, v_first_col: int = 0, v_mix: float = 0.0, q_maps: int = 1) -> None:
    """proj: float32 [N, >= H kd + G (kd + vd)] = [q | k | v | ...] (G = n_kv; 0: a call that stores nothing).  Adds the
    biases, norms and rotates the q and k heads, writes q_out float32 [N, H, kd] and stores k, v in the cache.
    norm_whole: one root mean square over all q heads and one over all k heads (weights [H kd], [G kd]).  v_first
    (float32 [N, ld], the values from column v_first_col on): v <- (1 - v_mix) v + v_mix v_first before the store.
    q_maps > 1: a head's kd numbers are q_maps queries, one per attention map over the same key row; q_out is then
    [N, H * q_maps, kd], every query a head of its own that is zero outside its part of the key row."""
    _check(proj, "projection rows", torch.float32, 2)
    _check(q_out, "queries", torch.float32, 3)
    n = proj.shape[0]
    if q_out.shape != (n, n_heads * q_maps, kd) or proj.shape[1] < n_heads * kd + n_kv * (kd + vd):
        raise KernelError("qk_prep: sizes disagree")
    if n_kv and (cache.head_dim != kd or cache.v_dim != vd or cache.n_kv_heads != n_kv):
        raise KernelError("qk_prep: the cache does not fit the keys and values")
    for wn, cols in ((q_norm, n_heads * kd), (k_norm, n_kv * kd)):
        if wn is not None and wn.shape[0] != (cols if norm_whole else kd):
            raise KernelError("qk_prep: a norm weight does not fit the heads")
    vf_ptr, vf_ld = None, 0
    if v_first is not None:
        _check(v_first, "the other layer's values", torch.float32, 2)
        if v_first.shape[0] != n or v_first_col + n_kv * vd > v_first.shape[1]:
            raise KernelError("qk_prep: the other layer's values do not fit this layer's")
        vf_ptr, vf_ld = ctypes.c_void_p(v_first.data_ptr() + 4 * v_first_col), v_first.shape[1]
    gated_attn_lib().call("hos_qk_prep", _ptr(proj), proj.shape[1], _ptr(bias), _ptr(q_norm), _ptr(k_norm), float(eps), _ptr(freq),
                  int(rot_dims), float(magnitude), _ptr(step.token_pos), _ptr(step.token_seq), _ptr(step.seq_slot),
                  _ptr(q_out), _ptr(cache.k_pages) if n_kv else None, _ptr(cache.v_pages) if n_kv else None,
                  dtype_code(cache.k_pages.dtype), _ptr(cache.page_table), cache.table_stride, cache.ring_pages, n,
                  int(n_heads), int(n_kv), int(kd), int(vd), 1 if norm_whole else 0, vf_ptr, vf_ld, float(v_mix),
                  int(q_maps), _stream())


def diff_combine(a: torch.Tensor, lam: float, mult: float, eps: float, gate: Optional[torch.Tensor], gate_col: int, step,
                 out: torch.Tensor, heads: int, vd: int) -> None:
    """a: float32 [N, heads * 2 * vd], the outputs of a head's two attention maps side by side; out [N, heads * vd] =
    rms_norm_per_head(a1 - lam a2) * mult * logistic(gate[:, gate_col + column])."""
    _check(a, "the maps' outputs", torch.float32, 2)
    n = a.shape[0]
    if a.shape[1] != heads * 2 * vd or out.shape != (n, heads * vd) or \
            (gate is not None and (gate.dtype != torch.float32 or gate_col + heads * vd > gate.shape[1])):
        raise KernelError("diff_combine: sizes disagree")
    gated_attn_lib().call("hos_diff_combine", _ptr(a), float(lam), float(mult), float(eps),
                          ctypes.c_void_p(gate.data_ptr() + gate_col * 4) if gate is not None else None,
                          gate.shape[1] if gate is not None else 0, _ptr(step.token_seq), _ptr(out), dtype_code(out.dtype),
                          n, int(heads), int(vd), _stream())


def gated_attn(q: torch.Tensor, cache: PagedKVArgs, sink: Optional[torch.Tensor], gate: Optional[torch.Tensor],
               gate_col: int, step, out: torch.Tensor, scale: float, chunk: int, window: int, n_splits: int = 1,
               keep_first: int = 0) -> None:
    """q: float32 [N, H, kd]; keys and values from the paged cache; out: [N, H * vd].  gate: float32 rows whose column
    gate_col + h is head h's gate logit."""
    _check(q, "queries", torch.float32, 3)
    n, heads, kd = q.shape
    vd = cache.v_dim
    if out.shape != (n, heads * vd) or kd != cache.head_dim:
        raise KernelError("gated_attn: sizes disagree")
    part_acc = part_ml = None
    if n_splits > 1:
        part_acc = torch.empty((n, heads, n_splits, vd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, heads, n_splits, 2), dtype=torch.float32, device=q.device)
    gated_attn_lib().call("hos_gated_attn", _ptr(q), _ptr(cache.k_pages), _ptr(cache.v_pages), dtype_code(cache.k_pages.dtype),
                  _ptr(cache.page_table), cache.table_stride, cache.ring_pages, _ptr(sink),
                  ctypes.c_void_p(gate.data_ptr() + gate_col * 4) if gate is not None else None,
                  gate.shape[1] if gate is not None else 0, _ptr(step.token_pos), _ptr(step.token_seq), _ptr(step.seq_slot),
                  _ptr(out), dtype_code(out.dtype), _ptr(part_acc), _ptr(part_ml), int(n_splits), n, heads,
                  cache.n_kv_heads, kd, vd, float(scale), int(chunk or 0), int(window or 0), int(keep_first or 0), _stream())


def gated_attn_mma(q: torch.Tensor, cache: PagedKVArgs, sink: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                   gate_col: int, step, out: torch.Tensor, scale: float, chunk: int, window: int, n_q_tiles: int,
                   keep_first: int = 0) -> bool:
    """The same attention on the tensor cores, for bfloat16 caches and rows that come many to a sequence.  False: the
    sizes are not that kernel's and nothing ran."""
    n, heads, kd = q.shape
    vd = cache.v_dim
    if out.dtype not in (torch.bfloat16, torch.float32) or cache.k_pages.dtype != torch.bfloat16 \
            or out.shape != (n, heads * vd):
        return False
    if kd not in (64, 128) or vd not in (64, 128) or q.data_ptr() % 16 or out.data_ptr() % 8:
        return False
    gated_attn_lib().call("hos_gated_attn_mma", _ptr(q), _ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(cache.page_table),
                  cache.table_stride, cache.ring_pages, _ptr(sink),
                  ctypes.c_void_p(gate.data_ptr() + gate_col * 4) if gate is not None else None,
                  gate.shape[1] if gate is not None else 0, _ptr(step.cu_seqlens), _ptr(step.token_pos),
                  _ptr(step.token_seq), _ptr(step.seq_slot), _ptr(out), 1 if out.dtype == torch.float32 else 0,
                  int(step.n_seqs), int(n_q_tiles), heads,
                  cache.n_kv_heads, kd, vd, float(scale), int(chunk or 0), int(window or 0), int(keep_first or 0), _stream())
    return True


def gated_attn_mma_decode(q: torch.Tensor, cache: PagedKVArgs, sink: Optional[torch.Tensor], gate: Optional[torch.Tensor],
                          gate_col: int, step, out: torch.Tensor, scale: float, chunk: int, window: int,
                          n_splits: int = 1, keep_first: int = 0) -> bool:
    """Single tokens on the tensor cores: the query heads that share a kv head are the rows of one tile.  False: the
    sizes are not that kernel's and nothing ran."""
    n, heads, kd = q.shape
    vd = cache.v_dim
    if out.dtype not in (torch.bfloat16, torch.float32) or cache.k_pages.dtype != torch.bfloat16 \
            or out.shape != (n, heads * vd):
        return False
    if kd not in (64, 128) or vd not in (64, 128) or heads // cache.n_kv_heads > 16 or q.data_ptr() % 16:
        return False
    part_acc = part_ml = None
    if n_splits > 1:
        part_acc = torch.empty((n, heads, n_splits, vd), dtype=torch.float32, device=q.device)
        part_ml = torch.empty((n, heads, n_splits, 2), dtype=torch.float32, device=q.device)
    gate_ptr = ctypes.c_void_p(gate.data_ptr() + gate_col * 4) if gate is not None else None
    gate_ld = gate.shape[1] if gate is not None else 0
    gated_attn_lib().call("hos_gated_attn_mma_decode", _ptr(q), _ptr(cache.k_pages), _ptr(cache.v_pages), _ptr(cache.page_table),
                  cache.table_stride, cache.ring_pages, _ptr(sink), gate_ptr, gate_ld, _ptr(step.token_pos),
                  _ptr(step.token_seq), _ptr(step.seq_slot), _ptr(out), 1 if out.dtype == torch.float32 else 0,
                  _ptr(part_acc), _ptr(part_ml), int(n_splits), n,
                  heads, cache.n_kv_heads, kd, vd, float(scale), int(chunk or 0), int(window or 0), int(keep_first or 0),
                  _stream())
    if n_splits > 1:
        gated_attn_lib().call("hos_attn_merge", _ptr(part_acc), _ptr(part_ml), int(n_splits), gate_ptr, gate_ld,
                      _ptr(step.token_seq), _ptr(out), dtype_code(out.dtype), n, heads, vd, _stream())
    return True


def state_scan(rows: torch.Tensor, q_col: int, k_col: int, v_col: int, silu_on_load: bool, g: torch.Tensor,
               per_token_g: bool, beta: Optional[torch.Tensor], state: torch.Tensor, step, out: torch.Tensor,
               heads: int, key_heads: int, dim: int, vdim: int, rot=None) -> None:
    """The matrix-state recurrence over the step's sequences.  rot = (freq, rot_dims, style, k_mult): q and k turn with
    their positions and the keys take a factor inside the walk (single-token steps), instead of by rotate_rows before.  rows: float32 [N, ld] holding q, k (key_heads x dim) and
    v (heads x vdim) from the given columns on.  g: [heads] constants, or [N, heads] per token; beta ([N, heads]): the
    delta rule, None: the plain decay rule.  state: [slots, heads, vdim, dim] float32.  out: float32 [N, heads * vdim]."""
    _check(rows, "recurrence inputs", torch.float32, 2)
    _check(state, "recurrent state", torch.float32, 4)
    _check(out, "recurrence output", torch.float32, 2)
    _check(g, "decays", torch.float32)
    n, ld = rows.shape
    if out.shape != (n, heads * vdim) or tuple(state.shape[1:]) != (heads, vdim, dim):
        raise KernelError("state_scan: sizes disagree")
    base = rows.data_ptr()
    if rot is not None and (silu_on_load or beta is not None or key_heads != heads):
        raise KernelError("state_scan: the rotation in the walk goes with the plain decay rule on rows as they are")
    in_walk = bool(silu_on_load) and beta is None and step.max_new == 1      # single tokens: no launch of its own for it
    if silu_on_load and not in_walk:        # q, k, v lie side by side from q_col on: x logistic(x) in place, once, before the walk
        if not (q_col < k_col < v_col) or v_col + heads * vdim - q_col != 2 * key_heads * dim + heads * vdim:
            raise KernelError("state_scan: q, k, v must lie side by side for the activation")
        mixers().call("hos_act_rows", ctypes.c_void_p(base + 4 * q_col), ld, 2 * key_heads * dim + heads * vdim, n, _stream())
    mixers().call("hos_state_scan", ctypes.c_void_p(base + 4 * q_col), ctypes.c_void_p(base + 4 * k_col),
                  ctypes.c_void_p(base + 4 * v_col), ld, 1 if in_walk else 0, _ptr(g), heads if per_token_g else 0,
                  _ptr(beta), heads if beta is not None else 0, _ptr(state), _ptr(step.token_pos), _ptr(step.token_seq),
                  _ptr(step.cu_seqlens), _ptr(step.seq_slot), _ptr(out), n, int(step.n_seqs), int(heads), int(key_heads),
                  int(dim), int(vdim), _ptr(rot[0]) if rot else None, int(rot[1]) if rot else 0, int(rot[2]) if rot else 0,
                  float(rot[3]) if rot else 1.0, _stream())


def act_rows(rows: torch.Tensor, cols: int) -> None:
    """x logistic(x), in place, on the first `cols` numbers of float32 rows."""
    _check(rows, "projection rows", torch.float32, 2)
    mixers().call("hos_act_rows", _ptr(rows), rows.shape[1], int(cols), rows.shape[0], _stream())


def rotate_rows(rows: torch.Tensor, q_heads: int, k_heads: int, dim: int, freq: Optional[torch.Tensor], rot_dims: int,
                style: int, step, k_mult: float = 1.0) -> None:
    """Rotary positions, in place, on the leading q_heads + k_heads heads of `dim` numbers of float32 rows (the first
    rot_dims numbers of each head, pairing `style`), then the key heads times k_mult."""
    _check(rows, "projection rows", torch.float32, 2)
    if rows.shape[1] < (q_heads + k_heads) * dim:
        raise KernelError("rotate_rows: sizes disagree")
    mixers().call("hos_rotate_rows", _ptr(rows), rows.shape[1], int(q_heads), int(k_heads), int(dim), int(rot_dims),
                  int(style), _ptr(freq), _ptr(step.token_pos), _ptr(step.token_seq), float(k_mult), rows.shape[0], _stream())


def conv_prep(raw: torch.Tensor, conv_w: torch.Tensor, conv_state: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
              step, act: torch.Tensor, beta: torch.Tensor, g: torch.Tensor, heads: int, key_heads: int, dim: int,
              vdim: int, keep_here: bool = False) -> None:
    """raw: float32 [N, ld] = [q | k | v | b | a | ...] projections; conv_w: [C, taps]; conv_state: [slots, taps - 1, C].
    keep_here (only where every sequence brings one token): the kept inputs move on in this launch, conv_keep is not needed."""
    _check(raw, "projection rows", torch.float32, 2)
    _check(conv_w, "convolution weights", torch.float32, 2)
    n, c = raw.shape[0], 2 * key_heads * dim + heads * vdim
    taps = conv_w.shape[1]
    if conv_w.shape[0] != c or raw.shape[1] < c + 2 * heads or act.shape != (n, c) \
            or tuple(conv_state.shape[1:]) != (max(taps - 1, 0), c):
        raise KernelError("conv_prep: sizes disagree")
    mixers().call("hos_conv_prep", _ptr(raw), raw.shape[1], _ptr(conv_w), taps, _ptr(conv_state), _ptr(a_log), _ptr(dt_bias),
                  _ptr(step.token_pos), _ptr(step.token_seq), _ptr(step.cu_seqlens), _ptr(step.seq_slot), _ptr(act),
                  _ptr(beta), _ptr(g), n, int(heads), int(key_heads), int(dim), int(vdim), 1 if keep_here else 0, _stream())


def conv_keep(raw: torch.Tensor, taps: int, conv_state: torch.Tensor, step, channels: int) -> None:
    mixers().call("hos_conv_keep", _ptr(raw), raw.shape[1], int(taps), _ptr(conv_state), _ptr(step.token_pos),
                  _ptr(step.token_seq), _ptr(step.cu_seqlens), _ptr(step.seq_slot), int(step.n_seqs), int(channels),
                  _stream())
