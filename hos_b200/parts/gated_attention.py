"""Softmax attention with grouped queries whose pieces are all options: keys of `dim` and values of `vdim`
numbers per head; biases on the q, k, v projections; an RMS norm of every query and key head (`qk_norm` true or
"head": a weight of `dim` numbers shared by the heads, before the rotation) or one over the whole query
projection and one over the whole key projection ("whole": weights of heads x dim numbers); a rotary position
part on the first numbers of a head; scores (q . k) * scale; a mask of chunks (position i sees j <= i with
floor(j / C) = floor(i / C), counted from the sequence's position 0) or of a window (the last W keys, and with
`keep_first` also the sequence's first keep_first keys), or plain causal; a sink (`sink` true: a learned number per
head whose exponential joins the softmax's denominator, without a key or a value; "zero": the constant 0, which
adds one to the denominator); a gate per head (the head's output times the logistic function of a projection of
the mixer's input); the output projection.

Values mixed across layers (`value_mix`): {"key": name, "role": "source"} leaves the layer's values, as projected,
in the step's shared store under that name; {"key": name, "role": "mixed"} blends its own values with them,
v <- (1 - m) v + m v_source with m the layer's scalar tensor `value_mix`, before they go to the cache.  Both are
values of the same token, so nothing but the blend is kept per sequence.

A call that reads another call's cache (`shares_kv`) has no key or value tensors: it projects its own queries
and gate and attends over the other call's keys and values as the cache holds them.

Every row stores its key and value first and then attends over the cache, whether its sequence starts in this
step or goes on: a position's result does not depend on how a prompt was cut.  The projections come out of
one product in 32-bit; norms, angles, scores, weights and the weighted sums are 32-bit; the cache holds keys
and values in the products' type.  In bfloat16, rows that come many to a sequence (more than FEW_TOKENS) run on
the tensor cores where the head sizes are that kernel's (64 or 128): queries rounded to bfloat16, scores
accumulated in 32-bit from exact products, the 32-bit weights fed as two bfloat16 terms.  Single tokens run there
too (up to 16 query heads to a kv head: they are the rows of one tile, the key tiles cut into shares where the
rows alone would leave the GPU idle); steps of 2 to FEW_TOKENS tokens and all other sizes keep the FMA kernel.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from .. import ops
from ..errors import KernelError, SpecError
from ..registry import part_impl, register_part
from . import linear
from .base import FEW_TOKENS, CallStore, KVNeed, Mixer, StepInfo, WeightSpec

SPLIT_MIN_KEYS = 256        # rows that see fewer keys are never cut into shares


class GatedSoftmaxAttention(Mixer):
    graph_safe = True
    use_tensor_cores = True      # tests switch it off to compare the two kernels on the same model

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.width = int(p["width"])
        self.n_heads, self.n_kv_heads = int(p["n_heads"]), int(p["n_kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.scale = float(p["scale"])
        self.eps = float(p.get("eps", 1e-6))
        self.chunk: Optional[int] = p.get("chunk")
        self.window: Optional[int] = p.get("window")
        self.has_bias, self.qk_norm = bool(p.get("bias", False)), bool(p.get("qk_norm", False))
        self.norm_whole = p.get("qk_norm") == "whole"
        self.has_sink, self.head_gate = bool(p.get("sink", False)), bool(p.get("head_gate", False))
        self.zero_sink = p.get("sink") == "zero"
        self.keep_first = int(p.get("keep_first") or 0)
        vm = p.get("value_mix")
        self.mix_key, self.mix_role = (str(vm["key"]), str(vm["role"])) if vm else (None, None)
        if self.mix_role not in (None, "source", "mixed") or (vm and bool(p.get("shares_kv", False))):
            raise SpecError("arch spec error: value_mix takes the role 'source' or 'mixed' on a layer with values of its own")
        if self.keep_first < 0 or (self.keep_first and not p.get("window")):
            raise SpecError("arch spec error: kept first keys go with a window")
        self.shares_kv = bool(p.get("shares_kv", False))
        if min(self.n_heads, self.n_kv_heads, self.dim, self.vdim) <= 0 or self.n_heads % self.n_kv_heads != 0:
            raise SpecError(f"arch spec error: {self.n_heads} heads of {self.dim}/{self.vdim} numbers over "
                            f"{self.n_kv_heads} kv heads")
        for name, v in (("chunk", self.chunk), ("window", self.window)):
            if v is not None and int(v) <= 0:
                raise SpecError(f"arch spec error: the attention's {name} must be positive")
        pos_spec = p.get("position")
        self.position = part_impl("position", pos_spec.kind)(pos_spec, rt) if pos_spec else None
        self.q_cols = self.n_heads * self.dim
        self.kv_cols = 0 if self.shares_kv else self.n_kv_heads * (self.dim + self.vdim)
        self.gate_col = self.q_cols + self.kv_cols

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        out = [WeightSpec(w["q"], (self.q_cols, self.width), "matrix", 0.02),
               WeightSpec(w["o"], (self.width, self.n_heads * self.vdim), "matrix", 0.02)]
        roles = [("q", self.q_cols)]
        if not self.shares_kv:
            out += [WeightSpec(w["k"], (self.n_kv_heads * self.dim, self.width), "matrix", 0.02),
                    WeightSpec(w["v"], (self.n_kv_heads * self.vdim, self.width), "matrix", 0.02)]
            roles += [("k", self.n_kv_heads * self.dim), ("v", self.n_kv_heads * self.vdim)]
        if self.has_bias:
            out += [WeightSpec(w[r + "_bias"], (n,), "vector", 0.1) for r, n in roles]
        if self.qk_norm:
            out += [WeightSpec(w[r + "_norm"], (n if self.norm_whole else self.dim,), "vector", 0.1)
                    for r, n in roles if r != "v"]
        if self.has_sink and not self.zero_sink:
            out.append(WeightSpec(w["sink"], (self.n_heads,), "vector", 0.5))
        if self.mix_role == "mixed":
            out.append(WeightSpec(w["value_mix"], (), "vector", 0.3))
        elif w.get("value_mix"):          # a format may write the scalar for layers that do not blend: read past it
            out.append(WeightSpec(w["value_mix"], (), "vector", 0.3, optional=True))
        if self.head_gate:
            out.append(WeightSpec(w["gate"], (self.n_heads, self.width), "matrix", 0.05))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = self.spec.weights
        roles = ["q"] if self.shares_kv else ["q", "k", "v"]
        mats = [self._matrix(tensors[w[r]]) for r in roles]
        if self.head_gate:
            mats.append(self._matrix(tensors[w["gate"]]))
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_in = torch.cat(mats, dim=0).contiguous()          # one product: q | k | v | gate logits
        self.bias = None
        if self.has_bias:
            parts = [self._vector32(tensors[w[r + "_bias"]]) for r in roles]
            if self.head_gate:
                parts.append(torch.zeros(self.n_heads, dtype=torch.float32, device=parts[0].device))
            self.bias = torch.cat(parts).contiguous()
        self.q_norm = self._vector32(tensors[w["q_norm"]]) if self.qk_norm else None
        self.k_norm = self._vector32(tensors[w["k_norm"]]) if self.qk_norm and not self.shares_kv else None
        self.sink = None
        if self.has_sink:
            self.sink = (torch.zeros(self.n_heads, dtype=torch.float32, device=self.w_in.device) if self.zero_sink
                         else self._vector32(tensors[w["sink"]]))
        self.v_mix = float(tensors[w["value_mix"]].float().reshape(-1)[0].item()) if self.mix_role == "mixed" else 0.0
        self.w_o = self._matrix(tensors[w["o"]])

    def kv_need(self) -> KVNeed:
        # every position is kept: rows attend over the cache in the step that stores them too, and a prompt may
        # be longer than any ring
        return KVNeed(self.n_kv_heads, self.dim, None, False, self.vdim if self.vdim != self.dim else None)

    def keys_seen(self, longest: int) -> int:
        n = longest
        if self.chunk:
            n = min(n, int(self.chunk))
        if self.window:
            n = min(n, int(self.window) + self.keep_first)
        return max(1, n)

    def n_splits(self, n_rows: int, longest: int) -> int:
        """Into how many shares a row's keys are cut: only where the rows alone leave most of the GPU idle."""
        keys = self.keys_seen(longest)
        vpl = max(1, (self.vdim + 31) // 32)
        together = next((c for c in (8, 4, 2) if (self.n_heads // self.n_kv_heads) % c == 0 and c * vpl <= 32), 1)
        warps = n_rows * self.n_heads // together      # query heads that share a kv head go to one warp
        room = 8 * ops.sm_count()
        if keys < SPLIT_MIN_KEYS or warps >= room:
            return 1
        return max(1, min(room // warps, keys // 64, 64))

    def forward(self, h, step: StepInfo, store: CallStore):
        return self._run(h, step, store, False)

    def forward_partial(self, h, step: StepInfo, store: CallStore):
        return self._run(h, step, store, True)

    def _run(self, h: torch.Tensor, step: StepInfo, store: CallStore, partial_ok: bool) -> torch.Tensor:
        cache = store.kv
        if cache is None:
            raise KernelError("attention needs a cache view")
        if store.owns_kv == self.shares_kv:
            raise KernelError("attention: the call's cache and the mixer's tensors do not fit (a mixer without key and "
                              "value tensors reads another call's cache, and only such a mixer does)")
        n = h.shape[0]
        proj = linear.matmul(h, self.w_in, out_dtype=torch.float32)
        q = torch.empty((n, self.n_heads, self.dim), dtype=torch.float32, device=h.device)
        freq, rot_dims, _ = self.position.kernel_args() if self.position else (None, 0, 0)
        v_col = self.q_cols + self.n_kv_heads * self.dim
        v_first = None
        if self.mix_role == "source":
            step.shared[self.mix_key] = (proj, v_col)          # the values as projected, for the layers that mix them in
        elif self.mix_role == "mixed":
            if self.mix_key not in step.shared:
                raise KernelError(f"attention: no layer of this step has left values under {self.mix_key!r}")
            v_first = step.shared[self.mix_key]
        ops.qk_prep(proj, self.bias, self.q_norm, self.k_norm, self.eps, freq, rot_dims,
                    getattr(self.position, "magnitude", 1.0), step, q, cache, self.n_heads,
                    0 if self.shares_kv else self.n_kv_heads, self.dim, self.vdim, self.norm_whole,
                    v_first[0] if v_first else None, v_first[1] if v_first else 0, self.v_mix)
        att = torch.empty((n, self.n_heads * self.vdim), dtype=h.dtype, device=h.device)
        gate = proj if self.head_gate else None
        if self.use_tensor_cores and h.dtype == torch.bfloat16 and step.max_new > FEW_TOKENS:
            # rows that come many to a sequence: 64 queries to a key tile on the tensor cores
            if step.cu_host:
                tiles = sum((step.cu_host[i + 1] - step.cu_host[i] + 63) // 64 for i in range(len(step.cu_host) - 1))
            else:
                tiles = (n + 63) // 64 + step.n_seqs
            if ops.gated_attn_mma(q, cache, self.sink, gate, self.gate_col, step, att, self.scale, self.chunk or 0,
                                  self.window or 0, tiles, self.keep_first):
                return linear.matmul_or_partials(att, self.w_o) if partial_ok else linear.matmul(att, self.w_o)
        if self.use_tensor_cores and h.dtype == torch.bfloat16 and step.max_new == 1:
            # single tokens: the query heads of a kv head are the rows of one tile; few rows: the key tiles in shares
            tiles = (self.keys_seen(step.max_len_after) + 63) // 64 + 1
            shares = max(1, min(tiles, 2 * ops.sm_count() // max(1, n * self.n_kv_heads), 32))
            if ops.gated_attn_mma_decode(q, cache, self.sink, gate, self.gate_col, step, att, self.scale, self.chunk or 0,
                                         self.window or 0, shares, self.keep_first):
                return linear.matmul_or_partials(att, self.w_o) if partial_ok else linear.matmul(att, self.w_o)
        ops.gated_attn(q, cache, self.sink, proj if self.head_gate else None, self.gate_col, step, att, self.scale,
                       self.chunk or 0, self.window or 0, self.n_splits(n, step.max_len_after), self.keep_first)
        return linear.matmul_or_partials(att, self.w_o) if partial_ok else linear.matmul(att, self.w_o)


register_part("mixer", "gated_softmax_attention", GatedSoftmaxAttention)
