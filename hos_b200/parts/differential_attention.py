"""Differential softmax attention with grouped queries: every head runs TWO attention maps over the same values
and outputs their difference.

q = W_q h has heads x 2 x dim rows and k = W_k h kv_heads x 2 x dim, head by head as [map 1 | map 2]; v = W_v h has
kv_heads x vdim (query head h reads key/value head h // (heads / kv_heads)); optional biases on all three.  No
position encoding.  Map m of a head is softmax((q_m . k_m) * scale) over the keys the mask lets through (causal; with
`window` the last W keys; with `keep_first` also the sequence's first keys) times v.  With
lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff (four vectors of dim numbers and the constant `diff`: one number for the
layer, taken once when the tensors are bound), a head's output is rms_norm(a1 - lambda a2) (per head, no weight) times
(1 - diff), times, with `gate`, logistic(W_g h) column by column; then the output projection.

How it runs: a key head's row in the cache is [k of map 1 | k of map 2], 2 x dim numbers, and the values are kept
once.  Every query is written as a head of its own over that row, zero outside its map's half, so that
(q_1, 0) . (k_1, k_2) = q_1 . k_1 exactly: the library's attention kernels for grouped queries (the FMA kernel, the
tensor-core kernels for prompts and for single tokens) then serve 2 x heads query heads over kv_heads key rows and
read every key and value once for both maps.  They hand back the maps' outputs in 32-bit; one more kernel takes the
difference, the norm, the constant and the gate.  Projections come out of one product in 32-bit; biases, scores,
weights, weighted sums, the difference, the norm and the gate are 32-bit; the cache holds keys and values in the
products' type.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from .. import ops
from ..errors import KernelError, SpecError
from ..registry import register_part
from . import linear
from .base import FEW_TOKENS, CallStore, KVNeed, Mixer, StepInfo, WeightSpec
from .gated_attention import SPLIT_MIN_KEYS

MAPS = 2


class DifferentialAttention(Mixer):
    graph_safe = True
    use_tensor_cores = True      # tests switch it off to compare the kernels on the same model

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.width = int(p["width"])
        self.n_heads, self.n_kv_heads = int(p["n_heads"]), int(p["n_kv_heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.scale, self.eps, self.diff = float(p["scale"]), float(p["eps"]), float(p["diff"])
        self.window: Optional[int] = p.get("window")
        self.keep_first = int(p.get("keep_first") or 0)
        self.has_bias, self.has_gate = bool(p.get("bias", False)), bool(p.get("gate", False))
        if min(self.width, self.n_heads, self.n_kv_heads, self.dim, self.vdim) <= 0 or self.n_heads % self.n_kv_heads != 0:
            raise SpecError(f"arch spec error: {self.n_heads} heads of 2 x {self.dim} / {self.vdim} numbers over "
                            f"{self.n_kv_heads} kv heads")
        if (self.window is not None and int(self.window) <= 0) or self.keep_first < 0 or (self.keep_first and not self.window):
            raise SpecError("arch spec error: the attention's window must be positive, and kept first keys go with a window")
        self.kd = MAPS * self.dim                                  # a key row: both maps' keys side by side
        self.q_cols = self.n_heads * self.kd
        self.kv_cols = self.n_kv_heads * (self.kd + self.vdim)
        self.gate_col = self.q_cols + self.kv_cols
        self.lam = 0.0

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        roles = [("q", self.q_cols), ("k", self.n_kv_heads * self.kd), ("v", self.n_kv_heads * self.vdim)]
        out = [WeightSpec(w[r], (n, self.width), "matrix", 0.02) for r, n in roles]
        if self.has_bias:
            out += [WeightSpec(w[r + "_bias"], (n,), "vector", 0.1) for r, n in roles]
        out += [WeightSpec(w[r], (self.dim,), "vector", 0.1) for r in ("lq1", "lk1", "lq2", "lk2")]
        if self.has_gate:
            out.append(WeightSpec(w["gate"], (self.n_heads * self.vdim, self.width), "matrix", 0.05))
        out.append(WeightSpec(w["o"], (self.width, self.n_heads * self.vdim), "matrix", 0.02))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = self.spec.weights
        roles = ["q", "k", "v"] + (["gate"] if self.has_gate else [])
        mats = [self._matrix(tensors[w[r]]) for r in roles]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_in = torch.cat(mats, dim=0).contiguous()          # one product: q | k | v | gate logits
        self.bias = None
        if self.has_bias:
            parts = [self._vector32(tensors[w[r + "_bias"]]) for r in ("q", "k", "v")]
            if self.has_gate:
                parts.append(torch.zeros(self.n_heads * self.vdim, dtype=torch.float32, device=parts[0].device))
            self.bias = torch.cat(parts).contiguous()
        lq1, lk1, lq2, lk2 = (self._vector32(tensors[w[r]]) for r in ("lq1", "lk1", "lq2", "lk2"))
        # one number for the layer, in 32-bit, read once, here
        self.lam = float((torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + self.diff).item())
        self.w_o = self._matrix(tensors[w["o"]])

    def kv_need(self) -> KVNeed:
        # every position is kept: rows attend over the cache in the step that stores them too, and a prompt may
        # be longer than any ring
        return KVNeed(self.n_kv_heads, self.kd, None, False, self.vdim if self.vdim != self.kd else None)

    def keys_seen(self, longest: int) -> int:
        n = longest
        if self.window:
            n = min(n, int(self.window) + self.keep_first)
        return max(1, n)

    def n_splits(self, n_rows: int, longest: int) -> int:
        """Into how many shares the FMA kernel cuts a row's keys: only where the rows alone leave most of the GPU idle."""
        keys = self.keys_seen(longest)
        vpl = max(1, (self.vdim + 31) // 32)
        per_kv = MAPS * self.n_heads // self.n_kv_heads
        together = next((c for c in (8, 4, 2) if per_kv % c == 0 and c * vpl <= 32), 1)
        warps = n_rows * MAPS * self.n_heads // together
        room = 8 * ops.sm_count()
        if keys < SPLIT_MIN_KEYS or warps >= room:
            return 1
        return max(1, min(room // warps, keys // 64, 64))

    def forward(self, h, step: StepInfo, store: CallStore):
        return self._run(h, step, store, False)

    def forward_partial(self, h, step: StepInfo, store: CallStore):
        return self._run(h, step, store, True)

    def _maps(self, q, cache, step, maps_out, n, bf16: bool) -> None:
        """The 2 x heads attention maps of the step's rows, 32-bit, into maps_out [N, heads * 2 * vdim]."""
        heads = MAPS * self.n_heads
        if self.use_tensor_cores and bf16 and step.max_new > FEW_TOKENS:
            if step.cu_host:
                tiles = sum((step.cu_host[i + 1] - step.cu_host[i] + 63) // 64 for i in range(len(step.cu_host) - 1))
            else:
                tiles = (n + 63) // 64 + step.n_seqs
            if ops.gated_attn_mma(q, cache, None, None, 0, step, maps_out, self.scale, 0, self.window or 0, tiles,
                                  self.keep_first):
                return
        if self.use_tensor_cores and bf16 and step.max_new == 1:
            tiles = (self.keys_seen(step.max_len_after) + 63) // 64 + 1
            shares = max(1, min(tiles, 2 * ops.sm_count() // max(1, n * self.n_kv_heads), 32))
            if ops.gated_attn_mma_decode(q, cache, None, None, 0, step, maps_out, self.scale, 0, self.window or 0, shares,
                                         self.keep_first):
                return
        ops.gated_attn(q, cache, None, None, 0, step, maps_out, self.scale, 0, self.window or 0,
                       self.n_splits(n, step.max_len_after), self.keep_first)

    def _run(self, h: torch.Tensor, step: StepInfo, store: CallStore, partial_ok: bool) -> torch.Tensor:
        cache = store.kv
        if cache is None or not store.owns_kv:
            raise KernelError("differential attention needs a cache of its own")
        n = h.shape[0]
        proj = linear.matmul(h, self.w_in, out_dtype=torch.float32)
        q = torch.empty((n, MAPS * self.n_heads, self.kd), dtype=torch.float32, device=h.device)
        ops.qk_prep(proj, self.bias, None, None, self.eps, None, 0, 1.0, step, q, cache, self.n_heads, self.n_kv_heads,
                    self.kd, self.vdim, q_maps=MAPS)
        maps_out = torch.empty((n, self.n_heads * MAPS * self.vdim), dtype=torch.float32, device=h.device)
        self._maps(q, cache, step, maps_out, n, h.dtype == torch.bfloat16)
        att = torch.empty((n, self.n_heads * self.vdim), dtype=h.dtype, device=h.device)
        ops.diff_combine(maps_out, self.lam, 1.0 - self.diff, self.eps, proj if self.has_gate else None, self.gate_col, step,
                         att, self.n_heads, self.vdim)
        return linear.matmul_or_partials(att, self.w_o) if partial_ok else linear.matmul(att, self.w_o)


register_part("mixer", "differential_attention", DifferentialAttention)
