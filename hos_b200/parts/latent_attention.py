"""Attention over a compressed (latent) cache.

Per position the layer keeps ONE row shared by all heads: the latent c (`kv_rank` numbers: the
first rows of the down projection, RMS-normed with a weight) and one rotated key part (`rot_dim`
numbers, not normed).  A head's key is [W_uk_h c | rotated part], its value W_uv_h c, its query
[dim unrotated | rot_dim rotated] numbers; the score is their dot product times `scale`.  The
mask is causal with an optional window of the last `window` keys; with `sink`, a learned number
per head joins the softmax's denominator as exp(sink_h) (no key, no value, unscaled).

Neither keys nor values are formed: the query absorbs W_uk (q'_h = W_uk_h^T q_h, `kv_rank`
numbers) and W_uv is applied to the weighted sum of latents, so the attention kernel reads
`kv_rank + rot_dim` numbers per key for all heads.  Everything between the projections (norm of
c, angles, scores, softmax, weighted sums) is 32-bit; with bfloat16 rows the two products run on the
tensor cores with every 32-bit operand as two bfloat16 terms (csrc/latent_attention.cu).

Cache: one keys-only group of row size kv_rank + rot_dim, a window ring if `window` is set.
A sequence that starts at position 0 attends over the step's own rows; one that goes on (by
one token or many) stores first and attends over the cache.

A call that reads another call's cache (`shares_kv`) has no down projection and no latent norm: it projects
and rotates its own queries and attends, with its own W_uk and W_uv, over the rows that the other call has
stored (this step's rows among them), every row over the cache.  The other call's kv_rank, rot_dim and
rotation are this one's.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from .. import ops
from ..errors import KernelError, SpecError
from ..registry import part_impl, register_part
from . import linear
from .base import CallStore, KVNeed, Mixer, StepInfo, WeightSpec


class LatentAttention(Mixer):
    graph_safe = True
    # bfloat16 rows whose sizes fit run the MMA kernel (the 32-bit query and weights as two bfloat16 terms each);
    # False keeps the FMA kernel everywhere (tests compare the two)
    use_tensor_cores = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.width = int(p["width"])
        self.n_heads = int(p["n_heads"])
        self.dim = int(p["dim"])                  # unrotated query/key numbers per head
        self.rot_dim = int(p["rot_dim"])          # rotated ones
        self.vdim = int(p["vdim"])
        self.rank = int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.window: Optional[int] = p.get("window")
        self.has_sink = bool(p.get("sink", False))
        self.shares_kv = bool(p.get("shares_kv", False))
        if self.shares_kv and self.window:
            raise SpecError("arch spec error: a latent attention that reads another call's cache keeps no window of its own")
        pos_spec = p.get("position")
        self.position = part_impl("position", pos_spec.kind)(pos_spec, rt) if pos_spec else None
        if min(self.n_heads, self.dim, self.rot_dim, self.vdim, self.rank) <= 0:
            raise SpecError("arch spec error: latent attention needs positive sizes")
        self.q_cols = self.n_heads * (self.dim + self.rot_dim)
        self.row = self.rank + self.rot_dim

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        out = [WeightSpec(w["q"], (self.q_cols, self.width), "matrix", 0.02)]
        if not self.shares_kv:
            out += [WeightSpec(w["dkv"], (self.row, self.width), "matrix", 0.02),
                    WeightSpec(w["dkv_norm"], (self.rank,), "vector", 0.1)]
        out += [WeightSpec(w["uk"], (self.n_heads * self.dim, self.rank), "matrix", 0.05),
               WeightSpec(w["uv"], (self.n_heads * self.vdim, self.rank), "matrix", 0.05),
               WeightSpec(w["o"], (self.width, self.n_heads * self.vdim), "matrix", 0.02)]
        if self.has_sink:
            out.append(WeightSpec(w["sink"], (self.n_heads,), "vector", 0.5))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = self.spec.weights
        q = self._matrix(tensors[w["q"]])
        if self.shares_kv:
            self.w_in, self.w_norm = q, None
        else:
            dkv = self._matrix(tensors[w["dkv"]])
            if q.dtype != dkv.dtype:
                q, dkv = q.float(), dkv.float()
            self.w_in = torch.cat([q, dkv], dim=0).contiguous()          # one product for q and the down projection
            self.w_norm = self._vector32(tensors[w["dkv_norm"]])
        uk = self._matrix(tensors[w["uk"]]).view(self.n_heads, self.dim, self.rank)
        self.w_uk_t = uk.transpose(1, 2).contiguous()                # [heads, rank, dim]: q'_h = W_uk_h^T q_h
        self.w_uv = self._matrix(tensors[w["uv"]]).view(self.n_heads, self.vdim, self.rank).contiguous()
        self.w_o = self._matrix(tensors[w["o"]])
        self.sink = self._vector32(tensors[w["sink"]]) if self.has_sink else None

    def kv_need(self) -> KVNeed:
        return KVNeed(1, self.row, self.window, keys_only=True)

    def plan(self, rows: int, step: StepInfo):
        """(shares of the keys, rows per block) for `rows` rows of a step.  Rows of one sequence that follow one another
        share the keys they read: four to a block (prompts, long pieces).  Few rows, or rows of different sequences
        (decoding), run one to a block, and their keys are cut into shares so that the GPU is filled about twice: at
        least two tiles of 32 keys per share, at most 32 shares."""
        if not step.single_token and rows >= 64:
            return 1, 4
        blocks = rows * ((self.n_heads + 7) // 8)
        sms = ops.sm_count()
        longest = step.max_len_after
        keys = min(int(self.window), longest) if self.window else longest
        return max(1, min(32, (keys + 63) // 64, (2 * sms + blocks - 1) // blocks)), 1

    def forward(self, h: torch.Tensor, step: StepInfo, store: CallStore) -> torch.Tensor:
        n = h.shape[0]
        cache = store.kv
        if cache is None or store.owns_kv == self.shares_kv:
            raise KernelError("latent attention: the call's cache and the mixer's tensors do not fit (a mixer without a "
                              "down projection reads another call's cache, and only such a mixer does)")
        H, R, D = self.n_heads, self.rank, self.row
        proj = linear.matmul(h, self.w_in)
        kc = None if self.shares_kv else torch.empty((n, D), dtype=h.dtype, device=h.device)
        q_lat = torch.empty((n, H, D), dtype=torch.float32, device=h.device)
        inv_freq, rot_dims, style = self.position.kernel_args() if self.position else (None, 0, 1)
        if inv_freq is not None and style != ops.ROPE_STYLES["interleaved"]:
            raise KernelError("latent attention rotates neighbouring pairs only")
        ops.latent_prep(proj, H, self.dim, R, self.rot_dim, self.w_norm, self.eps, inv_freq, rot_dims, step, kc, q_lat, cache)
        # q'_h = W_uk_h^T q_h into the first `rank` numbers of every head's latent query
        ops.heads_product(proj, 0, proj.shape[1], self.dim + self.rot_dim, self.w_uk_t, q_lat, 0, H * D, D, n)
        o_lat = torch.empty((n, H, R), dtype=h.dtype, device=h.device)      # what the value expansion reads
        nf = 0 if self.shares_kv else (n if step.from_zero else step.fresh_tokens)
        if nf > 0:
            shares, per_block = self.plan(nf, step)
            ops.latent_attn(q_lat, kc, None, self.sink, o_lat, step, 0, nf, R, self.scale, self.window, paged=False,
                            n_splits=shares, rows_per_block=per_block, tensor_cores=self.use_tensor_cores)
        if nf < n:
            if cache.ring_pages > 0 and not step.replayed:
                room = cache.ring_pages * ops.PAGE_TOKENS - int(self.window) + 1
                news = [step.cu_host[i + 1] - step.cu_host[i] for i in range(step.fresh_seqs, step.n_seqs)] if step.cu_host else []
                if news and max(news) > room:
                    raise KernelError(f"a step that continues sequences brings {max(news)} tokens to a layer that keeps "
                                      f"a window of {self.window} keys in a ring of {cache.ring_pages * ops.PAGE_TOKENS}: "
                                      f"at most {room} fit")
            rows = n - nf
            shares, per_block = self.plan(rows, step)
            ops.latent_attn(q_lat, None, cache, self.sink, o_lat, step, nf, rows, R, self.scale, self.window, paged=True,
                            n_splits=shares, rows_per_block=per_block, tensor_cores=self.use_tensor_cores)
        att = torch.empty((n, H * self.vdim), dtype=h.dtype, device=h.device)
        ops.heads_product(o_lat, 0, H * R, R, self.w_uv, att, 0, H * self.vdim, self.vdim, n)
        return linear.matmul(att, self.w_o)


register_part("mixer", "latent_attention", LatentAttention)
