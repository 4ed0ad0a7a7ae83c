"""Token embedding scaled by a constant: x = E[token] * scale, the product taken in
32-bit (src/forward.rs:271-281; Gemma's scale is sqrt(width), src/model.rs:899),
and the head: logits = soft-cap(E_head . h) in float32 (src/forward.rs:429-435),
where E_head is `lm_head.weight` if the checkpoint has it and the embedding table
otherwise (src/model.rs:879-883)."""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from .. import ops
from ..registry import part_impl, register_part
from . import linear
from .base import CallStore, Part, StateNeed, StepInfo, WeightSpec


class ScaledEmbedding(Part):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.vocab = int(spec.params["vocab"])
        self.width = int(spec.params["width"])
        self.scale = float(spec.params.get("scale", 1.0))
        self.table: Optional[torch.Tensor] = None
        norm = spec.params.get("norm")       # the spec of a norm part: the rows are normed, in place, on their way out
        self.norm = part_impl("norm", norm.kind)(norm, rt) if norm is not None else None
        if self.norm is not None and not self.norm.graph_safe:
            self.graph_safe = False

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.spec.weights["table"], (self.vocab, self.width), "table", 0.02)] + \
               (self.norm.weight_specs() if self.norm is not None else [])

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = self._matrix(tensors[self.spec.weights["table"]])
        if self.norm is not None:
            self.norm.bind(tensors)

    def forward(self, tokens: torch.Tensor, step: StepInfo = None) -> torch.Tensor:
        x = torch.empty((tokens.shape[0], self.width), dtype=torch.float32, device=tokens.device)
        ops.embed(tokens, self.table, self.scale, x)
        if self.norm is not None:
            self.norm.forward(x, out=x)
        return x


class PairHashEmbedding(Part):
    """x = E[token] + B[row]: a second table indexed by a hash of the token and the one before it,
    row = (previous * mul_prev + token * mul_cur) mod buckets, and row `buckets` (the table's last) for a
    sequence's first token.  The sum is 32-bit.  The previous token of a sequence that is under way is
    per-sequence state (one int per slot), moved on after every step.  With `norm` (the spec of a norm part) the
    sum is normed, in place, before it becomes the residual stream."""
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.vocab, self.width = int(p["vocab"]), int(p["width"])
        self.buckets, self.mul_prev, self.mul_cur = int(p["buckets"]), int(p["mul_prev"]), int(p["mul_cur"])
        self.table: Optional[torch.Tensor] = None
        self.pair_table: Optional[torch.Tensor] = None
        norm = p.get("norm")
        self.norm = part_impl("norm", norm.kind)(norm, rt) if norm is not None else None
        if self.norm is not None and not self.norm.graph_safe:
            self.graph_safe = False

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        return [WeightSpec(w["table"], (self.vocab, self.width), "table", 0.02),
                WeightSpec(w["pair_table"], (self.buckets + 1, self.width), "table", 0.02)] + \
               (self.norm.weight_specs() if self.norm is not None else [])

    def state_needs(self) -> List[StateNeed]:
        return [StateNeed("prev_token", (), torch.int32)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = self._matrix(tensors[self.spec.weights["table"]])
        self.pair_table = self._matrix(tensors[self.spec.weights["pair_table"]])
        if self.table.dtype != self.pair_table.dtype:
            self.table, self.pair_table = self.table.float(), self.pair_table.float()
        if self.norm is not None:
            self.norm.bind(tensors)

    def forward(self, tokens: torch.Tensor, step: StepInfo, store: CallStore) -> torch.Tensor:
        x = torch.empty((tokens.shape[0], self.width), dtype=torch.float32, device=tokens.device)
        prev = store.state["prev_token"]
        ops.embed_pair(step, prev, self.table, self.pair_table, self.buckets, self.mul_prev, self.mul_cur, x)
        ops.keep_last_token(step, prev)
        if self.norm is not None:
            self.norm.forward(x, out=x)
        return x


class LinearHead(Part):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.vocab = int(spec.params["vocab"])
        self.width = int(spec.params["width"])
        self.softcap = float(spec.params.get("softcap") or 0.0)
        self.table: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        return [WeightSpec(w["table"], (self.vocab, self.width), "table", 0.02,
                           fallback=w.get("tied_to"))]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.table = self._matrix(tensors[self.spec.weights["table"]])

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        epi = ops.EPI_SOFTCAP if self.softcap > 0.0 else ops.EPI_NONE
        return linear.matmul(h, self.table, out_dtype=torch.float32, epilogue=epi, cap=self.softcap)


register_part("embedding", "scaled_embedding", ScaledEmbedding)
register_part("embedding", "pair_hash_embedding", PairHashEmbedding)
register_part("head", "linear_head", LinearHead)
