"""A routed feed-forward (mixture of experts).

Router logits z = W_router h in 32-bit; scores s = softmax(z) over all router outputs (`scoring`
"softmax") or the logistic function of each logit alone ("logistic").  The `top` outputs with the largest
s + correction are chosen (the correction, if the model has one, only steers the choice); each chosen
expert is weighted by its plain score s, not renormalised: its output is (`weight_on` "output"), or its
input, expert(s h) ("input").  With `renormalise` (a number >= 0) the chosen scores are first divided by their sum
plus that number, and `weight_scale` is a constant on every weight after that.  The last `identity` router outputs are experts without tensors whose
output is the row itself.
Expert: g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), y = g * sigmoid(alpha * g) * (u + up_shift),
output W_down y; no biases (`up_shift` 1 and `alpha` 1.702 by default; 0 and 1 make the plain gated form
silu(g) * u).  `shared`, the spec of a feed-forward part, is an expert that every row uses; its output is
added.  The step stays on the device: rows are listed expert by expert and the experts' products run as
tiles of one launch each (csrc/moe.cu); the output is the 32-bit sum.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from .. import ops
from ..errors import SpecError
from ..registry import part_impl, register_part
from .base import FeedForward, StepInfo, WeightSpec


FEW_PAIRS = 32          # up to this many (row, choice) pairs take the kernels without lists and tiles


class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.width, self.inner = int(p["width"]), int(p["inner"])
        self.n_experts, self.n_identity, self.top = int(p["experts"]), int(p.get("identity", 0)), int(p["top"])
        self.limit = float(p.get("limit") or 0.0)
        self.alpha = float(p.get("alpha", 1.702))
        self.has_correction = bool(p.get("correction", False))
        self.up_shift = float(p.get("up_shift", 1.0))
        scoring, weight_on = p.get("scoring", "softmax"), p.get("weight_on", "output")
        if scoring not in ops.MOE_SCORING or weight_on not in ("output", "input"):
            raise SpecError(f"arch spec error: routed experts with scoring {scoring!r} and the weight on {weight_on!r}")
        self.scoring, self.weight_on_input = ops.MOE_SCORING[scoring], weight_on == "input"
        self.renormalise = p.get("renormalise")            # None, or the number added to the chosen scores' sum
        self.weight_scale = float(p.get("weight_scale", 1.0))
        if self.renormalise is not None and float(self.renormalise) < 0.0:
            raise SpecError("arch spec error: the number added to the chosen scores' sum cannot be negative")
        shared = p.get("shared")
        self.shared = part_impl("feed_forward", shared.kind)(shared, rt) if shared is not None else None
        if self.n_experts < 0 or self.n_identity < 0 or not 0 < self.top <= self.n_experts + self.n_identity:
            raise SpecError(f"arch spec error: {self.top} of {self.n_experts} + {self.n_identity} experts cannot be chosen")

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        out = [WeightSpec(w["router"], (self.n_experts + self.n_identity, self.width), "matrix", 0.3)]
        if self.has_correction:
            out.append(WeightSpec(w["correction"], (self.n_experts + self.n_identity,), "vector", 0.05))
        for e in range(self.n_experts):
            base = w["expert"].format(e)
            out += [WeightSpec(base + w["gate"], (self.inner, self.width), "matrix", 0.05),
                    WeightSpec(base + w["up"], (self.inner, self.width), "matrix", 0.05),
                    WeightSpec(base + w["down"], (self.width, self.inner), "matrix", 0.05)]
        if self.shared is not None:
            out += self.shared.weight_specs()
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = self.spec.weights
        if self.shared is not None:
            self.shared.bind(tensors)
        self.router = tensors[w["router"]].to(torch.float32).contiguous()
        self.correction = self._vector32(tensors[w["correction"]]) if self.has_correction else None
        dev = self.router.device
        dt = torch.float32 if self.rt.is_fp32 else torch.bfloat16
        self.w_gate_up = torch.empty((max(1, self.n_experts), 2 * self.inner, self.width), dtype=dt, device=dev)
        self.w_down = torch.empty((max(1, self.n_experts), self.width, self.inner), dtype=dt, device=dev)
        for e in range(self.n_experts):
            base = w["expert"].format(e)
            self.w_gate_up[e, : self.inner] = tensors[base + w["gate"]]
            self.w_gate_up[e, self.inner:] = tensors[base + w["up"]]
            self.w_down[e] = tensors[base + w["down"]]

    def forward(self, h: torch.Tensor, step: StepInfo = None) -> torch.Tensor:
        n, dev = h.shape[0], h.device
        top, tile = self.top, ops.moe_tile_rows()
        pairs = n * top
        choice = torch.empty(pairs, dtype=torch.int32, device=dev)
        weight = torch.empty(pairs, dtype=torch.float32, device=dev)
        ops.moe_route(h, self.router, self.correction, step.token_seq, choice, weight, top, self.scoring,
                      self.renormalise, self.weight_scale)
        out = torch.empty((n, self.width), dtype=torch.float32, device=dev)
        pair_out = None
        if self.n_experts > 0:
            pair_out = torch.empty((pairs, self.width), dtype=torch.float32, device=dev)
            done = False
            if pairs <= FEW_PAIRS and h.dtype == torch.bfloat16:
                # a handful of pairs: a block per pair and slice of the features, no lists, no tiles
                y = torch.empty((pairs, self.inner), dtype=h.dtype, device=dev)
                done = ops.moe_few(h, self.w_gate_up, self.w_down, choice, weight, y, pair_out, top, self.n_experts,
                                   self.limit, self.alpha, self.up_shift, self.weight_on_input)
            if not done:
                # every expert's list is padded to whole tiles: at most this many tiles whatever the router chooses
                max_tiles = min(pairs, self.n_experts) + pairs // tile
                listed = torch.empty(max_tiles * tile, dtype=torch.int32, device=dev)
                tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=dev)
                ops.moe_align(choice, self.n_experts, listed, tile_expert)
                y = torch.empty((max_tiles * tile, self.inner), dtype=h.dtype, device=dev)
                ops.moe_gate_up(h, self.w_gate_up, listed, tile_expert, y, top, self.limit, self.alpha, self.up_shift,
                                weight if self.weight_on_input else None)
                ops.moe_down(y, self.w_down, listed, tile_expert, None if self.weight_on_input else weight, pair_out)
        extra = self.shared.forward(h, step) if self.shared is not None else None
        ops.moe_combine(pair_out, choice, weight, h, out, top, self.n_experts, extra)
        return out


register_part("feed_forward", "routed_experts", RoutedExperts)
