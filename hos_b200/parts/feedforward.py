"""Gated feed-forward: down(act(gate(h)) * up(h)) (src/forward.rs:384-398), with the
activation as a parameter ("gelu_tanh" is Gemma's GeGLU, src/forward.rs:186-189;
"silu" is the reference's other branch, :393).  Gate and up are one product whose
epilogue applies the activation and the product, so the 2*inner-wide intermediate
is never written.

"clamped_swish" is the form g = min(gate(h), limit), u = clamp(up(h), -limit, limit), down(g logistic(alpha g)
(u + up_shift)) with `limit`, `alpha` (1.702 by default) and `up_shift` (1 by default) as parameters: the form the
routed experts' kernels know, for a dense layer.  With the usual constants (alpha 1.702, up_shift 1) it is the third
activation of the products' gated epilogues, the limit a parameter; with other constants gate and up come out of one
product as 32-bit rows and a kernel of its own takes the clamp, the activation and the product.  Both ways the clamp,
the activation and the product are 32-bit and rounded once."""
from __future__ import annotations

from typing import List, Mapping

import torch

from .. import ops
from ..errors import SpecError
from ..registry import register_part
from . import linear
from .base import FeedForward, StepInfo, WeightSpec


class GatedMLP(FeedForward):
    graph_safe = True
    fused = True          # tests switch it off to compare the clamped form's two ways

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.width = int(spec.params["width"])
        self.inner = int(spec.params["inner"])
        act = spec.params.get("activation", "gelu_tanh")
        self.clamped = act == "clamped_swish"
        if not self.clamped and act not in ops.ACTIVATIONS:
            raise SpecError(f"arch spec error: unknown activation {act!r}")
        self.act = 0 if self.clamped else ops.ACTIVATIONS[act]
        self.limit = float(spec.params.get("limit") or 0.0)
        self.alpha, self.up_shift = float(spec.params.get("alpha", 1.702)), float(spec.params.get("up_shift", 1.0))
        self.w_gate_up = self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        return [WeightSpec(w["gate"], (self.inner, self.width), "matrix", 0.02),
                WeightSpec(w["up"], (self.inner, self.width), "matrix", 0.02),
                WeightSpec(w["down"], (self.width, self.inner), "matrix", 0.02)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = self.spec.weights
        g, u = self._matrix(tensors[w["gate"]]), self._matrix(tensors[w["up"]])
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.w_gate_up = torch.cat([g, u], dim=0).contiguous()    # gate rows, then up rows
        self.w_down = self._matrix(tensors[w["down"]])

    def _inner(self, h: torch.Tensor) -> torch.Tensor:
        if not self.clamped:
            return linear.matmul(h, self.w_gate_up, epilogue=ops.EPI_GATED, act=self.act)
        if self.fused and self.alpha == ops.SWISH_ALPHA and self.up_shift == ops.SWISH_SHIFT:
            return linear.matmul(h, self.w_gate_up, epilogue=ops.EPI_GATED, act=ops.ACT_CLAMPED_SWISH, cap=self.limit)
        gu = linear.matmul(h, self.w_gate_up, out_dtype=torch.float32)
        z = torch.empty((h.shape[0], self.inner), dtype=h.dtype, device=h.device)
        ops.clamped_gated_act(gu, z, self.limit, self.alpha, self.up_shift)
        return z

    def forward(self, h: torch.Tensor, step: StepInfo = None) -> torch.Tensor:
        return linear.matmul(self._inner(h), self.w_down)

    def forward_partial(self, h: torch.Tensor, step: StepInfo = None) -> torch.Tensor:
        """As forward, but the down projection may come back as float32 partial sums
        [parts, N, width] for a consumer that adds them."""
        return linear.matmul_or_partials(self._inner(h), self.w_down)


class NoFeedForward(FeedForward):
    """A layer without a feed-forward: its output is None, which the arrangement leaves out of the sum."""
    graph_safe = True

    def forward(self, h: torch.Tensor, step: StepInfo = None):
        return None


register_part("feed_forward", "gated_mlp", GatedMLP)
register_part("feed_forward", "none", NoFeedForward)
