"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * (w + add_one)  (src/forward.rs:166-174;
`add_one` is Gemma's (1 + w) convention, src/hf.rs:101-107).  Statistics in 32-bit.
A norm may name a second tensor, `scale`: a multiplier per column on the norm's output (the layer scale of a
branch whose last act is this norm).  It is folded into the weight when the tensors are bound, (w + add_one) * scale
in 32-bit, which is exact for weights stored in bfloat16 (16 bits of product) and one rounding otherwise."""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from .. import ops
from ..registry import register_part
from .base import Norm, WeightSpec


class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.add_one = bool(spec.params.get("add_one", False))
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        out = [WeightSpec(self.spec.weights["weight"], (self.width,), "vector", 0.1)]
        if self.spec.weights.get("scale"):
            out.append(WeightSpec(self.spec.weights["scale"], (self.width,), "vector", 0.1))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        self.weight = self._vector32(tensors[self.spec.weights["weight"]])
        if self.spec.weights.get("scale"):
            # y * w * scale == y * (w * scale); with Gemma's convention the kernel adds one, so that is taken here
            scale = self._vector32(tensors[self.spec.weights["scale"]])
            self.weight = ((self.weight + 1.0) * scale - 1.0 if self.add_one else self.weight * scale).contiguous()

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        ops.rmsnorm(x, self.weight, self.eps, self.add_one, out)
        return out

    accepts_partials = True      # y may be [parts, N, width] float32 partial sums

    def add_to(self, y: torch.Tensor, x: torch.Tensor, then: Optional[Norm] = None):
        """x += self(y); with another RMSNorm as `then`, its output comes from the same kernel."""
        if then is None:
            ops.norm_add_norm(y, self.weight, self.eps, self.add_one, x)
            return None
        if isinstance(then, RMSNorm):
            h = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
            ops.norm_add_norm(y, self.weight, self.eps, self.add_one, x,
                              then.weight, then.eps, then.add_one, h)
            return h
        ops.norm_add_norm(y, self.weight, self.eps, self.add_one, x)
        return then.forward(x)


register_part("norm", "rmsnorm", RMSNorm)


class DynamicTanh(Norm):
    """y = tanh(alpha * x) * w + b: a norm that takes no mean and no variance (alpha one number, w and b a number
    per column; 32-bit).  `forward(x, out=x)` norms the 32-bit rows in place."""
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.width = int(spec.params["width"])
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.alpha = 1.0

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        return [WeightSpec(w["weight"], (self.width,), "vector", 0.1), WeightSpec(w["bias"], (self.width,), "vector", 0.1),
                WeightSpec(w["alpha"], (), "vector", 0.1)]

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = self.spec.weights
        self.weight = self._vector32(tensors[w["weight"]])
        self.bias = self._vector32(tensors[w["bias"]])
        self.alpha = float(tensors[w["alpha"]].float().reshape(-1)[0].item())     # read once, here

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        ops.add_dyt(None, None, 0.0, x, self.alpha, self.weight, self.bias, out)
        return out

    def add_then(self, a, f, mult: float, x: torch.Tensor) -> torch.Tensor:
        """x += mult * (a + f) and this norm of the new x, in one launch (a, f: rows or 32-bit partial sums, or None)."""
        h = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        ops.add_dyt(a, f, mult, x, self.alpha, self.weight, self.bias, h)
        return h


register_part("norm", "dynamic_tanh", DynamicTanh)


class NormPair:
    """Two RMSNorms of the same row, from one kernel: what a block needs whose mixer and feed-forward both
    read a norm of the same residual stream.  `forward(x)` gives (first, second)."""

    def __init__(self, first: RMSNorm, second: RMSNorm):
        if first.add_one or second.add_one:
            raise ValueError("a pair of norms takes plain weights")
        self.first, self.second = first, second

    def forward(self, x: torch.Tensor):
        h1 = torch.empty(x.shape, dtype=self.first.rt.dtype, device=x.device)
        h2 = torch.empty_like(h1)
        ops.scaled_add_norms(None, None, 0.0, x, self.first.weight, self.first.eps, h1,
                             self.second.weight, self.second.eps, h2)
        return h1, h2


class RowsAsGiven:
    """Stands where an arrangement expects the norm that a layer's first branch reads, for layers whose branches
    read the residual stream itself: `forward(x)` is x in the products' type (x itself in the 32-bit path)."""

    def __init__(self, rt):
        self.rt = rt

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.rt.is_fp32:
            return x
        h = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        ops.cast_rows(x, h)
        return h
