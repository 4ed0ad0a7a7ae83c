"""Arrangements: how one layer wires its norms, its mixer, its feed-forward and the
residual stream.  The residual stream x is float32 and is updated in place; the
sums are 32-bit.

"sandwich" (Gemma-2, src/forward.rs:291-414): norms before AND after each branch,
    x += post_mixer(mixer(pre_mixer(x)));  x += post_ffn(ffn(pre_ffn(x)))
    (a layer without a feed-forward has the first line only, and needs the first two norms only).
"prenorm" (the reference's other families): a norm before each branch only,
    x += mixer(pre_mixer(x));  x += ffn(pre_ffn(x))
"parallel": both branches read a norm (each its own weight) of the SAME x, and their sum is scaled,
    x += mult * (mixer(pre_mixer(x)) + ffn(pre_ffn(x)))
    (`mult`: the arrangement's own constant, LayerSpec.params["residual_mult"], default 1).
"parallel_shared_norm": both branches read ONE norm of x,
    h = pre(x);  x += mult * (mixer(h) + ffn(h))
"postnorm": the norm comes after the sum, and the branches read the residual stream itself,
    x <- post_mixer(alpha * x + mixer(x));  x <- post_ffn(alpha * x + ffn(x))
    (`alpha`: LayerSpec.params["alpha"], default 1; a layer without a feed-forward has the first line only).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.base import LayerSpec
from ..errors import SpecError
from ..registry import part_impl, register_part
from .base import CallStore, Runtime, StepInfo


class Layer:
    """Base of the arrangements: builds the layer's parts from the registry."""
    norm_roles = ()

    def __init__(self, spec: LayerSpec, rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.mixer = part_impl("mixer", spec.mixer.kind)(spec.mixer, rt)
        self.feed_forward = part_impl("feed_forward", spec.feed_forward.kind)(spec.feed_forward, rt)
        missing = [r for r in self.norm_roles if r not in spec.norms]
        if missing:
            raise SpecError(f"arch spec error: arrangement {spec.arrangement!r} needs norms {missing}")
        self.norms: Dict[str, object] = {
            role: part_impl("norm", ps.kind)(ps, rt) for role, ps in spec.norms.items()}

    def parts(self):
        return [self.mixer, self.feed_forward] + list(self.norms.values())

    # An arrangement whose first act is a norm of x may say so (`entry_norm`) and set
    # `chains = True`: the model then hands it `h_in`, that norm's output already computed by
    # the layer before, and `next_norm`, the entry norm of the layer after, whose output it
    # returns (computed in the kernel that makes its last residual sum).
    chains = False

    def entry_norm(self):
        return None

    def forward(self, x: torch.Tensor, step: StepInfo, store: CallStore, h_in=None, next_norm=None):
        raise NotImplementedError

    @staticmethod
    def _branch(part, takes_partials: bool, *args):
        """Run a mixer or feed-forward; let it hand back partial sums if it can and its consumer adds them."""
        if takes_partials and hasattr(part, "forward_partial"):
            return part.forward_partial(*args)
        return part.forward(*args)


class SandwichLayer(Layer):
    norm_roles = ("pre_mixer", "post_mixer")

    chains = True

    def __init__(self, spec: LayerSpec, rt: Runtime):
        super().__init__(spec, rt)
        from .feedforward import NoFeedForward
        self.has_ffn = not isinstance(self.feed_forward, NoFeedForward)
        missing = [r for r in ("pre_ffn", "post_ffn") if self.has_ffn and r not in spec.norms]
        if missing:
            raise SpecError(f"arch spec error: arrangement {spec.arrangement!r} needs norms {missing}")

    def entry_norm(self):
        return self.norms["pre_mixer"]

    def forward(self, x: torch.Tensor, step: StepInfo, store: CallStore, h_in=None, next_norm=None):
        n = self.norms
        h = h_in if h_in is not None else n["pre_mixer"].forward(x)
        a = self._branch(self.mixer, getattr(n["post_mixer"], "accepts_partials", False), h, step, store)
        if not self.has_ffn:
            return n["post_mixer"].add_to(a, x, then=next_norm)
        h = n["post_mixer"].add_to(a, x, then=n["pre_ffn"])     # x += post(a); h = pre_ffn(x)
        f = self._branch(self.feed_forward, getattr(n["post_ffn"], "accepts_partials", False), h, step)
        return n["post_ffn"].add_to(f, x, then=next_norm)       # x += post(f); next layer's entry norm


class PreNormLayer(Layer):
    norm_roles = ("pre_mixer", "pre_ffn")

    def forward(self, x: torch.Tensor, step: StepInfo, store: CallStore, h_in=None, next_norm=None):
        n = self.norms
        a = self.mixer.forward(n["pre_mixer"].forward(x), step, store)
        ops.residual_add(a, x)
        f = self.feed_forward.forward(n["pre_ffn"].forward(x), step)
        ops.residual_add(f, x)


class ParallelLayer(Layer):
    """x += mult * (mixer(n1(x)) + ffn(n2(x))), n1 and n2 norms of the same x.  One kernel makes the sum and
    both norms of the NEXT layer's input (or the model's last norm), so a layer costs one row-wise launch."""
    norm_roles = ("pre_mixer", "pre_ffn")
    chains = True

    def __init__(self, spec: LayerSpec, rt: Runtime):
        super().__init__(spec, rt)
        from .norm import NormPair, RMSNorm
        n = self.norms
        if not all(isinstance(n[r], RMSNorm) for r in self.norm_roles):
            raise SpecError("arch spec error: the parallel arrangement takes RMS norms")
        self.mult = float(spec.params.get("residual_mult", 1.0))
        self._pair = NormPair(n["pre_mixer"], n["pre_ffn"])

    def entry_norm(self):
        return self._pair

    def forward(self, x: torch.Tensor, step: StepInfo, store: CallStore, h_in=None, next_norm=None):
        from .norm import NormPair, RMSNorm
        h1, h2 = h_in if h_in is not None else self._pair.forward(x)
        a = self.mixer.forward(h1, step, store)
        f = self.feed_forward.forward(h2, step)
        if isinstance(next_norm, NormPair):
            o1 = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
            o2 = torch.empty_like(o1)
            ops.scaled_add_norms(a, f, self.mult, x, next_norm.first.weight, next_norm.first.eps, o1,
                                 next_norm.second.weight, next_norm.second.eps, o2)
            return o1, o2
        if isinstance(next_norm, RMSNorm) and not next_norm.add_one:
            o1 = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
            ops.scaled_add_norms(a, f, self.mult, x, next_norm.weight, next_norm.eps, o1)
            return o1
        ops.scaled_add_norms(a, f, self.mult, x)
        return next_norm.forward(x) if next_norm is not None else None


class SharedNormParallelLayer(Layer):
    """h = pre(x); x += mult * (mixer(h) + ffn(h)): one norm, read by both branches.  Where the next norm (the next
    layer's, or the model's last) can add and norm in one launch (`add_then`), the layer costs one row-wise launch;
    any other norm is run after a plain sum.  A branch may hand back 32-bit partial sums, which that launch adds."""
    norm_roles = ("pre",)
    chains = True

    def __init__(self, spec: LayerSpec, rt: Runtime):
        super().__init__(spec, rt)
        self.mult = float(spec.params.get("residual_mult", 1.0))

    def entry_norm(self):
        return self.norms["pre"]

    def forward(self, x: torch.Tensor, step: StepInfo, store: CallStore, h_in=None, next_norm=None):
        h = h_in if h_in is not None else self.norms["pre"].forward(x)
        fused = hasattr(next_norm, "add_then")
        a = self._branch(self.mixer, fused, h, step, store)
        f = self._branch(self.feed_forward, fused, h, step)
        if fused:
            return next_norm.add_then(a, f, self.mult, x)
        ops.scaled_add_norms(a, f, self.mult, x)
        return next_norm.forward(x) if next_norm is not None else None


class PostNormLayer(Layer):
    """x <- norm(alpha * x + branch(x)) for the mixer and then for the feed-forward.  The sum, the norm and the copy of
    the new x that the next branch's products read (or the model's last norm of it) are one kernel; x and the sums
    are 32-bit."""
    norm_roles = ("post_mixer",)
    chains = True

    def __init__(self, spec: LayerSpec, rt: Runtime):
        super().__init__(spec, rt)
        from .feedforward import NoFeedForward
        from .norm import RMSNorm, RowsAsGiven
        self.has_ffn = not isinstance(self.feed_forward, NoFeedForward)
        roles = ("post_mixer", "post_ffn") if self.has_ffn else ("post_mixer",)
        for r in roles:
            if not isinstance(self.norms.get(r), RMSNorm) or self.norms[r].add_one:
                raise SpecError(f"arch spec error: the postnorm arrangement takes a plain RMS norm as {r}")
        self.alpha = float(spec.params.get("alpha", 1.0))
        self._entry = RowsAsGiven(rt)

    def entry_norm(self):
        return self._entry

    def _sum_norm(self, y, x, norm, nxt):
        from .norm import RMSNorm, RowsAsGiven
        if isinstance(nxt, RowsAsGiven):
            if self.rt.is_fp32:
                ops.scale_add_norm(y, self.alpha, x, norm.weight, norm.eps)
                return x
            h = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
            ops.scale_add_norm(y, self.alpha, x, norm.weight, norm.eps, h)
            return h
        if isinstance(nxt, RMSNorm) and not nxt.add_one:
            h = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
            ops.scale_add_norm(y, self.alpha, x, norm.weight, norm.eps, h, nxt.weight, nxt.eps)
            return h
        ops.scale_add_norm(y, self.alpha, x, norm.weight, norm.eps)
        return nxt.forward(x) if nxt is not None else None

    def forward(self, x: torch.Tensor, step: StepInfo, store: CallStore, h_in=None, next_norm=None):
        h = h_in if h_in is not None else self._entry.forward(x)
        a = self._branch(self.mixer, True, h, step, store)
        if not self.has_ffn:
            return self._sum_norm(a, x, self.norms["post_mixer"], next_norm)
        h = self._sum_norm(a, x, self.norms["post_mixer"], self._entry)
        f = self._branch(self.feed_forward, True, h, step)
        return self._sum_norm(f, x, self.norms["post_ffn"], next_norm)


register_part("arrangement", "sandwich", SandwichLayer)
register_part("arrangement", "postnorm", PostNormLayer)
register_part("arrangement", "parallel", ParallelLayer)
register_part("arrangement", "parallel_shared_norm", SharedNormParallelLayer)
register_part("arrangement", "prenorm", PreNormLayer)
