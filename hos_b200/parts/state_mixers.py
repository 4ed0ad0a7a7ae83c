"""Two mixers that keep a matrix state S [dim keys x vdim values] per head and sequence instead of keys and values.

decay_linear_attention: q, k = act(W_q h), act(W_k h) (heads x dim), v = act(W_v h) (heads x vdim), act(x) = x
    logistic(x); per head S <- decay_h S + k v^T, o = S^T q with a constant decay per head and no other scale; the
    heads' outputs, side by side, are divided by their common root mean square, multiplied by a weight per column
    and by logistic(W_g h), and projected by W_o.  Each piece is a parameter: `activation` ("x_logistic", or None for
    q, k, v as projected); `position` (a rotary part: q and k turn with the token's position after the activation,
    angles in 32-bit); `key_scale` (a constant on k after the rotation); `norm` ("row": one root mean square over all
    heads; "head": one per head) with or without a weight (`norm_weight`); `gate` ("logistic" or "x_logistic").
gated_delta_rule: q, k (kv_heads x dim) and v (heads x vdim) each pass a short causal convolution over time per
    channel (`taps` wide, zeros before a sequence's start) and x logistic(x); q and k are divided by their lengths
    (sqrt(sum + 1e-6)) per head, q also by sqrt(dim); beta = logistic(W_b h) and the decay
    g = exp(-exp(A_log) softplus(W_a h + dt_bias)) are one number per head and token.  Per head (value head h reads
    key head h // (heads / kv_heads)):  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.  Each head's o
    is divided by its root mean square, multiplied by a weight shared by the heads and by W_g h times its logistic
    function, and projected by W_o.

The state (and the convolution's last taps - 1 inputs) is per-sequence state of fixed size: zero at a sequence's
start, carried from step to step.  Everything between the projections and the output projection is 32-bit: the
projections are one product that writes 32-bit rows.
"""
from __future__ import annotations

from typing import List, Mapping

import torch

from .. import ops
from ..errors import SpecError
from ..registry import part_impl, register_part
from . import linear
from .base import CallStore, Mixer, StateNeed, StepInfo, WeightSpec


class DecayLinearAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.width, self.n_heads = int(p["width"]), int(p["n_heads"])
        self.dim, self.vdim, self.eps = int(p["dim"]), int(p["vdim"]), float(p["eps"])
        self.decay = [float(d) for d in p["decay"]]
        if min(self.width, self.n_heads, self.dim, self.vdim) <= 0 or len(self.decay) != self.n_heads:
            raise SpecError("arch spec error: the decay mixer needs positive sizes and one decay per head")
        self.qk_cols, self.v_cols = self.n_heads * self.dim, self.n_heads * self.vdim
        act, norm, gate = p.get("activation", "x_logistic"), p.get("norm", "row"), p.get("gate", "logistic")
        if act not in (None, "x_logistic") or norm not in ("row", "head") or gate not in ("logistic", "x_logistic"):
            raise SpecError(f"arch spec error: the decay mixer with activation {act!r}, norm {norm!r}, gate {gate!r}")
        self.activates, self.norm_per_head = act is not None, norm == "head"
        self.norm_weight = bool(p.get("norm_weight", True))
        self.gate_act = ops.ACT_X_LOGISTIC if gate == "x_logistic" else ops.ACT_LOGISTIC
        self.key_scale = float(p.get("key_scale", 1.0))
        pos_spec = p.get("position")
        self.position = part_impl("position", pos_spec.kind)(pos_spec, rt) if pos_spec else None

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        out = [WeightSpec(w["q"], (self.qk_cols, self.width), "matrix", 0.05),
               WeightSpec(w["k"], (self.qk_cols, self.width), "matrix", 0.05),
               WeightSpec(w["v"], (self.v_cols, self.width), "matrix", 0.05),
               WeightSpec(w["gate"], (self.v_cols, self.width), "matrix", 0.05),
               WeightSpec(w["o"], (self.width, self.v_cols), "matrix", 0.02)]
        if self.norm_weight:       # a weight per column, or one shared by the heads where the norm is per head
            out.append(WeightSpec(w["norm"], (self.vdim if self.norm_per_head else self.v_cols,), "vector", 0.1))
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = self.spec.weights
        mats = [self._matrix(tensors[w[r]]) for r in ("q", "k", "v", "gate")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = self._matrix(tensors[w["o"]])
        if self.norm_weight:
            self.norm_w = self._vector32(tensors[w["norm"]])
        else:
            self.norm_w = torch.ones(self.vdim if self.norm_per_head else self.v_cols, dtype=torch.float32,
                                     device=self.w_o.device)
        self.decay_t = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(self.w_o.device)

    def state_needs(self) -> List[StateNeed]:
        return [StateNeed("S", (self.n_heads, self.vdim, self.dim), torch.float32)]      # kept as S^T per head

    def forward(self, h, step: StepInfo, store: CallStore):
        return self._run(h, step, store, False)

    def forward_partial(self, h, step: StepInfo, store: CallStore):
        return self._run(h, step, store, True)

    def _run(self, h, step, store, partial_ok):
        n = h.shape[0]
        proj = linear.matmul(h, self.w_in, out_dtype=torch.float32)
        o = torch.empty((n, self.v_cols), dtype=torch.float32, device=h.device)
        turns = self.position is not None or self.key_scale != 1.0
        rot = None
        if turns:
            # the rotation follows the activation, so the activation cannot ride in the scan's walk here
            if self.activates:
                ops.act_rows(proj, 2 * self.qk_cols + self.v_cols)
            freq, rot_dims, style = self.position.kernel_args() if self.position else (None, 0, 0)
            if step.max_new == 1 and not self.activates:
                rot = (freq, rot_dims, style, self.key_scale)       # single tokens: the scan turns what it stages
            else:
                ops.rotate_rows(proj, self.n_heads, self.n_heads, self.dim, freq, rot_dims, style, step, self.key_scale)
        ops.state_scan(proj, 0, self.qk_cols, 2 * self.qk_cols, self.activates and not turns, self.decay_t, False, None,
                       store.state["S"], step, o, self.n_heads, self.n_heads, self.dim, self.vdim, rot=rot)
        y = torch.empty((n, self.v_cols), dtype=h.dtype, device=h.device)
        if self.norm_per_head:
            ops.group_norm_gate(o, self.norm_w, proj, 2 * self.qk_cols + self.v_cols, self.gate_act, step.token_seq, y,
                                self.eps, self.n_heads, self.vdim)
        else:
            ops.group_norm_gate(o, self.norm_w, proj, 2 * self.qk_cols + self.v_cols, self.gate_act, step.token_seq, y,
                                self.eps, 1, self.v_cols)
        return linear.matmul_or_partials(y, self.w_o) if partial_ok else linear.matmul(y, self.w_o)


class GatedDeltaRule(Mixer):
    graph_safe = True

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = spec.params
        self.width, self.n_heads, self.n_kv_heads = int(p["width"]), int(p["n_heads"]), int(p["n_kv_heads"])
        self.dim, self.vdim, self.taps, self.eps = int(p["dim"]), int(p["vdim"]), int(p["taps"]), float(p["eps"])
        if min(self.width, self.n_heads, self.n_kv_heads, self.dim, self.vdim, self.taps) <= 0 \
                or self.n_heads % self.n_kv_heads != 0:
            raise SpecError("arch spec error: the delta-rule mixer needs positive sizes and heads that are a multiple of "
                            "its key heads")
        self.qk_cols, self.v_cols = self.n_kv_heads * self.dim, self.n_heads * self.vdim
        self.conv_cols = 2 * self.qk_cols + self.v_cols

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        out = []
        for r, rows in (("q", self.qk_cols), ("k", self.qk_cols), ("v", self.v_cols)):
            out.append(WeightSpec(w[r], (rows, self.width), "matrix", 0.05))
            out.append(WeightSpec(w[r + "_conv"], (rows, self.taps), "matrix", 0.4))
        out += [WeightSpec(w["beta"], (self.n_heads, self.width), "matrix", 0.05),
                WeightSpec(w["a"], (self.n_heads, self.width), "matrix", 0.05),
                WeightSpec(w["A_log"], (self.n_heads,), "vector", 0.5),
                WeightSpec(w["dt_bias"], (self.n_heads,), "vector", 0.5),
                WeightSpec(w["gate"], (self.v_cols, self.width), "matrix", 0.05),
                WeightSpec(w["norm"], (self.vdim,), "vector", 0.1),
                WeightSpec(w["o"], (self.width, self.v_cols), "matrix", 0.02)]
        return out

    def bind(self, tensors: Mapping[str, torch.Tensor]) -> None:
        w = self.spec.weights
        mats = [self._matrix(tensors[w[r]]) for r in ("q", "k", "v", "beta", "a", "gate")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.w_in = torch.cat(mats, dim=0).contiguous()           # q | k | v | beta | a | gate
        self.conv_w = torch.cat([tensors[w[r + "_conv"]].to(torch.float32) for r in ("q", "k", "v")], dim=0).contiguous()
        self.a_log, self.dt_bias = self._vector32(tensors[w["A_log"]]), self._vector32(tensors[w["dt_bias"]])
        self.norm_w = self._vector32(tensors[w["norm"]])
        self.w_o = self._matrix(tensors[w["o"]])

    def state_needs(self) -> List[StateNeed]:
        return [StateNeed("S", (self.n_heads, self.vdim, self.dim), torch.float32),
                StateNeed("conv", (max(self.taps - 1, 0), self.conv_cols), torch.float32)]

    def forward(self, h, step: StepInfo, store: CallStore):
        return self._run(h, step, store, False)

    def forward_partial(self, h, step: StepInfo, store: CallStore):
        return self._run(h, step, store, True)

    def _run(self, h, step, store, partial_ok):
        n, dev = h.shape[0], h.device
        raw = linear.matmul(h, self.w_in, out_dtype=torch.float32)
        act = torch.empty((n, self.conv_cols), dtype=torch.float32, device=dev)
        beta = torch.empty((n, self.n_heads), dtype=torch.float32, device=dev)
        g = torch.empty((n, self.n_heads), dtype=torch.float32, device=dev)
        kept = store.state["conv"]
        single = step.max_new == 1           # every sequence brings one token: the kept inputs move on in conv_prep itself
        ops.conv_prep(raw, self.conv_w, kept, self.a_log, self.dt_bias, step, act, beta, g, self.n_heads, self.n_kv_heads,
                      self.dim, self.vdim, keep_here=single)
        if not single:
            ops.conv_keep(raw, self.taps, kept, step, self.conv_cols)
        o = torch.empty((n, self.v_cols), dtype=torch.float32, device=dev)
        ops.state_scan(act, 0, self.qk_cols, 2 * self.qk_cols, False, g, True, beta, store.state["S"], step, o,
                       self.n_heads, self.n_kv_heads, self.dim, self.vdim)
        y = torch.empty((n, self.v_cols), dtype=h.dtype, device=dev)
        ops.group_norm_gate(o, self.norm_w, raw, self.conv_cols + 2 * self.n_heads, ops.ACT_X_LOGISTIC, step.token_seq, y,
                            self.eps, self.n_heads, self.vdim)
        return linear.matmul_or_partials(y, self.w_o) if partial_ok else linear.matmul(y, self.w_o)


register_part("mixer", "decay_linear_attention", DecayLinearAttention)
register_part("mixer", "gated_delta_rule", GatedDeltaRule)
