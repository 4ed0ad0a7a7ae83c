"""Fobilorn as data: the function from a `FobilornConfig` to a `ModelPlan`.

Embedding: the token table plus a hashed token-pair table, then a Dynamic Tanh norm (tanh(alpha x) w + b).  Every
layer is a parallel block with one such norm, h = norm1(x); x += mixer(h) + ff(h).  The mixer is softmax attention
with grouped queries: RMS norms over the whole query and the whole key projection, no rotation, a window that keeps
the sequence's first keys in sight, one added to the softmax's denominator, values blended with the first blending
layer's values of the same token, a gate per head.  The feed-forward is a gated dense one (x logistic(x)), or routed
experts with logistic scores whose weights multiply the experts' inputs, plus an expert that every token uses.  The
model ends with a Dynamic Tanh norm and an untied head.  Tensor names: `embed`, `bigram`, `embed.norm`,
`l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`; a norm `n` keeps its bias as `n.b`, its scalar as `n.alpha`.
"""
from __future__ import annotations

from ..config.base import LayerCall, LayerSpec, ModelPlan, PartSpec
from ..config.fobilorn import FobilornConfig
from ..registry import register_architecture

MAX_POSITIONS = 1 << 20        # the format names no limit: the cache alone bounds a sequence
VALUE_MIX_KEY = "first_values"


def _norm(cfg: FobilornConfig, name: str) -> PartSpec:
    return PartSpec("dynamic_tanh", {"width": cfg.width}, {"weight": name, "bias": name + ".b", "alpha": name + ".alpha"})


def _mixer(cfg: FobilornConfig, i: int, layer, p: str) -> PartSpec:
    m = layer["mixer"]
    mask = m.get("mask")
    value_mix = None
    if m.get("v_mix"):
        value_mix = {"key": VALUE_MIX_KEY, "role": "source" if cfg.first_value_mix() == i else "mixed"}
    return PartSpec(
        "gated_softmax_attention",
        {"width": cfg.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
         "scale": float(m["scale"]), "eps": cfg.norm_eps, "window": int(mask["size"]) if mask else None,
         "keep_first": int(mask.get("keep_first", 0)) if mask else 0, "bias": False, "qk_norm": "whole", "sink": "zero",
         "head_gate": True, "value_mix": value_mix, "position": None},
        {"q": p + "q", "k": p + "k", "v": p + "v", "q_norm": p + "q.norm", "k_norm": p + "k.norm", "gate": p + "g",
         "o": p + "o", "value_mix": p + "vmix"})


def _gated(cfg: FobilornConfig, inner: int, p: str) -> PartSpec:
    return PartSpec("gated_mlp", {"width": cfg.width, "inner": inner, "activation": "silu"},
                    {"gate": p + "gate", "up": p + "up", "down": p + "down"})


def _feed_forward(cfg: FobilornConfig, layer, p: str) -> PartSpec:
    mlp = layer.get("mlp")
    if mlp is None:
        return PartSpec("none")
    if mlp["kind"] == "dense":
        return _gated(cfg, mlp["ff"], p)
    shared = mlp.get("shared")
    return PartSpec("routed_experts",
                    {"width": cfg.width, "inner": mlp["expert"]["ff"], "experts": mlp["router"]["experts"],
                     "top": mlp["router"]["top"], "identity": 0, "limit": None, "alpha": 1.0, "up_shift": 0.0,
                     "scoring": "logistic", "weight_on": "input", "correction": False,
                     "shared": _gated(cfg, shared["ff"], p + "shared.") if shared else None},
                    {"router": p + "router", "expert": p + "e{}.", "gate": "gate", "up": "up", "down": "down"})


def fobilorn_plan(cfg: FobilornConfig) -> ModelPlan:
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        layers.append(LayerSpec("parallel_shared_norm", _mixer(cfg, i, layer, p + "mix."),
                                _feed_forward(cfg, layer, p + "mlp."), {"pre": _norm(cfg, p + "norm1")}))
    if cfg.bigram is not None:
        embedding = PartSpec("pair_hash_embedding",
                             {"vocab": cfg.vocab, "width": cfg.width, "buckets": cfg.bigram[0], "mul_prev": cfg.bigram[1],
                              "mul_cur": cfg.bigram[2], "norm": _norm(cfg, "embed.norm")},
                             {"table": "embed", "pair_table": "bigram"})
    else:
        embedding = PartSpec("scaled_embedding", {"vocab": cfg.vocab, "width": cfg.width, "scale": 1.0,
                                                  "norm": _norm(cfg, "embed.norm")}, {"table": "embed"})
    return ModelPlan(
        width=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS, embedding=embedding, layers=layers,
        schedule=[LayerCall(i) for i in range(len(layers))], final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "width": cfg.width, "softcap": 0.0}, {"table": "head"}),
    )


register_architecture("Fobilorn", FobilornConfig, fobilorn_plan)
