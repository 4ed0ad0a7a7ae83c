"""Tofodra as data: the function from a `TofodraConfig` to a `ModelPlan`.

Embedding: the token table times a constant.  Every layer is the sandwich arrangement with plain RMS norms,
x += ls1 * norm1b(mixer(norm1 x)); x += ls2 * norm2b(ff(norm2 x)), the multipliers per column (`ls1`, `ls2`) being a
second tensor of the norm after the branch.  Mixers: attention over a latent cache with interleaved rotary pairs
on the shared key part (a layer with `kv_from` reads an earlier layer's cache); retention, the decay-rule matrix
state with rotate-half rotary pairs on q and k, keys times dim^-1/2, a norm per head without a weight and an
x logistic(x) gate; differential attention, two softmax maps over the same values, with biases, a window that keeps
the first keys and a logistic gate per column.  Feed-forward: the clamped gated dense form, or routed experts with
logistic scores, weights normalised over the chosen and scaled, plus an expert every token uses.  Tensor names:
`embed`, `l<i>.norm1|norm1b|norm2|norm2b|ls1|ls2`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.base import LayerCall, LayerSpec, ModelPlan, PartSpec
from ..config.tofodra import TofodraConfig
from ..registry import register_architecture

MAX_POSITIONS = 1 << 20        # the format names no limit: the cache alone bounds a sequence
SWISH_ALPHA = 1.702            # the dense feed-forward's gate is g logistic(1.702 g)
WEIGHT_SUM_FLOOR = 1e-20       # added to the sum of the chosen experts' scores before the division


def _rotary(rot, style: str) -> PartSpec:
    return PartSpec("rotary", {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]), "style": style,
                               "table": "float64"})


def _mixer(cfg: TofodraConfig, layer, p: str) -> PartSpec:
    m, kind = layer["mixer"], layer["type"]
    if kind == "latent_attention":
        shares = m.get("kv_from") is not None
        names = {"q": p + "q", "uk": p + "uk", "uv": p + "uv", "o": p + "o"}
        if not shares:
            names.update({"dkv": p + "dkv", "dkv_norm": p + "dkv.norm"})
        return PartSpec("latent_attention",
                        {"width": cfg.width, "n_heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"],
                         "vdim": m["vdim"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "eps": cfg.norm_eps,
                         "window": None, "sink": False, "shares_kv": shares,
                         "position": _rotary(m["rot"], "interleaved")}, names)
    if kind == "retention":
        return PartSpec("decay_linear_attention",
                        {"width": cfg.width, "n_heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"],
                         "decay": tuple(float(d) for d in m["decay"]), "eps": cfg.norm_eps, "activation": None,
                         "position": _rotary(m["rot"], "rotate_half") if m.get("rot") else None,
                         "key_scale": float(m["dim"]) ** -0.5, "norm": "head", "norm_weight": False,
                         "gate": "x_logistic"},
                        {"q": p + "q", "k": p + "k", "v": p + "v", "gate": p + "g", "o": p + "o"})
    mask = m.get("mask")
    return PartSpec("differential_attention",
                    {"width": cfg.width, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "dim": m["dim"],
                     "vdim": m["vdim"], "scale": float(m["scale"]), "eps": cfg.norm_eps, "diff": float(m["diff"]),
                     "window": int(mask["size"]) if mask else None,
                     "keep_first": int(mask.get("keep_first", 0)) if mask else 0, "bias": True, "gate": True},
                    {"q": p + "q", "k": p + "k", "v": p + "v", "q_bias": p + "q.b", "k_bias": p + "k.b",
                     "v_bias": p + "v.b", "lq1": p + "lq1", "lk1": p + "lk1", "lq2": p + "lq2", "lk2": p + "lk2",
                     "gate": p + "g", "o": p + "o"})


def _gated(cfg: TofodraConfig, inner: int, p: str) -> PartSpec:
    return PartSpec("gated_mlp", {"width": cfg.width, "inner": inner, "activation": "silu"},
                    {"gate": p + "gate", "up": p + "up", "down": p + "down"})


def _feed_forward(cfg: TofodraConfig, layer, p: str) -> PartSpec:
    mlp = layer.get("mlp")
    if mlp is None:
        return PartSpec("none")
    if mlp["kind"] == "dense":
        return PartSpec("gated_mlp", {"width": cfg.width, "inner": mlp["ff"], "activation": "clamped_swish",
                                      "limit": float(mlp["limit"]), "alpha": SWISH_ALPHA, "up_shift": 1.0},
                        {"gate": p + "gate", "up": p + "up", "down": p + "down"})
    shared = mlp.get("shared")
    return PartSpec("routed_experts",
                    {"width": cfg.width, "inner": mlp["expert"]["ff"], "experts": mlp["router"]["experts"],
                     "top": mlp["router"]["top"], "identity": 0, "limit": None, "alpha": 1.0, "up_shift": 0.0,
                     "scoring": "logistic", "weight_on": "output", "correction": False,
                     "renormalise": WEIGHT_SUM_FLOOR, "weight_scale": float(mlp["router"].get("scale", 1.0)),
                     "shared": _gated(cfg, shared["ff"], p + "shared.") if shared else None},
                    {"router": p + "router", "expert": p + "e{}.", "gate": "gate", "up": "up", "down": "down"})


def tofodra_plan(cfg: TofodraConfig) -> ModelPlan:
    def norm(name: str, scale: str = None) -> PartSpec:
        names = {"weight": name}
        if scale:
            names["scale"] = scale
        return PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.norm_eps, "add_one": False}, names)

    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norms = {"pre_mixer": norm(p + "norm1"), "post_mixer": norm(p + "norm1b", p + "ls1")}
        if layer.get("mlp") is not None:
            norms.update({"pre_ffn": norm(p + "norm2"), "post_ffn": norm(p + "norm2b", p + "ls2")})
        layers.append(LayerSpec("sandwich", _mixer(cfg, layer, p + "mix."), _feed_forward(cfg, layer, p + "mlp."), norms))
        schedule.append(LayerCall(i, layer["mixer"].get("kv_from") if layer["type"] == "latent_attention" else None))
    return ModelPlan(
        width=cfg.width, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=PartSpec("scaled_embedding", {"vocab": cfg.vocab, "width": cfg.width, "scale": cfg.embedding_scale},
                           {"table": "embed"}),
        layers=layers, schedule=schedule, final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab": cfg.vocab, "width": cfg.width, "softcap": 0.0}, {"table": "head"}),
    )


register_architecture("Tofodra", TofodraConfig, tofodra_plan)
