"""Typed configuration of Fobilorn: a decoder-only model whose layers are listed one by one in config.json; every
layer is a parallel block with ONE norm (Dynamic Tanh), whose mixer is softmax attention over a window that keeps
the sequence's first keys in sight, and whose feed-forward is dense, a routed set of experts with a shared one, or
absent.

    {"architecture": "Fobilorn", "vocab": V, "width": D, "norm": {"eps": e},
     "embedding": {"bigram": {"buckets": B, "mul_prev": a, "mul_cur": b}},
     "layers": [{"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": v, "scale": s,
                           "mask": {"size": W, "keep_first": K}, "v_mix": true},
                 "mlp": MLP or null}]}
    MLP = {"kind": "dense", "ff": F}
        | {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k}, "shared": {"ff": S}}

`embedding.bigram`, `mask`, `mask.keep_first`, `v_mix`, `shared` and `mlp` may be absent (no pair table, every
earlier key in sight, no kept keys, values of the layer's own, no shared expert, no feed-forward).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from ..errors import MissingMetaError
from .base import ConfigReader, ModelConfig

MIXER_TYPES = ("attention",)
MLP_KINDS = ("dense", "moe")


def _section(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise MissingMetaError(f"missing model metadata: {where}{key} (an object is required)")
    return v


def _bad(msg: str):
    raise MissingMetaError("model metadata invalid: " + msg)


@dataclass(frozen=True)
class FobilornConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    bigram: Optional[Tuple[int, int, int]]     # (buckets, mul_prev, mul_cur), or no pair table
    layers: Tuple[Mapping[str, Any], ...]      # the entries as config.json has them, checked

    architecture = "Fobilorn"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "FobilornConfig":
        r = ConfigReader(raw)
        norm = ConfigReader(_section(raw, "norm", ""))
        eps = norm.opt_float("eps", None)
        if eps is None:
            raise MissingMetaError("missing model metadata: norm.eps")
        emb = raw.get("embedding") if isinstance(raw.get("embedding"), dict) else {}
        bigram = None
        if emb.get("bigram") is not None:
            b = ConfigReader(_section(emb, "bigram", "embedding."))
            bigram = (b.need_int("buckets"), b.need_int("mul_prev"), b.need_int("mul_cur"))
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise MissingMetaError("missing model metadata: layers (a list of layers is required)")
        cfg = cls(vocab=r.need_int("vocab"), width=r.need_int("width"), norm_eps=eps, bigram=bigram,
                  layers=tuple(copy.deepcopy(l) for l in layers))
        cfg.check()
        return cfg

    def check(self) -> None:
        for key in ("vocab", "width"):
            if getattr(self, key) <= 0:
                _bad(f"{key} must be positive")
        if not self.norm_eps > 0.0:
            _bad("norm.eps must be positive")
        if self.bigram is not None and self.bigram[0] <= 0:
            _bad("embedding.bigram.buckets must be positive")
        first_mix = None
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict):
                _bad(f"layers[{i}] must be an object")
            if layer.get("type") not in MIXER_TYPES:
                _bad(f"{where}type must be one of {MIXER_TYPES}, found {layer.get('type')!r}")
            m = ConfigReader(_section(layer, "mixer", where))
            for key in ("heads", "kv_heads", "dim", "vdim"):
                if m.need_int(key) <= 0:
                    _bad(f"{where}mixer.{key} must be positive")
            if m.need_int("heads") % m.need_int("kv_heads") != 0:
                _bad(f"{where}mixer.heads must be a multiple of mixer.kv_heads")
            if m.opt_float("scale", None) is None:
                _bad(f"{where}mixer.scale is required")
            mask = layer["mixer"].get("mask")
            if mask is not None:
                mk = ConfigReader(mask if isinstance(mask, dict) else {})
                if mk.need_int("size") <= 0 or mk.opt_int("keep_first", 0) < 0:
                    _bad(f"{where}mixer.mask needs a positive size and a keep_first of zero or more")
            if m.opt_bool("v_mix", False):
                shape = (m.need_int("kv_heads"), m.need_int("vdim"))
                if first_mix is None:
                    first_mix = (i, shape)
                elif shape != first_mix[1]:
                    _bad(f"{where}mixer mixes its values with layer {first_mix[0]}'s, whose kv_heads or vdim differ")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
                _bad(f"{where}mlp.kind must be one of {MLP_KINDS} (or mlp null)")
            if mlp["kind"] == "dense":
                if ConfigReader(mlp).need_int("ff") <= 0:
                    _bad(f"{where}mlp.ff must be positive")
                continue
            router = ConfigReader(_section(mlp, "router", where + "mlp."))
            if ConfigReader(_section(mlp, "expert", where + "mlp.")).need_int("ff") <= 0:
                _bad(f"{where}mlp.expert.ff must be positive")
            if not 0 < router.need_int("top") <= router.need_int("experts"):
                _bad(f"{where}mlp.router.top must lie between 1 and mlp.router.experts")
            if mlp.get("shared") is not None and ConfigReader(_section(mlp, "shared", where + "mlp.")).need_int("ff") <= 0:
                _bad(f"{where}mlp.shared.ff must be positive")

    def first_value_mix(self) -> Optional[int]:
        """The first layer that says v_mix: the one whose values the later such layers blend into theirs."""
        for i, layer in enumerate(self.layers):
            if layer["mixer"].get("v_mix"):
                return i
        return None

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "embedding": {},
               "layers": [copy.deepcopy(dict(l)) for l in self.layers]}
        if self.bigram is not None:
            out["embedding"]["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), self.bigram))
        return out
