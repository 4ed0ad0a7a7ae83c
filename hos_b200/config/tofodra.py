"""Typed configuration of Tofodra: a decoder-only model whose layers are listed one by one in config.json.  Every
layer has an RMS norm before and after each branch and a multiplier per column on each branch's normed output
(layer scale).  The mixer is attention over a latent cache (a layer may read an earlier layer's cache), retention
(a matrix state with a constant decay per head), or differential softmax attention over a window that keeps the
sequence's first keys in sight; the feed-forward is a clamped gated dense one, routed experts with a shared expert,
or absent.

    {"architecture": "Tofodra", "vocab": V, "width": D, "norm": {"eps": e}, "embedding": {"scale": s},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads": H, "dim": d, "rot_dim": r, "vdim": v, "kv_rank": R, "scale": s,
                           "rot": {"base": b, "dims": r}, "kv_from": j},
                 "mlp": MLP or null},
                {"type": "retention",
                 "mixer": {"heads": H, "dim": d, "vdim": v, "decay": [..H numbers..], "rot": {"base": b, "dims": n}}, ...},
                {"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": v, "scale": s, "diff": c,
                           "mask": {"size": W, "keep_first": K}}, ...}]}
    MLP = {"kind": "dense", "ff": F, "limit": L}
        | {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k, "scale": m}, "shared": {"ff": S}}

`kv_from`, `rot` (retention), `mask`, `mask.keep_first`, `shared`, `router.scale`, `embedding.scale` and `mlp` may be
absent (a cache of the layer's own, no rotation, every earlier key in sight, no kept keys, no shared expert, weights
that sum to one, rows as the table holds them, no feed-forward).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Mapping, Tuple

from ..errors import MissingMetaError
from .base import ConfigReader, ModelConfig

MIXER_TYPES = ("latent_attention", "retention", "attention")
MLP_KINDS = ("dense", "moe")


def _section(raw: Mapping[str, Any], key: str, where: str) -> Mapping[str, Any]:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise MissingMetaError(f"missing model metadata: {where}{key} (an object is required)")
    return v


def _bad(msg: str):
    raise MissingMetaError("model metadata invalid: " + msg)


def _positive(r: ConfigReader, keys, where: str) -> None:
    for key in keys:
        if r.need_int(key) <= 0:
            _bad(f"{where}{key} must be positive")


def _rot(m: Mapping[str, Any], where: str, at_most: int, required: bool):
    rot = m.get("rot")
    if rot is None:
        if required:
            raise MissingMetaError(f"missing model metadata: {where}rot (an object is required)")
        return
    r = ConfigReader(_section(m, "rot", where))
    dims, base = r.need_int("dims"), r.opt_float("base", None)
    if base is None or not base > 0.0:
        _bad(f"{where}rot.base must be a positive number")
    if dims <= 0 or dims % 2 or dims > at_most:
        _bad(f"{where}rot.dims must be even and lie between 2 and {at_most}")


@dataclass(frozen=True)
class TofodraConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[Mapping[str, Any], ...]      # the entries as config.json has them, checked

    architecture = "Tofodra"

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "TofodraConfig":
        r = ConfigReader(raw)
        eps = ConfigReader(_section(raw, "norm", "")).opt_float("eps", None)
        if eps is None:
            raise MissingMetaError("missing model metadata: norm.eps")
        emb = raw.get("embedding") if isinstance(raw.get("embedding"), dict) else {}
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise MissingMetaError("missing model metadata: layers (a list of layers is required)")
        cfg = cls(vocab=r.need_int("vocab"), width=r.need_int("width"), norm_eps=eps,
                  embedding_scale=ConfigReader(emb).opt_float("scale", 1.0), layers=tuple(copy.deepcopy(l) for l in layers))
        cfg.check()
        return cfg

    def check(self) -> None:
        for key in ("vocab", "width"):
            if getattr(self, key) <= 0:
                _bad(f"{key} must be positive")
        if not self.norm_eps > 0.0:
            _bad("norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict):
                _bad(f"layers[{i}] must be an object")
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                _bad(f"{where}type must be one of {MIXER_TYPES}, found {kind!r}")
            m = _section(layer, "mixer", where)
            getattr(self, "_check_" + kind)(i, m, where + "mixer.")
            self._check_mlp(layer.get("mlp"), where)

    def _check_latent_attention(self, i: int, m, where: str) -> None:
        r = ConfigReader(m)
        _positive(r, ("heads", "dim", "rot_dim", "vdim", "kv_rank"), where)
        if r.opt_float("scale", None) is None:
            _bad(f"{where}scale is required")
        _rot(m, where, r.need_int("rot_dim"), True)
        src = r.opt_int("kv_from", None)
        if src is None:
            return
        if not 0 <= src < i or self.layers[src].get("type") != "latent_attention" \
                or self.layers[src]["mixer"].get("kv_from") is not None:
            _bad(f"{where}kv_from must name an earlier latent_attention layer that keeps a cache of its own")
        other = self.layers[src]["mixer"]
        if any(other.get(k) != m.get(k) for k in ("kv_rank", "rot_dim", "rot")):
            _bad(f"{where}kv_from names layer {src}, whose kv_rank, rot_dim or rot differ")

    def _check_retention(self, i: int, m, where: str) -> None:
        r = ConfigReader(m)
        _positive(r, ("heads", "dim", "vdim"), where)
        decay = m.get("decay")
        if not isinstance(decay, list) or len(decay) != r.need_int("heads") \
                or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
            _bad(f"{where}decay must list one number per head")
        _rot(m, where, r.need_int("dim"), False)

    def _check_attention(self, i: int, m, where: str) -> None:
        r = ConfigReader(m)
        _positive(r, ("heads", "kv_heads", "dim", "vdim"), where)
        if r.need_int("heads") % r.need_int("kv_heads") != 0:
            _bad(f"{where}heads must be a multiple of {where}kv_heads")
        if r.opt_float("scale", None) is None or r.opt_float("diff", None) is None:
            _bad(f"{where}scale and {where}diff are required")
        mask = m.get("mask")
        if mask is not None:
            mk = ConfigReader(mask if isinstance(mask, dict) else {})
            if mk.need_int("size") <= 0 or mk.opt_int("keep_first", 0) < 0:
                _bad(f"{where}mask needs a positive size and a keep_first of zero or more")

    @staticmethod
    def _check_mlp(mlp, where: str) -> None:
        if mlp is None:
            return
        if not isinstance(mlp, dict) or mlp.get("kind") not in MLP_KINDS:
            _bad(f"{where}mlp.kind must be one of {MLP_KINDS} (or mlp null)")
        if mlp["kind"] == "dense":
            r = ConfigReader(mlp)
            if r.need_int("ff") <= 0:
                _bad(f"{where}mlp.ff must be positive")
            limit = r.opt_float("limit", None)
            if limit is None or not limit > 0.0:
                _bad(f"{where}mlp.limit must be a positive number")
            return
        router = ConfigReader(_section(mlp, "router", where + "mlp."))
        if ConfigReader(_section(mlp, "expert", where + "mlp.")).need_int("ff") <= 0:
            _bad(f"{where}mlp.expert.ff must be positive")
        if not 0 < router.need_int("top") <= router.need_int("experts"):
            _bad(f"{where}mlp.router.top must lie between 1 and mlp.router.experts")
        router.opt_float("scale", 1.0)
        if mlp.get("shared") is not None and ConfigReader(_section(mlp, "shared", where + "mlp.")).need_int("ff") <= 0:
            _bad(f"{where}mlp.shared.ff must be positive")

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
                "layers": [copy.deepcopy(dict(l)) for l in self.layers]}
