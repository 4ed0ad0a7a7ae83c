"""Shared by the Tofodra tests: small configurations that differ from one another in every size and constant, model
folders with random weights scaled so that every mechanism matters to the logits (sharp attention, norm weights and
layer scales around one, a lambda far from its constant, router logits of a few units, clamps that bite), and the
comparison rules.

Tolerances, fixed before the first run (the ones the other designs' tests use): 32-bit: every row's error (root mean
square over the vocabulary) at most 2e-5 of the logits' root mean square; bfloat16: at most 4e-2 of it for at least
nine rows in ten (a router choice that rounding flips is no fault)."""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Optional

import torch

from satapel_cases import assert_rows, oracle_view, row_errors, tokens  # noqa: F401  (the rules are the same)


def latent(heads, dim, rot_dim, vdim, rank, scale, base=10000.0, kv_from=None, mlp="dense"):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def retention(decay, dim, vdim, rot=None, base=10000.0, mlp="dense"):
    m = {"heads": len(decay), "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot:
        m["rot"] = {"base": base, "dims": rot}
    return {"type": "retention", "mixer": m, "mlp": mlp}


def attention(heads, kv_heads, dim, vdim, scale, diff, window=None, keep=None, mlp="dense"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if window:
        m["mask"] = {"size": window}
        if keep is not None:
            m["mask"]["keep_first"] = keep
    return {"type": "attention", "mixer": m, "mlp": mlp}


def moe(experts, top, ff, shared=None, scale=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if scale is not None:
        out["router"]["scale"] = scale
    if shared:
        out["shared"] = {"ff": shared}
    return out


def model(width, vocab, layers, ff=48, limit=1.0, eps=1e-6, scale=4.0):
    out = []
    for layer in layers:
        layer = json.loads(json.dumps(layer))
        if layer["mlp"] == "dense":
            layer["mlp"] = {"kind": "dense", "ff": ff, "limit": limit}
        out.append(layer)
    return {"architecture": "Tofodra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": out}


# retention first (three heads, keys wider than values, a third of a head rotated), a latent layer whose cache the
# LAST layer reads with other heads, a differential layer with three query heads to a kv head and a window of 70 (no
# multiple of a page) that keeps 3, routed experts with and without a shared one, a layer without a feed-forward
CASE_A = model(72, 211, [retention((0.9, 0.97, 0.995), 24, 16, rot=8, mlp=moe(5, 2, 40, shared=24, scale=1.7)),
                         latent(3, 16, 8, 24, 40, 0.35),
                         attention(3, 1, 16, 24, 0.8, 0.35, window=70, keep=3, mlp=None),
                         retention((0.8,), 8, 32, mlp=moe(3, 3, 16)),
                         latent(2, 24, 8, 16, 40, 0.3, kv_from=1)], ff=56, limit=0.8)
# a latent layer read by TWO later layers with a layer in between; a window and a kept run of exactly one page; a
# window of one key; a kv head to every query head; top 1; a decay of exactly one; a whole head rotated
CASE_B = model(64, 150, [latent(4, 8, 16, 8, 24, 0.5, base=500.0, mlp=moe(4, 1, 24, shared=40)),
                         attention(2, 2, 8, 8, 1.2, 0.8, window=64, keep=64),
                         latent(1, 32, 16, 40, 24, 0.25, base=500.0, kv_from=0, mlp=None),
                         retention((1.0, 0.5), 16, 16, rot=16, base=100.0),
                         attention(4, 2, 16, 8, 0.4, 0.1, window=1, keep=0),
                         latent(5, 8, 16, 8, 24, 0.6, base=500.0, kv_from=0)], ff=40, limit=2.5, eps=1e-5, scale=1.0)
# attention first and without a mask; more kept keys than two pages hold; two latent caches, each with a reader
CASE_C = model(80, 90, [attention(2, 1, 40, 16, 0.3, 0.5),
                        latent(2, 16, 4, 16, 36, 0.4),
                        latent(4, 8, 2, 8, 20, 0.7, base=50.0, mlp=moe(6, 4, 24, shared=8, scale=0.5)),
                        latent(3, 8, 4, 24, 36, 0.5, kv_from=1, mlp=None),
                        attention(6, 2, 8, 8, 0.9, 0.25, window=10, keep=130),
                        latent(1, 16, 2, 8, 20, 0.4, base=50.0, kv_from=2),
                        retention((0.99, 0.9, 0.7, 0.3), 8, 8, rot=2)], ff=24, limit=0.5, scale=9.0)
# sizes that are multiples of nothing (a width of 100 is no multiple of 8: the tensor-core products step aside)
CASE_D = model(100, 77, [latent(5, 12, 6, 20, 30, 0.4, mlp=moe(7, 3, 36, shared=20, scale=3.0)),
                         retention((0.95, 0.6, 0.999, 0.9, 0.85), 12, 20, rot=6),
                         attention(5, 5, 6, 20, 0.7, 0.45, window=33, keep=6),
                         latent(5, 12, 6, 20, 30, 0.4, kv_from=0, mlp=moe(3, 2, 12))], ff=36, limit=1.2, eps=3e-5, scale=2.5)
# wider layers: differential maps of 32 and 64 numbers (key rows of 64 and 128: the tensor-core attention kernels), a
# window longer than four pages that keeps more than a page, retention heads of 64 x 128 and 128 x 64, a latent of
# 200 numbers, experts of several feature tiles
CASE_E = model(256, 500, [attention(8, 2, 32, 128, 0.25, 0.3, window=300, keep=70, mlp=moe(6, 2, 264, shared=136, scale=2.0)),
                          retention((0.97, 0.999), 64, 128, rot=64),
                          latent(16, 16, 16, 24, 200, 0.3),
                          attention(4, 4, 64, 64, 0.2, 0.7, window=64, keep=64, mlp=None),
                          retention((0.9,), 128, 64, rot=32, mlp=moe(9, 1, 72)),
                          latent(4, 32, 16, 40, 200, 0.25, kv_from=2)], ff=264, limit=2.0, scale=8.0)
CASES = {"A": (CASE_A, 41), "B": (CASE_B, 42), "C": (CASE_C, 43), "D": (CASE_D, 44), "E": (CASE_E, 45)}


def _scaled(name: str, t: torch.Tensor) -> torch.Tensor:
    t = t.float()
    if name.endswith(("norm1", "norm2", "norm1b", "norm2b", "final.norm", "dkv.norm")):
        return 1.0 + t
    if name.endswith((".ls1", ".ls2")):
        return 0.7 + 2.0 * t
    if name.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
        return 3.0 * t
    if name == "embed":
        return t * 25.0
    if name == "head":
        return t * 10.0
    if name.endswith(("mix.q", "mix.dkv")):
        return t * 6.0
    if name.endswith("mix.o"):
        return t * 5.0
    if name.endswith((".gate", ".up", ".down", "mix.uk", "mix.uv", "mix.k", "mix.v", "mix.g")):
        return t * 3.0
    return t


def make_folder(tmp_path, raw: dict, seed: int, name: str = "m",
                edit: Optional[Callable[[Dict[str, torch.Tensor]], None]] = None) -> str:
    from hos_b200.model import weight_specs_for
    from hos_b200.registry import config_from_dict
    from hos_b200.weights import RandomSource
    from hos_b200.weights.safetensors import SINGLE_FILE, write_safetensors
    cfg = config_from_dict(raw)
    src = RandomSource(weight_specs_for(cfg), seed)
    tensors = {n: _scaled(n, src.read(n)) for n in src.names()}
    if edit is not None:
        edit(tensors)
    d = os.path.join(str(tmp_path), name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg.to_dict(), f)
    write_safetensors(os.path.join(d, SINGLE_FILE), ((n, t.to(torch.bfloat16)) for n, t in tensors.items()),
                      metadata={"format": "pt"})
    return d
