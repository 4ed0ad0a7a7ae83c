"""Shared by the Fobilorn tests: small configurations that differ from one another in every size and constant, model
folders with random weights scaled so that every mechanism matters to the logits (sharp attention, norms whose
scalar and bias are far from 1 and 0, blending weights between a fifth and four fifths, router logits of a few
units), and the comparison rules.

Tolerances, fixed before the first run (the ones the other designs' tests use): 32-bit: every row's error (root mean
square over the vocabulary) at most 2e-5 of the logits' root mean square; bfloat16: at most 4e-2 of it for at least
nine rows in ten (a router choice that rounding flips is no fault)."""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Optional

import torch

from satapel_cases import assert_rows, oracle_view, row_errors, tokens  # noqa: F401  (the rules are the same)


def attention(heads, kv_heads, dim, vdim, scale, window=None, keep=None, v_mix=False, mlp="dense"):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
        if keep is not None:
            m["mask"]["keep_first"] = keep
    if v_mix:
        m["v_mix"] = True
    return {"type": "attention", "mixer": m, "mlp": mlp}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def model(width, vocab, layers, ff=48, eps=1e-6, bigram=(13, 5, 3)):
    out = []
    for layer in layers:
        layer = json.loads(json.dumps(layer))
        if layer["mlp"] == "dense":
            layer["mlp"] = {"kind": "dense", "ff": ff}
        out.append(layer)
    raw = {"architecture": "Fobilorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {}, "layers": out}
    if bigram:
        raw["embedding"]["bigram"] = dict(zip(("buckets", "mul_prev", "mul_cur"), bigram))
    return raw


# a layer that blends nothing first; three query heads over one kv head, values wider than keys, a window of 70 (no
# multiple of a page) that keeps 3 keys; then the layer whose values the later ones blend in (top 2 of 5 with a shared
# expert), a blending layer without a feed-forward, and one that sees all keys and uses every expert it has
CASE_A = model(72, 211, [attention(3, 1, 16, 24, 0.8, window=70, keep=3),
                         attention(4, 2, 16, 8, 0.6, window=5, keep=2, v_mix=True, mlp=moe(5, 2, 40, shared=24)),
                         attention(2, 2, 24, 8, 0.5, window=33, keep=0, v_mix=True, mlp=None),
                         attention(4, 2, 8, 8, 1.1, v_mix=True, mlp=moe(3, 3, 16))], ff=56)
# blending from the first layer on; a window and a kept run of exactly one page; a window of one key that keeps one;
# nine heads over three kv heads; top 1; multipliers beyond 32 bits and one bucket
CASE_B = model(64, 150, [attention(9, 3, 8, 8, 1.2, window=64, keep=64, v_mix=True, mlp=moe(4, 1, 24, shared=40)),
                         attention(3, 3, 16, 8, 0.4, window=1, keep=1, v_mix=True),
                         attention(1, 1, 32, 16, 0.3, window=7, mlp=None),
                         attention(6, 3, 8, 8, 0.9, window=20, keep=30, v_mix=True, mlp=moe(2, 1, 8))],
               ff=40, eps=1e-5, bigram=(1, 6_000_000_007, 4_000_000_009))
# no pair table, no blending anywhere; keys wider than values; more kept keys than two pages hold
CASE_C = model(80, 90, [attention(2, 1, 40, 16, 0.3, window=10, keep=130),
                        attention(4, 4, 8, 8, 1.5, mlp=moe(6, 4, 24, shared=8)),
                        attention(5, 1, 16, 16, 0.7, window=129, keep=1, mlp=None)], ff=24, bigram=None)
# sizes that are multiples of nothing (a width of 100 is no multiple of 8: the tensor-core products step aside)
CASE_D = model(100, 77, [attention(5, 5, 12, 20, 0.7, window=33, keep=6, v_mix=True, mlp=moe(7, 3, 36, shared=20)),
                         attention(5, 5, 12, 20, 0.7, window=9, keep=7, v_mix=True),
                         attention(10, 5, 6, 20, 0.9, v_mix=True, mlp=moe(3, 2, 12))], ff=36, eps=3e-5, bigram=(10, 3, 1))
# wider layers: heads of 64/128 numbers (the tensor-core attention kernels), a window longer than four pages (decoding
# cuts a row's keys into shares) that keeps more than a page, experts of several feature tiles
CASE_E = model(256, 500, [attention(16, 4, 64, 128, 0.25, window=300, keep=70, v_mix=True, mlp=moe(6, 2, 264, shared=136)),
                          attention(8, 4, 128, 128, 0.2, window=130, keep=5, v_mix=True),
                          attention(4, 2, 128, 64, 0.15, window=64, keep=64, mlp=None),
                          attention(16, 4, 64, 128, 0.25, v_mix=True, mlp=moe(9, 1, 72))], ff=264, bigram=(509, 31, 7))
CASES = {"A": (CASE_A, 31), "B": (CASE_B, 32), "C": (CASE_C, 33), "D": (CASE_D, 34), "E": (CASE_E, 35)}


def _scaled(name: str, t: torch.Tensor) -> torch.Tensor:
    t = t.float()
    if name.endswith(".alpha"):
        return 0.6 + 2.0 * t.abs()
    if name.endswith((".norm.b", "norm1.b")):
        return 2.0 * t
    if name.endswith(("norm1", "final.norm", "embed.norm", "q.norm", "k.norm")):
        return 1.0 + t
    if name.endswith("vmix"):
        return (0.5 + t).clamp(0.2, 0.8)
    if name in ("embed", "bigram"):
        return t * 25.0
    if name == "head":
        return t * 10.0
    if name.endswith(("mix.o", ".down")):
        return t * 5.0
    if name.endswith(("mix.q", "mix.k", "mix.v", "mix.g", ".gate", ".up")):
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
