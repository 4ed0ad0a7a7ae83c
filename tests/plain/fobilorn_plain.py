"""Fobilorn in plain, slow PyTorch (float64 by default, whole sequences, loops): the oracle of the tests.

One function per mechanism, written from the design's equations; nothing here is shared with the
library.  A model is (cfg, w): cfg the dict that config.json holds, w a dict of tensors by
checkpoint name.

  dyt               tanh(alpha x) * weight + bias  (no mean, no variance)
  rms               x / sqrt(mean(x^2) + eps)
  embed             table row + pair-table row (hash of previous and current token), then dyt
  visible           the mask: causal, the last `size` keys, and the first `keep_first` keys
  attention_mixer   q/k norm over the whole projection, scores, mask, softmax with one more in the
                    denominator, values mixed with the first mixing layer's, a gate per head
  dense_ff          down(silu(gate h) * up h)
  routed_ff         logistic router scores, the `top` largest, expert(score * h) summed, a shared expert
  forward           per layer: h = dyt(x); x += mixer(h) + ff(h)
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch


def dyt(x, w, name):
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z / (1.0 + torch.exp(-z))


def embed(cfg, w, tokens):
    big = cfg.get("embedding", {}).get("bigram")
    rows = []
    for t, tok in enumerate(tokens):
        row = w["embed"][tok]
        if big:
            r = big["buckets"] if t == 0 else (tokens[t - 1] * big["mul_prev"] + tok * big["mul_cur"]) % big["buckets"]
            row = row + w["bigram"][r]
        rows.append(row)
    return dyt(torch.stack(rows), w, "embed.norm")


def visible(i: int, j: int, mask: Optional[dict]) -> bool:
    if j > i:
        return False
    if not mask:
        return True
    return i - j < mask["size"] or j < mask.get("keep_first", 0)


def attention_mixer(m, eps, w, p, h, v_first, mixes: bool, sink: bool = True):
    """h: [T, width].  Returns (output [T, width], the values this layer made before mixing).  `mixes`: this layer
    blends its values with `v_first`.  `sink` False leaves the one out of the denominator (what a test compares with)."""
    T, H, G, d, vd = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms(h @ w[p + "q"].T, eps) * w[p + "q.norm"]          # over all heads at once
    k = rms(h @ w[p + "k"].T, eps) * w[p + "k.norm"]
    v = h @ w[p + "v"].T
    v_own = v
    if mixes:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v + lam * v_first
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, vd)
    gate = torch.sigmoid(h @ w[p + "g"].T)                    # [T, H]
    out = torch.zeros(T, H, vd, dtype=h.dtype)
    for i in range(T):
        js = torch.tensor([j for j in range(T) if visible(i, j, m.get("mask"))])
        for hd in range(H):
            g = hd // (H // G)
            e = torch.exp((k[js, g] @ q[i, hd]) * m["scale"])
            pr = e / ((1.0 if sink else 0.0) + e.sum())
            out[i, hd] = (pr[:, None] * v[js, g]).sum(0) * gate[i, hd]
    return out.reshape(T, H * vd) @ w[p + "o"].T, v_own


def gated_ff(w, p, h):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_ff(mlp, w, p, h):
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        s = torch.sigmoid(h[t] @ w[p + "router"].T)
        order = sorted(range(n), key=lambda e: (-float(s[e]), e))[:top]
        for e in order:
            out[t] += gated_ff(w, f"{p}e{e}.", (s[e] * h[t])[None])[0]
    if mlp.get("shared"):
        out = out + gated_ff(w, p + "shared.", h)
    return out


def feed_forward(mlp, w, p, h):
    if mlp is None:
        return torch.zeros_like(h)
    if mlp["kind"] == "dense":
        return gated_ff(w, p, h)
    return routed_ff(mlp, w, p, h)


def forward(cfg, w, tokens: List[int], taps: Optional[list] = None, edit=None, sink: bool = True):
    """Logits [T, vocab] of one sequence.  `taps`, a list, receives the residual stream after the embedding and after
    every layer.  `edit(cfg_layer_mixer)` may return a changed copy of a mixer's constants (tests use it to move a
    window's edge)."""
    eps = cfg["norm"]["eps"]
    x = embed(cfg, w, tokens)
    if taps is not None:
        taps.append(x.clone())
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = dyt(x, w, p + "norm1")
        m = layer["mixer"] if edit is None else edit(dict(layer["mixer"]))
        wants = bool(m.get("v_mix"))
        a, v_own = attention_mixer(m, eps, w, p + "mix.", h, v_first, wants and v_first is not None, sink)
        if wants and v_first is None:
            v_first = v_own
        x = x + (a + feed_forward(layer.get("mlp"), w, p + "mlp.", h))
        if taps is not None:
            taps.append(x.clone())
    return dyt(x, w, "final.norm") @ w["head"].T
