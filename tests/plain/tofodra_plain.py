"""Tofodra in plain, slow PyTorch (float64 by default, whole sequences, loops): the oracle of the tests.

One function per mechanism, written from the design's equations; nothing here is shared with the
library.  A model is (cfg, w): cfg the dict that config.json holds, w a dict of tensors by
checkpoint name.

  rms                 x / sqrt(mean(x^2) + eps)
  rotate_pairs        rotary positions on neighbouring pairs (2i, 2i+1) of the first `dims` numbers
  rotate_halves       rotary positions on pairs (i, i + dims/2) of the first `dims` numbers
  latent_mixer        attention whose keys and values are expanded from one normed latent row per position,
                      plus one rotated key part shared by the heads; a layer may read another layer's rows
  retention_mixer     S <- decay S + k v^T, o = S^T q per head; head norm without weight; silu gate
  visible             the mask: causal, the last `size` keys, and the first `keep_first` keys
  differential_mixer  two softmax maps over the same values, a1 - lambda a2, head norm, a logistic gate per column
  dense_ff            down(g logistic(1.702 g) (u + 1)) with g, u clamped
  routed_ff           logistic router scores, the `top` largest, normalised and scaled, a shared expert
  forward             per layer: x += ls1 norm1b(mixer(norm1 x)); x += ls2 norm2b(ff(norm2 x))
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z / (1.0 + torch.exp(-z))


def _angles(pos: int, rot, dtype):
    dims, base = rot["dims"], rot["base"]
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=dtype)
    a = pos * f
    return torch.cos(a), torch.sin(a)


def rotate_pairs(vec, pos: int, rot):
    """vec [..., n]: the first rot.dims numbers rotated, number 2i with number 2i+1."""
    dims = rot["dims"]
    c, s = _angles(pos, rot, vec.dtype)
    out = vec.clone()
    u, v = vec[..., 0:dims:2], vec[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def rotate_halves(vec, pos: int, rot):
    """vec [..., n]: the first rot.dims numbers rotated, number i with number i + dims/2."""
    dims = rot["dims"]
    half = dims // 2
    c, s = _angles(pos, rot, vec.dtype)
    out = vec.clone()
    u, v = vec[..., :half], vec[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def latent_rows(m, eps, w, p, h):
    """What a latent layer keeps per position: (normed latent [T, rank], rotated shared key part [T, rot_dim])."""
    R, r = m["kv_rank"], m["rot_dim"]
    d = h @ w[p + "dkv"].T
    c = rms(d[:, :R], eps) * w[p + "dkv.norm"]
    kr = torch.stack([rotate_pairs(d[t, R:R + r], t, m["rot"]) for t in range(h.shape[0])])
    return c, kr


def latent_mixer(m, eps, w, p, h, rows):
    """`rows` = (c, kr) of this layer or of the layer it reads.  The design's latent layers see every earlier key; a
    test may name a mask in the constants to take keys away."""
    T, H, d, r, vd = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = rows
    q = (h @ w[p + "q"].T).view(T, H, d + r)
    k = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, vd)
    out = torch.zeros(T, H, vd, dtype=h.dtype)
    for i in range(T):
        for hd in range(H):
            qr = rotate_pairs(q[i, hd, d:], i, m["rot"])
            js = torch.tensor([j for j in range(T) if visible(i, j, m.get("mask"))])
            s = (k[js, hd] @ q[i, hd, :d] + kr[js] @ qr) * m["scale"]
            pr = torch.softmax(s, 0)
            out[i, hd] = pr @ v[js, hd]
    return out.reshape(T, H * vd) @ w[p + "o"].T


def retention_mixer(m, eps, w, p, h):
    T, H, d, vd = h.shape[0], m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, vd)
    out = torch.zeros(T, H, vd, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(d, vd, dtype=h.dtype)
        for t in range(T):
            qt, kt = q[t, hd], k[t, hd]
            if m.get("rot"):            # a layer whose constants name no rotation turns nothing
                qt, kt = rotate_halves(qt, t, m["rot"]), rotate_halves(kt, t, m["rot"])
            kt = kt * d ** -0.5
            S = m["decay"][hd] * S + torch.outer(kt, v[t, hd])
            out[t, hd] = rms(S.T @ qt, eps)
    return (out.reshape(T, H * vd) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def visible(i: int, j: int, mask: Optional[dict]) -> bool:
    if j > i:
        return False
    if not mask:
        return True
    return i - j < mask["size"] or j < mask.get("keep_first", 0)


def differential_mixer(m, eps, w, p, h):
    T, H, G, d, vd = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, 2, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, 2, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, vd)
    lam = torch.exp((w[p + "lq1"] * w[p + "lk1"]).sum()) - torch.exp((w[p + "lq2"] * w[p + "lk2"]).sum()) + m["diff"]
    out = torch.zeros(T, H, vd, dtype=h.dtype)
    for i in range(T):
        js = torch.tensor([j for j in range(T) if visible(i, j, m.get("mask"))])
        for hd in range(H):
            g = hd // (H // G)
            a = [torch.softmax((k[js, g, mp] @ q[i, hd, mp]) * m["scale"], 0) @ v[js, g] for mp in (0, 1)]
            out[i, hd] = rms(a[0] - lam * a[1], eps) * (1.0 - m["diff"])
    return (out.reshape(T, H * vd) * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def dense_ff(mlp, w, p, h):
    lim = mlp["limit"]
    g = torch.clamp(h @ w[p + "gate"].T, max=lim)
    u = torch.clamp(h @ w[p + "up"].T, -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def expert_ff(w, p, h):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_ff(mlp, w, p, h):
    n, top, mult = mlp["router"]["experts"], mlp["router"]["top"], mlp["router"].get("scale", 1.0)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        s = torch.sigmoid(h[t] @ w[p + "router"].T)
        chosen = sorted(range(n), key=lambda e: (-float(s[e]), e))[:top]
        total = sum(s[e] for e in chosen) + 1e-20
        for e in chosen:
            out[t] += s[e] / total * mult * expert_ff(w, f"{p}e{e}.", h[t][None])[0]
    if mlp.get("shared"):
        out = out + expert_ff(w, p + "shared.", h)
    return out


def feed_forward(mlp, w, p, h):
    if mlp["kind"] == "dense":
        return dense_ff(mlp, w, p, h)
    return routed_ff(mlp, w, p, h)


def forward(cfg, w, tokens: List[int], taps: Optional[list] = None, edit=None):
    """Logits [T, vocab] of one sequence.  `taps`, a list, receives the residual stream after every layer.
    `edit(layer index, mixer constants)` may return a changed copy of a mixer's constants (tests use it to move a
    window's edge or to read another layer's rows)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"] if edit is None else edit(i, dict(layer["mixer"]))
        h = rms(x, eps) * w[p + "norm1"]
        if layer["type"] == "latent_attention":
            if m.get("kv_from") is None:
                kept[i] = latent_rows(m, eps, w, p + "mix.", h)
            a = latent_mixer(m, eps, w, p + "mix.", h, kept[i if m.get("kv_from") is None else m["kv_from"]])
        elif layer["type"] == "retention":
            a = retention_mixer(m, eps, w, p + "mix.", h)
        else:
            a = differential_mixer(m, eps, w, p + "mix.", h)
        x = x + rms(a, eps) * w[p + "norm1b"] * w[p + "ls1"]
        if layer.get("mlp") is not None:
            h = rms(x, eps) * w[p + "norm2"]
            f = feed_forward(layer["mlp"], w, p + "mlp.", h)
            x = x + rms(f, eps) * w[p + "norm2b"] * w[p + "ls2"]
        if taps is not None:
            taps.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["head"].T
