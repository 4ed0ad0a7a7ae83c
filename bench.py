#!/usr/bin/env python3
"""Measurement: decode and prompt throughput of Gemma-2 2B sizes with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch B] [--ctx C] [--layers L]

A "step" is one decode step of the whole batch.  The timed region is K decode steps that end
at context length C (default 8192, the benchmark context of the 2B configuration), timed on
the device with CUDA events; `value` is decoded tokens per second.  `e2e` is the same steps
through the public entry point (`Engine.generate_from_ids` on conversations that hold the
context): every step uploads which slots run from pinned memory and brings the sampled ids
back to the host, where the loop reads them one step late.  `prefill` is one prompt of 2,048 tokens.  `roofline` relates the bytes a decode
step must read (every weight once, and the cache of the live sequences) to its time.
`points` holds decoding at batch 1 and 64.  One JSON line is printed.

`--design satapel` (or `vagonex`, `fobilorn`, `tofodra`) is another measurement (not the line above): prompt and decode throughput of that design at
a few sizes beside Gemma-2 at equal size, and each of the design's kernels against its roofline; one JSON line per size.
With `--profile prefill|decode` it measures nothing and runs two such steps of one block of layers kernel by kernel, for a profiler.

Random weights are made on the device; the cache of the decode measurements is filled with
random keys and values instead of being computed by a prompt (a decode step reads the same
bytes either way), and says so under config.cache_fill.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Gemma-2 2B layer sizes
GEMMA2_2B = dict(
    architectures=["Gemma2ForCausalLM"], model_type="gemma2", num_hidden_layers=26, hidden_size=2304,
    num_attention_heads=8, num_key_value_heads=4, head_dim=256, intermediate_size=9216,
    vocab_size=256000, rope_theta=10000.0, sliding_window=4096, max_position_embeddings=8192,
    query_pre_attn_scalar=256, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
    rms_norm_eps=1e-6, tie_word_embeddings=True)
# Gemma-2 9B and 27B layer sizes; not part of the default line
GEMMA2_9B = dict(GEMMA2_2B, num_hidden_layers=42, hidden_size=3584, num_attention_heads=16,
                 num_key_value_heads=8, head_dim=256, intermediate_size=14336, query_pre_attn_scalar=256)
GEMMA2_27B = dict(GEMMA2_2B, num_hidden_layers=46, hidden_size=4608, num_attention_heads=32,
                  num_key_value_heads=16, head_dim=128, intermediate_size=36864, query_pre_attn_scalar=144)
MODELS = {"2b": GEMMA2_2B, "9b": GEMMA2_9B, "27b": GEMMA2_27B}
FULL_LAYERS = 26
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                raw = json.load(f)
            out, found = dict(FALLBACK_PEAKS), 0

            def look(node):            # the keys may sit at the top or one level down
                nonlocal found
                if not isinstance(node, dict):
                    return
                for k, v in node.items():
                    if k in out and isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0:
                        out[k] = float(v)
                        found += 1
                    elif isinstance(v, dict):
                        look(v)
            look(raw)
            if found:
                return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi in the background while the timed region runs (reading only)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons)}


def weight_bytes(cfg, n_layers) -> int:
    """Bytes of every weight a decode step reads once (bfloat16): the layers' matrices and
    norm vectors, the final norm, and the head (the tied embedding table, read whole by the
    head; the embedding lookup reads one row per sequence, which is not counted)."""
    d, qd = cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim
    kvd, f = cfg.num_key_value_heads * cfg.head_dim, cfg.intermediate_size
    per_layer = (qd + 2 * kvd) * d + d * qd + 2 * f * d + d * f
    norms = 4 * d * 4                       # float32 vectors
    return n_layers * (per_layer * 2 + norms) + d * 4 + cfg.vocab_size * d * 2


def kv_bytes_at(cfg, n_layers, length) -> int:
    """Cache bytes one sequence of `length` tokens makes a decode step read (bfloat16 keys
    and values; even layers see the last sliding_window keys only)."""
    per_tok = 2 * cfg.num_key_value_heads * cfg.head_dim * 2
    sliding = sum(1 for l in range(n_layers) if cfg.layer_is_sliding(l))
    return per_tok * (sliding * min(length, cfg.sliding_window) + (n_layers - sliding) * length)


def prefill_flops(cfg, n_layers, t) -> float:
    d, qd = cfg.hidden_size, cfg.num_attention_heads * cfg.head_dim
    kvd, f = cfg.num_key_value_heads * cfg.head_dim, cfg.intermediate_size
    linear = 2.0 * t * ((qd + 2 * kvd) * d + d * qd + 3 * f * d)
    flops = 0.0
    for l in range(n_layers):
        w = cfg.sliding_window if cfg.layer_is_sliding(l) else t
        pairs = sum(min(p + 1, w) for p in range(t))
        flops += linear + 4.0 * cfg.head_dim * cfg.num_attention_heads * pairs
    return flops + 2.0 * d * cfg.vocab_size          # the head runs on the last row


def fill_cache_random(runner):
    import torch
    for g in runner.cache.groups:
        for t in g.k + g.v:
            flat = t.view(-1)
            for lo in range(0, flat.numel(), 1 << 28):
                flat[lo:lo + (1 << 28)].normal_(0.0, 0.5)


MIXED = (1.0, 0.5, 0.25, 0.125, 0.0625, 0.0625, 0.03125, 0.03125)     # --mixed-lengths: fractions of the context, in turn


def measure_decode(eng, batch, ctx, steps, warmup, rng, clocks=None, mixed=False):
    """K timed decode steps that end at length ctx (with `mixed`: at the fractions MIXED of it, in turn).  Returns
    (device ms per step, e2e ms per step, kernel launches in the timed region, h2d bytes per step, d2h bytes per
    step, mean length, or with `mixed` the list of the sequences' mean lengths)."""
    import torch
    r = eng.runner
    vocab = r.vocab_size
    ends = [max(warmup + steps + 1, int(ctx * MIXED[i % len(MIXED)])) if mixed else ctx for i in range(batch)]
    starts = [e - (warmup + steps) for e in ends]

    def prepare():
        slots = r.admit(batch)
        r.cache.extend_all(slots, starts)
        return slots

    # ---- device-timed: steps issued back to back, tokens stay on the device ----
    slots = prepare()
    toks = [[rng.randrange(vocab)] for _ in range(batch)]
    ms_dev, launches = r.decode_steps_timed(slots, toks, warmup, steps, clocks)
    for s in slots:
        r.release(s)

    # ---- end to end: the public entry point (Engine.generate_from_ids on conversations that hold the
    # context), token ids back on the host; every step uploads which slots run and brings its tokens back ----
    convs = eng.open(batch)
    r.cache.extend_all([c.slot for c in convs], starts)
    r.write_records([c.slot for c in convs], pos=starts)
    for c, start in zip(convs, starts):
        c.position = start
    kw = dict(temp=0.0, top_k=0, top_p=1.0, rep_penalty=1.0, stop_ids=[])
    eng.generate_from_ids(convs, [[rng.randrange(vocab)] for _ in range(batch)], max_tokens=warmup, **kw)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = eng.generate_from_ids(convs, [[] for _ in range(batch)], max_tokens=steps, **kw)
    torch.cuda.synchronize()
    ms_e2e = (time.perf_counter() - t0) * 1e3 / steps
    assert all(len(o) == steps for o in outs), "every sequence decodes every step"
    for c in convs:
        c.close()
    from hos_b200.engine.decode import META, bucket_for
    h2d = (META + bucket_for(batch)) * 4       # live rows, stop ids, the slots that run
    d2h = bucket_for(batch) * 4                # the sampled ids
    mean_len = [e - steps / 2.0 for e in ends] if mixed else ctx - steps / 2.0
    return ms_dev, ms_e2e, launches, h2d, d2h, mean_len


def measure_prefill(eng, tokens, rng, reps=3, pieces=1):
    """Milliseconds of one prompt of `tokens` tokens (the best of `reps` runs after a warm-up
    run), fed whole or as `pieces` steps of equal size that continue one another."""
    import torch
    r = eng.runner
    prompt = [rng.randrange(r.vocab_size) for _ in range(tokens)]
    size = (tokens + pieces - 1) // pieces
    best = None
    for i in range(reps + 1):
        slot = r.admit(1)[0]
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for lo in range(0, tokens, size):
            r.step([slot], [prompt[lo:lo + size]])
        e1.record()
        torch.cuda.synchronize()
        r.release(slot)
        ms = e0.elapsed_time(e1)
        if i > 0:                              # the first run warms up
            best = ms if best is None else min(best, ms)
    return best


def run_baseline_workload(args) -> int:
    """The workloads that go with the 9B and 27B layer sizes: 9B, 16 prompts of seeded lengths
    U[64, 2048] in one ragged prompt step, then 256 greedy tokens each, context 4096; 27B, 8 prompts of
    1,024 tokens, then 256 each; 2B, 8 prompts of 512 and decoding as far as --decode-tokens says.
    Method of the reference's own bench (src/lib.rs:683-727): one warm-up prompt step, then the prompt
    step and the greedy decoding timed apart, through `Engine.bench`, the public entry point."""
    import random
    import torch
    from hos_b200 import Engine
    from hos_b200 import models  # noqa: F401
    from hos_b200.registry import config_from_dict
    full_layers = MODELS[args.model]["num_hidden_layers"]
    layers = args.layers or full_layers
    ctx = 4096 if args.model != "2b" else 8192
    cfg = config_from_dict(dict(MODELS[args.model], num_hidden_layers=layers, max_position_embeddings=ctx))
    rng = random.Random(0)
    if args.model == "9b":
        lens = [rng.randint(64, 2048) for _ in range(16)]
    elif args.model == "27b":
        lens = [1024] * 8
    else:
        lens = [512] * 8
    decode = args.decode_tokens
    prompts = [[rng.randrange(cfg.vocab_size) for _ in range(n)] for n in lens]
    pk, pk_src = peaks()
    eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_batch=len(lens),
                             max_tokens=sum((n + decode + 63) // 64 * 64 for n in lens), max_seq_len=ctx)
    clocks = ClockSampler(torch.cuda.current_device())
    clocks.start()
    n_prompt, pre_s, pre_tps, produced, dec_s, dec_tps = eng.bench(prompts, decode)
    clock_rec = clocks.stop()
    fl = sum(prefill_flops(cfg, layers, n) for n in lens)
    steps = produced / len(lens)
    wbytes = weight_bytes(cfg, layers)
    step_bytes = wbytes + sum(kv_bytes_at(cfg, layers, n + int(steps / 2)) for n in lens)
    ms_step = dec_s * 1e3 / max(steps, 1e-9)
    print(json.dumps({
        "workload": "baseline", "model": f"gemma-2-{args.model} sizes, random weights", "layers": layers,
        "layers_full": full_layers, "batch": len(lens), "prompt_tokens": n_prompt, "prompt_lengths": "U[64,2048] seeded"
        if args.model == "9b" else str(lens[0]), "context": ctx, "dtype": "bf16", "peaks": pk_src, "clocks": clock_rec,
        "prefill": {"tokens": n_prompt, "ms": pre_s * 1e3, "value": pre_tps, "unit": "tok/s", "tflop": fl / 1e12,
                    "frac": fl / pre_s / (pk["bf16_tflops_sustained"] * 1e12), "peak_tflops": pk["bf16_tflops_sustained"],
                    "of": pk_src + " (sustained)"},
        "decode": {"tokens": produced, "steps": steps, "ms_per_step": ms_step, "value": dec_tps, "unit": "tok/s",
                   "bytes_per_step": step_bytes, "achieved_gbs": step_bytes / (ms_step * 1e-3) / 1e9,
                   "frac": step_bytes / (ms_step * 1e-3) / 1e9 / pk["hbm_gbs"], "peak_gbs": pk["hbm_gbs"], "of": pk_src}}))
    return 0


# ---- --design satapel: the Satapel design beside Gemma-2 at equal size --------------------------------
# Sizes that resemble a real model's layers.  Gemma-2 "at equal size": the same width, layer count and
# vocabulary, as many query heads of as many numbers (dim + rot_dim), an intermediate size equal to what a
# Satapel token uses (top x ff), a window of the same length on its windowed layers.
SATAPEL_SIZES = {
    "s": dict(width=1024, vocab=32000, blocks=2, heads=8, dim=96, rot=32, vdim=64, rank=256, window=1024,
              wkv_heads=16, wkv_dim=64, decay_rank=64, experts=8, identity=1, top=2, ff=1024),
    "m": dict(width=2048, vocab=32000, blocks=2, heads=16, dim=64, rot=64, vdim=128, rank=512, window=1024,
              wkv_heads=32, wkv_dim=64, decay_rank=64, experts=16, identity=1, top=2, ff=1536),
    "l": dict(width=4096, vocab=64000, blocks=1, heads=32, dim=64, rot=64, vdim=128, rank=512, window=2048,
              wkv_heads=64, wkv_dim=64, decay_rank=128, experts=32, identity=2, top=4, ff=1024),
}
FP32_TFLOPS = 148 * 128 * 2 * 1.9e9 / 1e12      # the FMA pipes of 148 SMs at 1.9 GHz: the bound of 32-bit arithmetic


def satapel_raw(z):
    mlp = {"kind": "moe", "expert": {"ff": z["ff"], "limit": 7.0},
           "router": {"experts": z["experts"], "identity": z["identity"], "top": z["top"]}}
    att = {"type": "latent_attention", "mlp": mlp,
           "mixer": {"heads": z["heads"], "dim": z["dim"], "rot_dim": z["rot"], "vdim": z["vdim"], "kv_rank": z["rank"],
                     "scale": (z["dim"] + z["rot"]) ** -0.5, "mask": {"size": z["window"]},
                     "rot": {"base": 10000.0, "dims": z["rot"]}}}
    rec = {"type": "wkv", "mlp": mlp, "mixer": {"heads": z["wkv_heads"], "dim": z["wkv_dim"], "decay_rank": z["decay_rank"]}}
    return {"architecture": "Satapel", "vocab": z["vocab"], "width": z["width"], "residual_mult": 0.5, "norm": {"eps": 1e-5},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 10007}},
            "layers": [rec, att, att, att] * z["blocks"]}


def gemma_raw_like(z):
    hd = z["dim"] + z["rot"]
    return dict(architectures=["Gemma2ForCausalLM"], model_type="gemma2", num_hidden_layers=4 * z["blocks"],
                hidden_size=z["width"], num_attention_heads=z["heads"], num_key_value_heads=max(1, z["heads"] // 2),
                head_dim=hd, intermediate_size=z["top"] * z["ff"], vocab_size=z["vocab"], rope_theta=10000.0,
                sliding_window=z["window"], max_position_embeddings=8192, query_pre_attn_scalar=hd,
                attn_logit_softcapping=50.0, final_logit_softcapping=30.0, rms_norm_eps=1e-6, tie_word_embeddings=True)


def satapel_kernel_work(z, tokens, batch, ctx):
    """Per launch of each of the design's own kernels: (bytes that must move, FLOPs of the mathematics) for a prompt of
    `tokens` tokens and for a decode step of `batch` sequences at length `ctx` (bfloat16 storage)."""
    H, D, R, W = z["heads"], z["rank"] + z["rot"], z["rank"], z["window"]
    pairs = sum(min(p + 1, W) for p in range(tokens))
    keys = min(ctx, W)
    wh, wd, C = z["wkv_heads"], z["wkv_dim"], z["wkv_heads"] * z["wkv_dim"]
    top, ff, width = z["top"], z["ff"], z["width"]
    real = z["experts"] / float(z["experts"] + z["identity"])           # share of the choices that are real experts
    touched = min(z["experts"], batch * top)
    return {
        "hos_latent_attn": {"prefill": (tokens * D * 2 + tokens * H * (D + R) * 4, 2.0 * pairs * H * (D + R)),
                            "decode": (batch * keys * D * 2, 2.0 * batch * keys * H * (D + R))},
        "hos_wkv_scan": {"prefill": (tokens * C * 4 * 5, 6.0 * tokens * wh * wd * wd),
                         "decode": (batch * wh * wd * wd * 4 * 2, 6.0 * batch * wh * wd * wd)},
        "hos_moe_gate_up": {"prefill": (z["experts"] * 2 * ff * width * 2, 4.0 * tokens * top * real * ff * width),
                            "decode": (touched * 2 * ff * width * 2, 4.0 * batch * top * real * ff * width)},
        "hos_moe_down": {"prefill": (z["experts"] * ff * width * 2, 2.0 * tokens * top * real * ff * width),
                         "decode": (touched * ff * width * 2, 2.0 * batch * top * real * ff * width)},
        "hos_heads_product": {"prefill": (0, 2.0 * tokens * H * R * (z["dim"] + z["vdim"]) / 2),
                              "decode": (H * R * (z["dim"] + z["vdim"]) * 2 / 2, 2.0 * batch * H * R * (z["dim"] + z["vdim"]) / 2)},
    }


# ---- --design vagonex: the Vagonex design beside Gemma-2 at equal size -----------------------------------
# Layers in the order (decay, delta, attention, delta) x blocks; attention with chunks; a dense gated feed-forward.
# Gemma-2 "at equal size": the same width, layer count, vocabulary, heads, head size and intermediate size, its
# window as long as the chunks.
VAGONEX_SIZES = {
    "s": dict(width=1024, vocab=32000, blocks=2, heads=8, kv_heads=2, dim=128, vdim=128, chunk=1024, ff=4096,
              state_heads=8, state_kv=4, state_dim=128, state_vdim=128, conv=4),
    "m": dict(width=2048, vocab=32000, blocks=2, heads=16, kv_heads=4, dim=128, vdim=128, chunk=2048, ff=8192,
              state_heads=16, state_kv=8, state_dim=128, state_vdim=128, conv=4),
    "l": dict(width=4096, vocab=64000, blocks=1, heads=32, kv_heads=8, dim=128, vdim=128, chunk=2048, ff=14336,
              state_heads=32, state_kv=16, state_dim=128, state_vdim=128, conv=4),
}


def vagonex_raw(z):
    mlp = {"kind": "dense", "ff": z["ff"]}
    att = {"type": "attention", "mlp": mlp,
           "mixer": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"],
                     "scale": z["dim"] ** -0.5, "mask": {"size": z["chunk"]},
                     "rot": {"base": 10000.0, "dims": z["dim"] // 2,
                             "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}}
    dec = {"type": "lightning", "mlp": mlp,
           "mixer": {"heads": z["state_heads"], "dim": z["state_dim"], "vdim": z["state_vdim"],
                     "decay": [1.0 - 2.0 ** -(3 + 5 * i / max(1, z["state_heads"] - 1)) for i in range(z["state_heads"])]}}
    dlt = {"type": "delta", "mlp": mlp,
           "mixer": {"heads": z["state_heads"], "kv_heads": z["state_kv"], "dim": z["state_dim"], "vdim": z["state_vdim"],
                     "conv": z["conv"]}}
    return {"architecture": "Vagonex", "vocab": z["vocab"], "width": z["width"], "postln_alpha": 2.0, "norm": {"eps": 1e-6},
            "embedding": {"scale": float(z["width"]) ** 0.5}, "layers": [dec, dlt, att, dlt] * z["blocks"]}


def gemma_raw_like_vagonex(z):
    return dict(architectures=["Gemma2ForCausalLM"], model_type="gemma2", num_hidden_layers=4 * z["blocks"],
                hidden_size=z["width"], num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"],
                head_dim=z["dim"], intermediate_size=z["ff"], vocab_size=z["vocab"], rope_theta=10000.0,
                sliding_window=z["chunk"], max_position_embeddings=8192, query_pre_attn_scalar=z["dim"],
                attn_logit_softcapping=50.0, final_logit_softcapping=30.0, rms_norm_eps=1e-6, tie_word_embeddings=True)


def vagonex_kernel_work(z, tokens, batch, ctx):
    """Per launch of each of the design's own kernels: (bytes that must move, FLOPs of the mathematics) for a prompt of
    `tokens` tokens and for a decode step of `batch` sequences at length `ctx` (bfloat16 cache, 32-bit state and rows)."""
    H, G, kd, vd, C = z["heads"], z["kv_heads"], z["dim"], z["vdim"], z["chunk"]
    pairs = sum(p % C + 1 for p in range(tokens))
    keys = (ctx - 1) % C + 1
    sh, sk, sd, sv = z["state_heads"], z["state_kv"], z["state_dim"], z["state_vdim"]
    cols = 2 * sk * sd + sh * sv                      # the delta rule's q, k, v columns (the decay rule has sh key heads)
    width = z["width"]

    def scan(n, seqs):        # rows in and out, the state in and out; S update and read-out: 4 (decay) to 7 (delta) per cell
        return n * (cols + sh * sv) * 4 + seqs * sh * sd * sv * 4 * 2, 7.0 * n * sh * sd * sv
    attn = {"prefill": (tokens * G * (kd + vd) * 2 + tokens * H * (kd * 4 + vd * 2), 2.0 * pairs * H * (kd + vd)),
            "decode": (batch * keys * G * (kd + vd) * 2, 2.0 * batch * keys * H * (kd + vd))}
    return {
        "hos_gated_attn": attn, "hos_gated_attn_mma": attn, "hos_gated_attn_mma_decode": attn,
        "hos_state_scan": {"prefill": scan(tokens, 1), "decode": scan(batch, batch)},
        "hos_qk_prep": {"prefill": (tokens * (H * kd * 8 + G * (kd + vd) * 6), 0.0),
                        "decode": (batch * (H * kd * 8 + G * (kd + vd) * 6), 0.0)},
        "hos_conv_prep": {"prefill": (tokens * cols * 8, 0.0), "decode": (batch * cols * (8 + 4 * (z["conv"] - 1)), 0.0)},
        "hos_group_norm_gate": {"prefill": (tokens * sh * sv * 10, 0.0), "decode": (batch * sh * sv * 10, 0.0)},
        "hos_scale_add_norm": {"prefill": (tokens * width * 12, 0.0), "decode": (batch * width * 12, 0.0)},
    }


# ---- --design fobilorn: the Fobilorn design beside Gemma-2 at equal size ---------------------------------
# A dense layer first, then layers of routed experts with a shared one; attention with a window that keeps the first
# keys, values blended with the first layer's.  Gemma-2 "at equal size": the same width, layer count, vocabulary, heads,
# head size, an intermediate size equal to what a Fobilorn token uses (top x ff + shared), the same window on its
# windowed layers.
FOBILORN_SIZES = {
    "s": dict(width=1024, vocab=32000, layers=8, heads=8, kv_heads=2, dim=128, vdim=128, window=1024, keep=4,
              dense_ff=4096, experts=8, top=2, ff=1024, shared=2048),
    "m": dict(width=2048, vocab=32000, layers=8, heads=16, kv_heads=4, dim=128, vdim=128, window=1024, keep=4,
              dense_ff=8192, experts=16, top=2, ff=1536, shared=3072),
    "l": dict(width=4096, vocab=64000, layers=4, heads=32, kv_heads=8, dim=128, vdim=128, window=1024, keep=4,
              dense_ff=14336, experts=32, top=4, ff=1024, shared=4096),
}


def fobilorn_raw(z):
    mixer = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
             "mask": {"size": z["window"], "keep_first": z["keep"]}, "v_mix": True}
    moe = {"kind": "moe", "expert": {"ff": z["ff"]}, "router": {"experts": z["experts"], "top": z["top"]},
           "shared": {"ff": z["shared"]}}
    layers = [{"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": z["dense_ff"]}}] + \
             [{"type": "attention", "mixer": mixer, "mlp": moe} for _ in range(z["layers"] - 1)]
    return {"architecture": "Fobilorn", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 10007}}, "layers": layers}


def gemma_raw_like_fobilorn(z):
    return dict(architectures=["Gemma2ForCausalLM"], model_type="gemma2", num_hidden_layers=z["layers"],
                hidden_size=z["width"], num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"],
                head_dim=z["dim"], intermediate_size=z["top"] * z["ff"] + z["shared"], vocab_size=z["vocab"],
                rope_theta=10000.0, sliding_window=z["window"], max_position_embeddings=8192, query_pre_attn_scalar=z["dim"],
                attn_logit_softcapping=50.0, final_logit_softcapping=30.0, rms_norm_eps=1e-6, tie_word_embeddings=True)


def fobilorn_kernel_work(z, tokens, batch, ctx):
    """Per launch of each of the design's own kernels: (bytes that must move, FLOPs of the mathematics) for a prompt of
    `tokens` tokens and for a decode step of `batch` sequences at length `ctx` (bfloat16 cache and products, 32-bit rows)."""
    H, G, kd, vd, W, K = z["heads"], z["kv_heads"], z["dim"], z["vdim"], z["window"], z["keep"]
    seen = lambda p: min(p + 1, W) + min(K, max(0, p + 1 - W))        # keys position p sees
    pairs = sum(seen(p) for p in range(tokens))
    keys = seen(ctx - 1)
    top, ff, width, E = z["top"], z["ff"], z["width"], z["experts"]
    touched = min(E, batch * top)
    attn = {"prefill": (tokens * G * (kd + vd) * 2 + tokens * H * (kd * 4 + vd * 2), 2.0 * pairs * H * (kd + vd)),
            "decode": (batch * keys * G * (kd + vd) * 2, 2.0 * batch * keys * H * (kd + vd))}
    return {
        "hos_gated_attn": attn, "hos_gated_attn_mma": attn, "hos_gated_attn_mma_decode": attn,
        # the fused row in (32-bit), the other layer's values in, queries out (32-bit), keys and values out
        "hos_qk_prep": {"prefill": (tokens * (H * kd * 8 + G * (kd * 6 + vd * 10)), 0.0),
                        "decode": (batch * (H * kd * 8 + G * (kd * 6 + vd * 10)), 0.0)},
        # x in and out (32-bit), two branch outputs in, the normed rows out
        "hos_add_dyt": {"prefill": (tokens * width * 14, 0.0), "decode": (batch * width * 14, 0.0)},
        "hos_moe_gate_up": {"prefill": (E * 2 * ff * width * 2, 4.0 * tokens * top * ff * width),
                            "decode": (touched * 2 * ff * width * 2, 4.0 * batch * top * ff * width)},
        "hos_moe_down": {"prefill": (E * ff * width * 2, 2.0 * tokens * top * ff * width),
                         "decode": (touched * ff * width * 2, 2.0 * batch * top * ff * width)},
        # the few-rows forms of both (a handful of pairs): the weights of the experts that were chosen
        "hos_moe_gate_up_few": {"prefill": (0, 0.0), "decode": (touched * 2 * ff * width * 2, 4.0 * batch * top * ff * width)},
        "hos_moe_down_few": {"prefill": (0, 0.0), "decode": (touched * ff * width * 2, 2.0 * batch * top * ff * width)},
        "hos_moe_combine": {"prefill": (tokens * width * (4 * top + 2 + 4), 0.0), "decode": (batch * width * (4 * top + 2 + 4), 0.0)},
    }


# ---- --design tofodra: the Tofodra design beside Vagonex at equal size -----------------------------------
# Layers in the order (latent attention, retention, differential attention, latent attention that reads the first one's
# cache) x blocks; dense clamped feed-forwards on the first and third of a block, routed experts with a shared one on
# the others.  The closest existing model is Vagonex (layers listed one by one, a decay-rule matrix state, attention
# through the same grouped-query kernels, a layer that reads another layer's cache, a dense gated feed-forward):
# "Vagonex at equal size" has the same width, layer count and vocabulary, a decay-rule layer where Tofodra has retention
# (same heads), attention of as many heads over as many kv heads with keys as wide as both maps together where Tofodra
# has any attention (chunks as long as the window; the fourth layer of a block reads the third's cache), and a dense
# feed-forward as wide as what a Tofodra token uses on average.
TOFODRA_SIZES = {
    "s": dict(width=1024, vocab=32000, blocks=2, lat_heads=8, lat_dim=64, lat_rot=32, lat_vdim=64, rank=256,
              ret_heads=8, ret_dim=128, ret_vdim=128, heads=8, kv_heads=2, dim=64, vdim=128, window=1024, keep=4,
              dense_ff=4096, experts=8, top=2, ff=1024, shared=2048),
    "m": dict(width=2048, vocab=32000, blocks=2, lat_heads=16, lat_dim=64, lat_rot=64, lat_vdim=128, rank=512,
              ret_heads=16, ret_dim=128, ret_vdim=128, heads=16, kv_heads=4, dim=64, vdim=128, window=1024, keep=4,
              dense_ff=8192, experts=16, top=2, ff=1536, shared=3072),
    "l": dict(width=4096, vocab=64000, blocks=1, lat_heads=32, lat_dim=64, lat_rot=64, lat_vdim=128, rank=512,
              ret_heads=32, ret_dim=128, ret_vdim=128, heads=32, kv_heads=8, dim=64, vdim=128, window=2048, keep=4,
              dense_ff=14336, experts=32, top=4, ff=1024, shared=4096),
}


def tofodra_raw(z):
    dense = {"kind": "dense", "ff": z["dense_ff"], "limit": 7.0}
    moe = {"kind": "moe", "expert": {"ff": z["ff"]}, "router": {"experts": z["experts"], "top": z["top"], "scale": 2.0},
           "shared": {"ff": z["shared"]}}
    lat = {"heads": z["lat_heads"], "dim": z["lat_dim"], "rot_dim": z["lat_rot"], "vdim": z["lat_vdim"], "kv_rank": z["rank"],
           "scale": (z["lat_dim"] + z["lat_rot"]) ** -0.5, "rot": {"base": 10000.0, "dims": z["lat_rot"]}}
    ret = {"heads": z["ret_heads"], "dim": z["ret_dim"], "vdim": z["ret_vdim"], "rot": {"base": 10000.0, "dims": z["ret_dim"]},
           "decay": [1.0 - 2.0 ** -(5 + 5 * i / max(1, z["ret_heads"] - 1)) for i in range(z["ret_heads"])]}
    att = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"], "scale": z["dim"] ** -0.5,
           "diff": 0.5, "mask": {"size": z["window"], "keep_first": z["keep"]}}
    layers = []
    for b in range(z["blocks"]):
        layers += [{"type": "latent_attention", "mixer": lat, "mlp": dense}, {"type": "retention", "mixer": ret, "mlp": moe},
                   {"type": "attention", "mixer": att, "mlp": dense},
                   {"type": "latent_attention", "mixer": dict(lat, kv_from=4 * b), "mlp": moe}]
    return {"architecture": "Tofodra", "vocab": z["vocab"], "width": z["width"], "norm": {"eps": 1e-6},
            "embedding": {"scale": float(z["width"]) ** 0.5}, "layers": layers}


def vagonex_raw_like_tofodra(z):
    used = (z["dense_ff"] + z["top"] * z["ff"] + z["shared"]) // 2 // 64 * 64      # what a token uses, averaged over a block
    mlp = {"kind": "dense", "ff": used}
    att = {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": 2 * z["dim"], "vdim": z["vdim"], "scale": (2 * z["dim"]) ** -0.5,
           "mask": {"size": z["window"]}, "rot": {"base": 10000.0, "dims": z["dim"]}}
    dec = {"heads": z["ret_heads"], "dim": z["ret_dim"], "vdim": z["ret_vdim"],
           "decay": [1.0 - 2.0 ** -(5 + 5 * i / max(1, z["ret_heads"] - 1)) for i in range(z["ret_heads"])]}
    layers = []
    for b in range(z["blocks"]):
        layers += [{"type": "attention", "mixer": att, "mlp": mlp}, {"type": "lightning", "mixer": dec, "mlp": mlp},
                   {"type": "attention", "mixer": att, "mlp": mlp},
                   {"type": "attention", "mixer": dict(att, kv_from=4 * b + 2), "mlp": mlp}]
    return {"architecture": "Vagonex", "vocab": z["vocab"], "width": z["width"], "postln_alpha": 2.0, "norm": {"eps": 1e-6},
            "embedding": {"scale": float(z["width"]) ** 0.5}, "layers": layers}


def tofodra_kernel_work(z, tokens, batch, ctx):
    """Per launch of each of the design's own kernels: (bytes that must move, FLOPs of the mathematics) for a prompt of
    `tokens` tokens and for a decode step of `batch` sequences at length `ctx` (bfloat16 cache and products, 32-bit rows
    and states).  The differential attention's mathematics counts both maps' scores over `dim` numbers each; the kernel
    issues them over key rows of 2 x dim."""
    LH, D, R = z["lat_heads"], z["rank"] + z["lat_rot"], z["rank"]
    all_pairs = tokens * (tokens + 1) // 2
    H, G, d, vd, W, K = z["heads"], z["kv_heads"], z["dim"], z["vdim"], z["window"], z["keep"]
    kd = 2 * d
    seen = lambda p: min(p + 1, W) + min(K, max(0, p + 1 - W))        # keys position p sees
    pairs, keys = sum(seen(p) for p in range(tokens)), seen(ctx - 1)
    sh, sd, sv = z["ret_heads"], z["ret_dim"], z["ret_vdim"]
    top, ff, width, E = z["top"], z["ff"], z["width"], z["experts"]
    touched = min(E, batch * top)
    maps = {"prefill": (tokens * G * (kd + vd) * 2 + tokens * 2 * H * (kd * 4 + vd * 4), 2.0 * pairs * 2 * H * (d + vd)),
            "decode": (batch * keys * G * (kd + vd) * 2, 2.0 * batch * keys * 2 * H * (d + vd))}

    def scan(n, seqs):        # q, k, v rows in, o rows out, the state in and out; the update and the read-out: 4 per cell
        return n * (2 * sh * sd + 2 * sh * sv) * 4 + seqs * sh * sd * sv * 4 * 2, 4.0 * n * sh * sd * sv
    return {
        "hos_latent_attn": {"prefill": (tokens * D * 2 + tokens * LH * (D + R) * 4, 2.0 * all_pairs * LH * (D + R)),
                            "decode": (batch * ctx * D * 2, 2.0 * batch * ctx * LH * (D + R))},
        "hos_heads_product": {"prefill": (0, 2.0 * tokens * LH * R * (z["lat_dim"] + z["lat_vdim"]) / 2),
                              "decode": (LH * R * (z["lat_dim"] + z["lat_vdim"]) * 2 / 2,
                                         2.0 * batch * LH * R * (z["lat_dim"] + z["lat_vdim"]) / 2)},
        "hos_state_scan": {"prefill": scan(tokens, 1), "decode": scan(batch, batch)},
        # q and k rows read and written in place (32-bit)
        "hos_rotate_rows": {"prefill": (tokens * 2 * sh * sd * 8, 0.0), "decode": (batch * 2 * sh * sd * 8, 0.0)},
        "hos_group_norm_gate": {"prefill": (tokens * sh * sv * 10, 0.0), "decode": (batch * sh * sv * 10, 0.0)},
        "hos_gated_attn": maps, "hos_gated_attn_mma": maps, "hos_gated_attn_mma_decode": maps,
        # the fused row in (32-bit), the padded queries out (32-bit, both maps), keys and values out
        "hos_qk_prep": {"prefill": (tokens * (H * kd * 4 + 2 * H * kd * 4 + G * (kd + vd) * 6), 0.0),
                        "decode": (batch * (H * kd * 4 + 2 * H * kd * 4 + G * (kd + vd) * 6), 0.0)},
        # both maps' outputs and the gate logits in (32-bit), the gated heads out
        "hos_diff_combine": {"prefill": (tokens * H * vd * (8 + 4 + 2), 0.0), "decode": (batch * H * vd * (8 + 4 + 2), 0.0)},
        "hos_clamped_gated_act": {"prefill": (tokens * z["dense_ff"] * (8 + 2), 0.0), "decode": (batch * z["dense_ff"] * (8 + 2), 0.0)},
        # x in and out (32-bit), the branch's output in, the normed rows out
        "hos_norm_add_norm": {"prefill": (tokens * width * 12, 0.0), "decode": (batch * width * 12, 0.0)},
        "hos_moe_gate_up": {"prefill": (E * 2 * ff * width * 2, 4.0 * tokens * top * ff * width),
                            "decode": (touched * 2 * ff * width * 2, 4.0 * batch * top * ff * width)},
        "hos_moe_down": {"prefill": (E * ff * width * 2, 2.0 * tokens * top * ff * width),
                         "decode": (touched * ff * width * 2, 2.0 * batch * top * ff * width)},
        "hos_moe_gate_up_few": {"prefill": (0, 0.0), "decode": (touched * 2 * ff * width * 2, 4.0 * batch * top * ff * width)},
        "hos_moe_down_few": {"prefill": (0, 0.0), "decode": (touched * ff * width * 2, 2.0 * batch * top * ff * width)},
        "hos_moe_combine": {"prefill": (tokens * width * (4 * top + 2 + 4), 0.0), "decode": (batch * width * (4 * top + 2 + 4), 0.0)},
    }


DESIGNS = {"fobilorn": lambda: (FOBILORN_SIZES, fobilorn_raw, gemma_raw_like_fobilorn, fobilorn_kernel_work,
                                ("hos_gated_attn",)),
           "satapel": lambda: (SATAPEL_SIZES, satapel_raw, gemma_raw_like, satapel_kernel_work, ("hos_wkv_scan",)),
           "vagonex": lambda: (VAGONEX_SIZES, vagonex_raw, gemma_raw_like_vagonex, vagonex_kernel_work,
                               ("hos_state_scan", "hos_gated_attn")),
           "tofodra": lambda: (TOFODRA_SIZES, tofodra_raw, vagonex_raw_like_tofodra, tofodra_kernel_work,
                               ("hos_state_scan", "hos_gated_attn"))}


def _vagonex_work_like_tofodra(z, tokens, batch, ctx):
    """The compared model's kernels at the equal-size configuration: attention over keys of 2 x dim numbers in chunks as
    long as the window, the decay-rule scan of as many heads."""
    H, G, kd, vd, C = z["heads"], z["kv_heads"], 2 * z["dim"], z["vdim"], z["window"]
    pairs, keys = sum(p % C + 1 for p in range(tokens)), (ctx - 1) % C + 1
    sh, sd, sv = z["ret_heads"], z["ret_dim"], z["ret_vdim"]
    attn = {"prefill": (tokens * G * (kd + vd) * 2 + tokens * H * (kd * 4 + vd * 2), 2.0 * pairs * H * (kd + vd)),
            "decode": (batch * keys * G * (kd + vd) * 2, 2.0 * batch * keys * H * (kd + vd))}

    def scan(n, seqs):
        return n * (2 * sh * sd + 2 * sh * sv) * 4 + seqs * sh * sd * sv * 4 * 2, 4.0 * n * sh * sd * sv
    return {"hos_gated_attn": attn, "hos_gated_attn_mma": attn, "hos_gated_attn_mma_decode": attn,
            "hos_state_scan": {"prefill": scan(tokens, 1), "decode": scan(batch, batch)},
            "hos_qk_prep": {"prefill": (tokens * (H * kd * 8 + G * (kd + vd) * 6), 0.0),
                            "decode": (batch * (H * kd * 8 + G * (kd + vd) * 6), 0.0)},
            "hos_group_norm_gate": {"prefill": (tokens * sh * sv * 10, 0.0), "decode": (batch * sh * sv * 10, 0.0)},
            "hos_scale_add_norm": {"prefill": (tokens * z["width"] * 12, 0.0), "decode": (batch * z["width"] * 12, 0.0)}}


OTHER_WORK = {"tofodra": _vagonex_work_like_tofodra}
OTHER_ARM = {"tofodra": "vagonex_equal_size"}      # the closest existing model per design (Gemma-2 where none is named)


def run_design_profile_step(args) -> int:
    """For a profiler: one block of the design's layers (4 layers at the first of --sizes), two steps of the asked kind
    launched kernel by kernel (no CUDA graph): a prompt of --prefill-tokens tokens, or a single-token step of the last
    of --batches sequences that hold --ctx tokens.  Holds about 1 GB on the device.  Prints "ok"."""
    import random
    import torch
    from hos_b200 import Engine
    from hos_b200.registry import config_from_dict
    sizes, raw_of, _, _, _ = DESIGNS[args.design]()
    z = dict(sizes[args.sizes.split(",")[0]], blocks=1)
    if args.arm == "other":
        raw_of = DESIGNS[args.design]()[2]
    if "layers" in z:
        z["layers"] = min(4, z["layers"])
    b = int(args.batches.split(",")[-1])
    ctx = args.ctx if args.ctx != 8192 else 1024
    eng = Engine.from_config(config_from_dict(raw_of(z)), seed=0, dtype="bfloat16", max_batch=b,
                             max_tokens=b * (ctx + 64) + args.prefill_tokens + 64, max_seq_len=max(ctx, args.prefill_tokens) + 64)
    r, rng = eng.runner, random.Random(0)
    r.use_sessions = False
    if args.profile == "prefill":
        for _ in range(2):
            s = r.admit(1)
            r.step(s, [[rng.randrange(r.vocab_size) for _ in range(args.prefill_tokens)]])
            r.release(s[0])
    else:
        s = r.admit(b)
        r.cache.extend_all(s, [ctx - 2] * b)
        r.write_records(s, pos=[ctx - 2] * b)
        for _ in range(2):
            r.step(s, [[rng.randrange(r.vocab_size)] for _ in range(b)])
    torch.cuda.synchronize()
    print("ok")
    return 0


def run_design_comparison(args) -> int:
    """Prompt and decode throughput of Satapel beside Gemma-2 at equal size, and where each of the design's own
    kernels stands against its roofline: the larger of (bytes over the measured copy rate) and (the FLOPs of the
    mathematics over the measured bfloat16 tensor rate; for the recurrence, which is 32-bit FMA work, over the FMA
    pipes' rate).  The attention kernel issues twice its mathematics' FLOPs (two bfloat16 terms per 32-bit operand);
    the fraction counts the mathematics only.  The Vagonex attention and scans are 32-bit FMA work and are held to the
    FMA pipes' rate.  One JSON line per size."""
    import random
    import torch
    from hos_b200 import Engine, ops
    from hos_b200.registry import config_from_dict
    pk, pk_src = peaks()
    rng = random.Random(0)
    tokens, ctx = args.prefill_tokens, args.ctx if args.ctx != 8192 else 2048
    sizes, raw_of, gemma_of, work_of, fma_kernels = DESIGNS[args.design]()
    for name in args.sizes.split(","):
        z = sizes[name]
        line = {"design": args.design, "size": name, "sizes": z, "prompt_tokens": tokens, "decode_ctx": ctx, "peaks": pk_src,
                "dtype": "bf16", "data": "synthetic (random weights)"}
        for which, raw in ((args.design, raw_of(z)), (OTHER_ARM.get(args.design, "gemma2_equal_size"), gemma_of(z))):
            cfg = config_from_dict(raw)
            batches = [int(b) for b in args.batches.split(",")]
            eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_batch=max(batches),
                                     max_tokens=max(batches) * (ctx + 64) + tokens + 64, max_seq_len=max(ctx, tokens) + 64)
            r = eng.runner
            out = {"prefill_ms": measure_prefill(eng, tokens, rng)}
            out["prefill_tok_s"] = tokens * 1e3 / out["prefill_ms"]
            for b in batches:
                slots = r.admit(b)
                r.cache.extend_all(slots, [ctx - args.steps - args.warmup] * b)
                ms, launches = r.decode_steps_timed(slots, [[rng.randrange(r.vocab_size)] for _ in range(b)], args.warmup, args.steps)
                for s in slots:
                    r.release(s)
                out[f"decode_b{b}_ms"] = ms
                out[f"decode_b{b}_tok_s"] = b * 1e3 / ms
                out[f"decode_b{b}_launches"] = launches
            # per kernel: one prompt and one decode step launched kernel by kernel, every call between two events
            r.use_sessions = False
            b = batches[-1]
            kern = {}
            for phase in ("prefill", "decode"):
                slots = r.admit(1 if phase == "prefill" else b)
                if phase == "decode":
                    r.cache.extend_all(slots, [ctx - 2] * b)
                    r.write_records(slots, pos=[ctx - 2] * b)
                    feed = [[rng.randrange(r.vocab_size)] for _ in range(b)]
                else:
                    feed = [[rng.randrange(r.vocab_size) for _ in range(tokens)]]
                r.step(slots, feed)                          # warm-up of this shape
                if phase == "decode":
                    ops.time_calls(True)
                    r.step(slots, [[t[0]] for t in feed])
                else:
                    for s in slots:
                        r.release(s)
                    slots = r.admit(1)
                    ops.time_calls(True)
                    r.step(slots, feed)
                times = ops.call_times()
                ops.time_calls(False)
                for s in slots:
                    r.release(s)
                work = work_of(z, tokens, b, ctx) if which == args.design else \
                    (OTHER_WORK[args.design](z, tokens, b, ctx) if args.design in OTHER_WORK else {})
                rows = {}
                for fn, (n, ms) in sorted(times.items(), key=lambda kv: -kv[1][1]):
                    row = {"calls": n, "ms": round(ms, 4)}
                    if fn in work:
                        by, fl = work[fn][phase]
                        tensor = fn not in fma_kernels       # bfloat16 products and the latent attention: tensor cores
                        t_mem = by / (pk["hbm_gbs"] * 1e9)
                        t_fl = fl / ((pk["bf16_tflops"] if tensor else FP32_TFLOPS) * 1e12)
                        row["roofline_us_per_call"] = round(max(t_mem, t_fl) * 1e6, 2)
                        row["bound"] = "hbm" if t_mem >= t_fl else ("bf16 tensor" if tensor else "fp32")
                        row["frac"] = round(max(t_mem, t_fl) * 1e3 / (ms / n), 4)
                    rows[fn] = row
                kern[phase] = rows
            out["kernels"] = kern
            line[which] = out
            del eng, r
            torch.cuda.empty_cache()
        print(json.dumps(line), flush=True)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the configuration has, for a quick run")
    ap.add_argument("--model", default="2b", choices=sorted(MODELS), help="layer sizes (default: Gemma-2 2B)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--workload", default="step", choices=["step", "baseline"],
                    help="step: the decode step at the context's end (the default line); baseline: prompts then 256 "
                         "greedy tokens, the workload that goes with the model's sizes")
    ap.add_argument("--decode-tokens", type=int, default=256, help="tokens decoded per sequence by --workload baseline")
    ap.add_argument("--mixed-lengths", action="store_true",
                    help="the sequences end at 1, 1/2, 1/4, 1/8, 1/16, 1/16, 1/32, 1/32 of the context, in turn, "
                         "instead of all at its end (not the driver's line: how a batch of unequal lengths decodes)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="length of the timed prompt (default: 2,048)")
    ap.add_argument("--design", default=None, choices=sorted(DESIGNS),
                    help="not the driver's line: prompt and decode throughput of this design beside Gemma-2 at equal "
                         "size, with its kernels against their rooflines (--sizes, --batches, --ctx, --prefill-tokens)")
    ap.add_argument("--profile", default=None, choices=["prefill", "decode"],
                    help="with --design: no measurement, just two steps of that kind of one block of layers, kernel by "
                         "kernel, for a profiler to capture")
    ap.add_argument("--sizes", default="s,m", help="with --design: which of the sizes s, m, l")
    ap.add_argument("--arm", default="design", choices=["design", "other"],
                    help="with --design and --profile: the design itself, or the model it is compared with")
    ap.add_argument("--batches", default="1,8,64", help="with --design: decode batch sizes")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust crate: no cargo/rustc in this image and no network "
                          "to fetch its 38 crates; it also runs Gemma-2 on the CPU only"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU only: this library runs on a single GPU, --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.design and args.profile:
        return run_design_profile_step(args)
    if args.design:
        return run_design_comparison(args)
    if args.workload == "baseline":
        return run_baseline_workload(args)

    import random
    import torch
    from hos_b200 import Engine
    from hos_b200 import models  # noqa: F401
    from hos_b200.registry import config_from_dict

    full_layers = MODELS[args.model]["num_hidden_layers"]
    if args.layers is None:
        args.layers = full_layers
    raw = dict(MODELS[args.model], num_hidden_layers=args.layers)
    cfg = config_from_dict(raw)
    pk, pk_src = peaks()
    rng = random.Random(0)
    batches = [args.batch] + ([] if args.no_points else [1, 64])
    cap_tokens = max(batches) * ((args.ctx + 63) // 64 * 64)
    eng = Engine.from_config(cfg, seed=0, dtype="bfloat16", max_batch=max(batches), max_tokens=cap_tokens,
                             max_seq_len=args.ctx)
    fill_cache_random(eng.runner)
    torch.cuda.synchronize()

    clocks = ClockSampler(torch.cuda.current_device())
    ms_dev, ms_e2e, launches, h2d, d2h, mean_len = measure_decode(
        eng, args.batch, args.ctx, args.steps, args.warmup, rng, clocks, mixed=args.mixed_lengths)
    clock_rec = clocks.result

    wbytes = weight_bytes(cfg, args.layers)
    if args.mixed_lengths:
        step_bytes = wbytes + sum(kv_bytes_at(cfg, args.layers, int(n)) for n in mean_len)
    else:
        step_bytes = wbytes + args.batch * kv_bytes_at(cfg, args.layers, int(mean_len))
    achieved = step_bytes / (ms_dev * 1e-3) / 1e9
    line = {
        "metric": "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Gemma-2 2B)",
        "value": args.batch * 1e3 / ms_dev, "unit": "tok/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_dev, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": {
            "model": f"gemma-2-{args.model} sizes, random weights", "global_batch": args.batch, "seq_len": args.ctx,
            "parallelism": "single_gpu", "layers": args.layers, "layers_full": full_layers,
            "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "sliding_window": cfg.sliding_window,
            "decode_ends_at": "1, 1/2, 1/4, 1/8, 1/16, 1/16, 1/32, 1/32 of %d in turn" % args.ctx if args.mixed_lengths else args.ctx,
            "cache_fill": "random keys and values", "l2": "inputs larger than L2 (weights %.1f GB per step)" % (wbytes / 1e9),
            "peaks": pk_src, "prefill_tokens": args.prefill_tokens},
        "clocks": clock_rec,
        "e2e": {"value": args.batch * 1e3 / ms_e2e, "unit": "tok/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "bytes_per_step": step_bytes, "of": pk_src},
    }
    if not args.no_prefill:
        ms = measure_prefill(eng, args.prefill_tokens, rng)
        fl = prefill_flops(cfg, args.layers, args.prefill_tokens)
        line["prefill"] = {"value": args.prefill_tokens * 1e3 / ms, "tokens": args.prefill_tokens, "ms": ms,
                           "frac": fl / (ms * 1e-3) / (pk["bf16_tflops"] * 1e12), "tflop": fl / 1e12,
                           "peak_tflops": pk["bf16_tflops"], "of": pk_src}
        if args.prefill_tokens % 4 == 0:       # the same prompt as four steps that continue one another
            line["prefill"]["ms_in_4_pieces"] = measure_prefill(eng, args.prefill_tokens, rng, pieces=4)
    if not args.no_points:
        pts, pts_e2e = {}, {f"decode_b{args.batch}": line["e2e"]["value"]}
        for b in (1, 64):
            m, me, _, _, _, _ = measure_decode(eng, b, args.ctx, args.steps, args.warmup, rng)
            pts[f"decode_b{b}"] = b * 1e3 / m
            pts_e2e[f"decode_b{b}"] = b * 1e3 / me
        line["points"] = pts
        line["points_e2e"] = pts_e2e
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
