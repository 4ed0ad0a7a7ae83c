"""Fobilorn on the GPU against the plain oracle (tests/plain/fobilorn_plain.py): every mechanism alone, whole prompts,
decoding through the cache, prompts in pieces, batches against each request alone, reuse of slots and pages, the
edges of windows, kept keys and pages, the first tokens, far keys and the one in the denominator, long decoding,
other sizes, and generation through the engine, the replay program and the command line."""
import copy
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from fobilorn_cases import CASES, assert_rows, attention, make_folder, model, moe, oracle_view, row_errors, tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("fobilorn")
    return {k: make_folder(base, raw, seed, k) for k, (raw, seed) in CASES.items()}


def _runner(folder, dtype, **kw):
    from hos_b200.engine import Runner
    kw.setdefault("max_tokens", 4096)
    kw.setdefault("max_seq_len", 1024)
    return Runner.from_folder(folder, dtype=dtype, **kw)


def _oracle(folder, seqs):
    from plain import fobilorn_plain as P
    cfg, w = oracle_view(folder)
    return [P.forward(cfg, w, s) for s in seqs]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C", "D"])
def test_whole_prompts_of_unequal_lengths(folders, case, dtype):
    vocab = CASES[case][0]["vocab"]
    seqs = [tokens(i, n, vocab) for i, n in enumerate((1, 2, 37, 150))]      # 150: beyond two pages and every window
    want = _oracle(folders[case], seqs)
    r = _runner(folders[case], dtype)
    slots = r.admit(len(seqs))
    got = r.step(slots, seqs, [list(range(len(s))) for s in seqs]).cpu()
    assert_rows(got, torch.cat(want), dtype, f"case {case}")
    for s in slots:
        r.release(s)
    r.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "B", "C", "D"])
def test_a_prompt_then_token_by_token(folders, case, dtype):
    """Two requests decoded side by side through the replayed single-token step, across page borders (64, 128), every
    window's edge and the end of every kept run; the shorter one leaves first.  The longer one is decoded for 141
    steps, so every window passes wholly over decoded tokens."""
    vocab = CASES[case][0]["vocab"]
    seqs = [tokens(20, 150, vocab), tokens(21, 90, vocab)]
    plens = [9, 61]
    want = _oracle(folders[case], seqs)
    r = _runner(folders[case], dtype)
    slots = r.admit(2)
    first = r.step(slots, [s[:n] for s, n in zip(seqs, plens)]).cpu()
    got = [[first[0:1]], [first[1:2]]]
    pos, live = list(plens), [0, 1]
    while live:
        out = r.step([slots[i] for i in live], [[seqs[i][pos[i]]] for i in live]).cpu()
        for j, i in enumerate(live):
            got[i].append(out[j:j + 1])
            pos[i] += 1
        for i in [i for i in live if pos[i] == len(seqs[i])]:
            r.release(slots[i])
        live = [i for i in live if pos[i] < len(seqs[i])]
    for i in range(2):
        assert_rows(torch.cat(got[i]), want[i][plens[i] - 1:], dtype, f"case {case} request {i}")
    r.cache.check()


@pytest.mark.parametrize("case, dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("C", "float32"), ("D", "bfloat16")])
def test_a_prompt_in_pieces_of_many_sizes(folders, case, dtype):
    """Pieces down to two tokens and one, pieces that end on a page's border and one past it: the pair table's row
    needs the token before the piece, the blended values are those of the piece's own tokens."""
    vocab = CASES[case][0]["vocab"]
    seq = tokens(30, 230, vocab)
    want = _oracle(folders[case], [seq])[0]
    r = _runner(folders[case], dtype)
    (slot,) = r.admit(1)
    at, got = 0, []
    for k in [2, 3, 59, 1, 65, 7, 2, 40, 1, 1, 30, 19]:
        piece = seq[at:at + k]
        got.append(r.step([slot], [piece], [list(range(len(piece)))]).cpu())
        at += len(piece)
    assert at == len(seq)
    assert_rows(torch.cat(got), want, dtype, f"case {case}")
    r.release(slot)
    r.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["A", "C"])
def test_a_batch_gives_what_each_request_gives_alone(folders, case, dtype):
    """Also a step in which one request starts while others go on by one token and by several."""
    vocab = CASES[case][0]["vocab"]
    seqs = [tokens(40 + i, n, vocab) for i, n in enumerate((75, 3, 130))]
    r = _runner(folders[case], dtype)
    alone = []
    for s in seqs:
        (slot,) = r.admit(1)
        alone.append(r.step([slot], [s], [list(range(len(s)))]).cpu())
        r.release(slot)
    slots = r.admit(3)
    both = r.step(slots, seqs, [list(range(len(s))) for s in seqs]).cpu()
    for s in slots:
        r.release(s)
    tol = 2e-5 if dtype == "float32" else 4e-2      # no row shares a sum with another: in practice they are equal
    assert float(row_errors(both, torch.cat(alone)).max()) <= tol
    slots = r.admit(2)
    r.step(slots, [seqs[0][:74], seqs[2][:100]])
    (late,) = r.admit(1)
    mixed = r.step([late, slots[1], slots[0]], [seqs[1], seqs[2][100:109], seqs[0][74:75]],
                   [[0, 1, 2], list(range(9)), [0]]).cpu()
    ref = torch.cat([alone[1], alone[2][100:109], alone[0][74:75]])
    assert float(row_errors(mixed, ref).max()) <= tol
    r.cache.check()


def test_slots_pages_and_state_that_are_freed_are_used_again(folders):
    """What a freed slot's pages and its kept previous token still hold must never be read: they are overwritten
    before the slot is taken again."""
    vocab = CASES["A"][0]["vocab"]
    first, second = tokens(50, 140, vocab), tokens(51, 100, vocab)
    want = _oracle(folders["A"], [second])[0]
    r = _runner(folders["A"], "float32", max_tokens=256)       # four pages: the second request must reuse them
    (slot,) = r.admit(1)
    r.step([slot], [first[:130]])
    for t in first[130:]:
        r.step([slot], [[t]])
    r.release(slot)
    for g in r.cache.groups:
        for t in g.k + g.v:
            t.fill_(1e4)
    for t in r.cache.state_tensors():
        t.fill_(77)
    (again,) = r.admit(1)
    assert again == slot
    got = [r.step([again], [second[:70]], [list(range(70))]).cpu()]
    for t in second[70:]:
        got.append(r.step([again], [[t]]).cpu())
    assert_rows(torch.cat(got), want, "float32", "second request in a used slot")
    r.release(again)
    # a request that starts with single tokens in a used slot: its first token takes the pair table's last row
    for t in r.cache.state_tensors():
        t.fill_(77)
    (again,) = r.admit(1)
    got = [r.step([again], [[t]]).cpu() for t in second[:12]]
    assert_rows(torch.cat(got), want[:12], "float32", "token by token from the first in a used slot")
    r.release(again)
    r.cache.check()


@pytest.mark.parametrize("case", ["A", "B", "C", "D"])
def test_the_edges_of_every_window_in_prompts_and_in_decoding(folders, case):
    """The oracle with every window one key longer or shorter, or with one kept key more or fewer, is far from the
    oracle itself (so an edge that is off by one cannot pass), and the library agrees with the oracle at every
    position, whether the token comes in a prompt or alone."""
    from plain import fobilorn_plain as P
    raw = CASES[case][0]
    cfg, w = oracle_view(folders[case])
    seq = tokens(60, 160, raw["vocab"])
    want = P.forward(cfg, w, seq)
    for key, d in (("size", 1), ("size", -1), ("keep_first", 1), ("keep_first", -1)):
        def edit(m):
            if m.get("mask") and m["mask"].get(key, 0) + d > 0:
                m["mask"] = dict(m["mask"], **{key: m["mask"].get(key, 0) + d})
            return m
        # one key more or fewer among up to 140: at least ten times what the 32-bit comparison below allows
        assert float(row_errors(P.forward(cfg, w, seq, edit=edit)[140:], want[140:]).median()) > 2e-4, \
            f"the test would not see {key} off by {d}"
    r = _runner(folders[case], "float32")
    (slot,) = r.admit(1)
    assert_rows(r.step([slot], [seq], [list(range(len(seq)))]).cpu(), want, "float32", "in a prompt")
    r.release(slot)
    (slot,) = r.admit(1)
    r.step([slot], [seq[:5]])
    got = [r.step([slot], [[t]]).cpu() for t in seq[5:]]
    assert_rows(torch.cat(got), want[5:], "float32", "decoded alone")
    r.release(slot)


def test_far_keys_kept_keys_and_the_one_in_the_denominator(tmp_path):
    """Two layers with soft scores: one sees all keys, one has a short window and keeps the sequence's first five
    keys.  Without the keys that lie more than 600 tokens back, without the kept keys (at a distance of 600 and more),
    or without the one in the denominator the oracle's logits move by far more than the tolerance.  In decoding a
    row's keys are cut into shares that are merged (more than 256 keys)."""
    from plain import fobilorn_plain as P
    raw = model(48, 60, [attention(2, 1, 8, 12, 0.15, mlp=None), attention(4, 2, 8, 12, 0.3, window=9, keep=5, mlp=None)],
                bigram=(7, 3, 2))
    folder = make_folder(tmp_path, raw, 5, "far")
    cfg, w = oracle_view(folder)
    seq = tokens(70, 640, 60)
    want = P.forward(cfg, w, seq)
    assert float(row_errors(P.forward(cfg, w, seq, sink=False), want).median()) > 2e-3

    def no_far(m):
        return dict(m, mask={"size": 600}) if not m.get("mask") else m

    def no_kept(m):
        return dict(m, mask={"size": m["mask"]["size"]}) if m.get("mask") else m
    assert float(row_errors(P.forward(cfg, w, seq, edit=no_far)[610:], want[610:]).median()) > 1e-4
    assert float(row_errors(P.forward(cfg, w, seq, edit=no_kept)[610:], want[610:]).median()) > 2e-3
    for dtype in ("float32", "bfloat16"):
        r = _runner(folder, dtype)
        (slot,) = r.admit(1)
        got = [r.step([slot], [seq[:600]], [list(range(600))]).cpu()] + [r.step([slot], [[t]]).cpu() for t in seq[600:]]
        assert_rows(torch.cat(got), want, dtype, "far keys and kept keys")
        r.release(slot)


def test_every_layer_alone(folders):
    """The residual stream after the embedding (both tables and the norm) and after every layer, in 32-bit, for a
    prompt; then the same for the prompt's second half fed after its first (every mixer resumes from its cache, the
    pair table from the kept token)."""
    from plain import fobilorn_plain as P
    for case in ("A", "B", "C", "D"):
        cfg, w = oracle_view(folders[case])
        seq = tokens(80, 90, cfg["vocab"])
        want = []
        P.forward(cfg, w, seq, taps=want)
        r = _runner(folders[case], "float32")
        (slot,) = r.admit(1)
        taps = r.hidden_states([slot], [seq])
        assert len(taps) == len(want)
        for i, (g, x) in enumerate(zip(taps, want)):
            assert float(row_errors(g.cpu(), x).max()) < 1e-5, f"case {case}: after {i} layers"
        r.release(slot)
        (slot,) = r.admit(1)
        r.step([slot], [seq[:47]])
        taps = r.hidden_states([slot], [seq[47:]])
        for i, (g, x) in enumerate(zip(taps, want)):
            assert float(row_errors(g.cpu(), x[47:]).max()) < 1e-5, f"case {case}: after {i} layers, second half"
        r.release(slot)


SINGLE = {
    "keys wider than values, all keys in sight": attention(3, 3, 40, 8, 0.3, mlp=None),
    "heads of 200 and 264 numbers": attention(2, 1, 200, 264, 0.1, window=50, keep=3, mlp=None),
    "twenty query heads to a kv head": attention(20, 1, 8, 8, 0.5, window=100, keep=1, mlp=None),
    "one head of one number, values of three": attention(1, 1, 1, 3, 0.9, window=2, keep=2, mlp=None),
    "kept keys beyond the prompt": attention(4, 2, 16, 16, 0.5, window=3, keep=120, mlp=None),
    "a dense feed-forward alone matters": attention(1, 1, 8, 8, 0.2, window=4),
    "every expert chosen, no shared one": attention(2, 2, 8, 8, 0.4, mlp=moe(4, 4, 24)),
    "one expert of one": attention(2, 1, 8, 8, 0.4, window=30, keep=2, mlp=moe(1, 1, 40, shared=8)),
    "forty experts, six chosen": attention(2, 1, 8, 8, 0.4, mlp=moe(40, 6, 8, shared=72)),
    "experts wider than the model": attention(2, 1, 8, 8, 0.4, mlp=moe(3, 2, 136, shared=264)),
}


@pytest.mark.parametrize("name", list(SINGLE))
def test_one_layer_models_of_other_sizes(tmp_path, name):
    """Sizes that the kernels' shapes switch on, each as a model of one layer: a prompt, then pieces of one to five
    tokens, in 32-bit."""
    raw = model(40, 50, [SINGLE[name]], ff=16, bigram=(11, 2, 9))
    folder = make_folder(tmp_path, raw, 31, "one")
    seq = tokens(33, 150, 50)
    want = _oracle(folder, [seq])[0]
    r = _runner(folder, "float32")
    (slot,) = r.admit(1)
    got, at = [r.step([slot], [seq[:101]], [list(range(101))]).cpu()], 101
    for k in [1, 1, 2, 5, 1, 3, 1, 1, 4, 30]:
        got.append(r.step([slot], [seq[at:at + k]], [list(range(k))]).cpu())
        at += k
    assert at == len(seq)
    assert_rows(torch.cat(got), want, "float32", name)
    r.release(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wider_layers_and_a_longer_prompt(folders, dtype):
    """A prompt of 700 tokens (a window of 300 that keeps 70: decoding rows see more than 256 keys and are cut into
    shares), a piece of 90, then single tokens beside a second request that starts later.  At these widths and lengths
    the 32-bit rounding noise is larger: every row within 1e-4 of the logits' size and the median within 2e-5."""
    vocab = CASES["E"][0]["vocab"]
    seqs = [tokens(140, 820, vocab), tokens(141, 75, vocab)]
    want = _oracle(folders["E"], seqs)
    r = _runner(folders["E"], dtype, max_seq_len=2048)
    a, b = r.admit(2)
    probe = list(range(0, 700, 7))
    got = [r.step([a], [seqs[0][:700]], [probe]).cpu(), r.step([a], [seqs[0][700:790]], [list(range(90))]).cpu()]
    out = r.step([b, a], [seqs[1][:60], seqs[0][790:791]], [[59], [0]]).cpu()
    got.append(out[1:2])
    got_b = [out[0:1]]
    for k in range(15):
        out = r.step([a, b], [[seqs[0][791 + k]], [seqs[1][60 + k]]]).cpu()
        got.append(out[0:1])
        got_b.append(out[1:2])
    for k in range(15, 29):
        got.append(r.step([a], [[seqs[0][791 + k]]]).cpu())
    pairs = ((torch.cat(got), torch.cat([want[0][probe], want[0][700:820]])), (torch.cat(got_b), want[1][59:75]))
    for g, x in pairs:
        e = row_errors(g, x)
        if dtype == "float32":
            assert float(e.median()) <= 2e-5 and float(e.max()) <= 1e-4, f"median {float(e.median()):.2e}, worst {float(e.max()):.2e}"
        else:
            assert_rows(g, x, dtype, "wider layers")
    r.release(a)
    r.release(b)
    r.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_at_the_tensor_core_kernels_sizes(folders, dtype):
    """Requests of one and two tokens at head sizes that the tensor-core kernels take: a single token at position 0,
    two short prompts side by side, then both decoded, then a prompt of nine tokens beside them."""
    vocab = CASES["E"][0]["vocab"]
    seqs = [tokens(150, 12, vocab), tokens(151, 14, vocab), tokens(152, 9, vocab)]
    want = _oracle(folders["E"], seqs)
    r = _runner(folders["E"], dtype)
    (a,) = r.admit(1)
    got_a = [r.step([a], [seqs[0][:1]]).cpu()]
    (b,) = r.admit(1)
    out = r.step([b, a], [seqs[1][:2], seqs[0][1:3]], [[0, 1], [0, 1]]).cpu()
    got_b, got_a = [out[:2]], got_a + [out[2:]]
    for k in range(9):
        out = r.step([a, b], [[seqs[0][3 + k]], [seqs[1][2 + k]]]).cpu()
        got_a.append(out[0:1])
        got_b.append(out[1:2])
    (c,) = r.admit(1)
    out = r.step([c, b], [seqs[2], seqs[1][11:14]], [list(range(9)), [0, 1, 2]]).cpu()
    got_b.append(out[9:])
    for g, x in ((torch.cat(got_a), want[0]), (torch.cat(got_b), want[1]), (out[:9], want[2])):
        if dtype == "float32":
            e = row_errors(g, x)
            assert float(e.max()) <= 1e-4, f"worst {float(e.max()):.2e}"
        else:
            assert_rows(g, x, dtype, "first tokens")
    for s_ in (a, b, c):
        r.release(s_)
    r.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(folders, dtype):
    """The public entry point and its scheduler: more prompts than run side by side, unequal lengths."""
    from plain import fobilorn_plain as P
    from hos_b200 import Engine
    cfg, w = oracle_view(folders["A"])
    prompts = [tokens(100 + i, n, cfg["vocab"]) for i, n in enumerate((5, 70, 1))]
    eng = Engine(folders["A"], dtype=dtype, max_batch=2, max_seq_len=256)
    got = eng.generate_ids(prompts, 10, stop_ids=[])
    for p, g in zip(prompts, got):
        assert len(g) == 10
        seq = list(p)
        for t in g if dtype == "float32" else g[:4]:
            l = P.forward(cfg, w, seq)[-1]
            if dtype == "float32":
                assert float(l.max() - l[t]) < 1e-3, "the chosen token is not the oracle's best"
            else:
                assert float(l.max() - l[t]) < 0.25, "bfloat16 chose a token far from the best"
            seq.append(t)
    eng.runner.cache.check()


def test_the_replay_program_on_a_model_folder(folders, tmp_path):
    vocab = CASES["B"][0]["vocab"]
    seqs = {"x": tokens(110, 80, vocab), "y": tokens(111, 30, vocab), "z": tokens(112, 1, vocab)}
    want = dict(zip(seqs, _oracle(folders["B"], list(seqs.values()))))
    steps, rows = [], {}
    steps.append({"step": 0, "entries": [{"id": "z", "tokens": seqs["z"], "want": [0]}], "end": ["z"]})
    rows[0] = [("z", 0)]
    steps.append({"step": 1, "entries": [{"id": "x", "tokens": seqs["x"][:70], "want": [0, 69]},
                                         {"id": "y", "tokens": seqs["y"][:25], "want": []}], "end": []})
    rows[1] = [("x", 0), ("x", 69)]
    for k in range(10):
        ents = [{"id": "x", "tokens": [seqs["x"][70 + k]], "want": [0]}]
        rws = [("x", 70 + k)]
        if k < 5:
            ents.append({"id": "y", "tokens": [seqs["y"][25 + k]], "want": [0] if k % 2 else []})
            if k % 2:
                rws.append(("y", 25 + k))
        steps.append({"step": 2 + k, "entries": ents, "end": (["y"] if k == 4 else []) + (["x"] if k == 9 else [])})
        rows[2 + k] = rws
    for dtype in ("float32", "bfloat16"):
        out = str(tmp_path / ("out_" + dtype))
        p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folders["B"], "--dtype", dtype, "--out", out,
                            "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps).encode(),
                           stdout=subprocess.PIPE, stderr=subprocess.PIPE, timeout=900)
        assert p.returncode == 0, p.stderr.decode()[-2000:]
        assert [l for l in p.stdout.decode().splitlines() if l.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
        got, ref = [], []
        for n, rws in rows.items():
            got.append(torch.from_numpy(np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(len(rws), vocab).copy()))
            ref.append(torch.stack([want[i][pos] for i, pos in rws]))
        assert_rows(torch.cat(got), torch.cat(ref), dtype, "replayed steps")


def test_generation_through_the_command_line(folders):
    from plain import fobilorn_plain as P
    cfg, w = oracle_view(folders["C"])
    prompt = tokens(120, 6, cfg["vocab"])
    p = subprocess.run([os.path.join(ROOT, "bin", "hos"), "-m", folders["C"], "--fp32", "--repeat-penalty", "1.0", "-n", "5",
                        "-p", ",".join(map(str, prompt))], stdout=subprocess.PIPE, stderr=subprocess.PIPE, timeout=900)
    assert p.returncode == 0, p.stderr.decode()[-2000:]
    ids = [int(t) for t in p.stdout.decode().strip().split(",")]
    assert ids[:len(prompt)] == prompt and len(ids) == len(prompt) + 5
    seq = list(prompt)
    for t in ids[len(prompt):]:
        l = P.forward(cfg, w, seq)[-1]
        assert float(l.max() - l[t]) < 1e-3
        seq.append(t)


def test_the_two_attention_kernels_agree_in_bfloat16(folders):
    """The tensor-core kernels against the FMA kernel on the same bfloat16 model: a prompt, a piece, single tokens."""
    from hos_b200.parts.gated_attention import GatedSoftmaxAttention
    vocab = CASES["E"][0]["vocab"]
    seq = tokens(130, 400, vocab)
    outs = []
    for use in (True, False):
        GatedSoftmaxAttention.use_tensor_cores = use
        try:
            r = _runner(folders["E"], "bfloat16")
            (slot,) = r.admit(1)
            got = [r.step([slot], [seq[:310]], [list(range(0, 310, 3))]), r.step([slot], [seq[310:380]], [list(range(70))])]
            got += [r.step([slot], [[t]]) for t in seq[380:]]
            outs.append(torch.cat(got).cpu())
            r.release(slot)
        finally:
            GatedSoftmaxAttention.use_tensor_cores = True
    assert_rows(outs[0], outs[1], "bfloat16", "the two kernels")


def test_the_norm_kernel_alone_against_float64():
    """x += mult (a + f); h = tanh(alpha x) w + b: rows and 32-bit partial sums, widths that are and are not multiples
    of four, 32-bit in place and bfloat16 out, and the plain norm without a sum."""
    from hos_b200 import ops
    dev = "cuda"
    torch.manual_seed(11)
    for n, d in ((37, 100), (5, 256), (1, 3), (300, 1028)):
        x = torch.randn(n, d, device=dev) * 2
        a = torch.randn(3, n, d, device=dev)
        f = torch.randn(n, d, device=dev).to(torch.bfloat16)
        w, b = torch.randn(d, device=dev), torch.randn(d, device=dev)
        alpha, mult = 0.7, 1.5
        x64 = x.double().cpu() + mult * (a.double().cpu().sum(0) + f.double().cpu())
        h64 = torch.tanh(alpha * x64) * w.double().cpu() + b.double().cpu()
        for out_dtype in (torch.float32, torch.bfloat16):
            xs = x.clone()
            h = torch.empty(n, d, device=dev, dtype=out_dtype)
            ops.add_dyt(a, f, mult, xs, alpha, w, b, h)
            assert float((xs.double().cpu() - x64).abs().max()) < 1e-5
            tol = 1e-5 if out_dtype == torch.float32 else 2e-2
            assert float((h.double().cpu() - h64).abs().max()) < tol * max(1.0, float(h64.abs().max()))
        xs = x.clone()
        ops.add_dyt(None, None, 0.0, xs, alpha, w, b, xs)            # the plain norm, in place
        want = torch.tanh(alpha * x.double().cpu()) * w.double().cpu() + b.double().cpu()
        assert float((xs.double().cpu() - want).abs().max()) < 1e-5
        xs = x.clone()
        ops.add_dyt(None, f, mult, xs, alpha, None, None, None)      # the sum alone
        assert float((xs.double().cpu() - (x.double().cpu() + mult * f.double().cpu())).abs().max()) < 1e-5


def _paged(rows_k, rows_v, table, G, kd, vd, dtype, dev):
    """Keys and values of several sequences laid into pages by a page table, with the cache's permutation of groups of
    eight numbers where a row is a multiple of 64 numbers."""
    n_pages = int(table.max()) + 2
    kp = torch.zeros(n_pages, G, 64, kd, device=dev, dtype=dtype)
    vp = torch.zeros(n_pages, G, 64, vd, device=dev, dtype=dtype)

    def place(pages, rows, hd):
        swz = hd % 64 == 0
        for sq, r in enumerate(rows):
            for t in range(r.shape[0]):
                if not swz:
                    pages[table[sq, t // 64], :, t % 64] = r[t].to(dev).to(dtype)
                    continue
                for d0 in range(0, hd, 8):
                    c = (d0 // 8) ^ (t % 64 % 8)
                    pages[table[sq, t // 64], :, t % 64, c * 8:c * 8 + 8] = r[t, :, d0:d0 + 8].to(dev).to(dtype)
    place(kp, rows_k, kd)
    place(vp, rows_v, vd)
    return kp, vp


def test_the_attention_kernels_alone_against_float64():
    """Whole-projection norms and blended values (qk_prep), then attention with a window that keeps first keys and a
    zero sink: the FMA kernel in one share and several, the tensor-core kernels for prompts and for single tokens;
    three sequences of which one goes on from position 100, pages in no order."""
    from hos_b200 import ops
    from hos_b200.parts.base import StepInfo
    dev = "cuda"
    torch.manual_seed(4)
    H, G, scale = 6, 2, 0.2
    lens, starts = (150, 70, 3), (0, 100, 0)
    tot = [a + b for a, b in zip(lens, starts)]
    n = sum(lens)
    pos = torch.cat([s0 + torch.arange(ln) for s0, ln in zip(starts, lens)]).to(torch.int32).to(dev)
    seqid = torch.cat([torch.full((ln,), i) for i, ln in enumerate(lens)]).to(torch.int32).to(dev)
    cu = torch.tensor([0, 150, 220, 223], dtype=torch.int32, device=dev)
    slots = torch.arange(3, dtype=torch.int32, device=dev)
    table, nxt = torch.zeros(3, 4, dtype=torch.int32), 7
    for sq, t in enumerate(tot):
        for e in range((t + 63) // 64):
            table[sq, e] = nxt
            nxt = nxt - 1 if sq == 1 else nxt + 3                     # pages lie apart and in no order
        nxt += 20
    step = StepInfo(n, 3, None, pos, seqid, cu, slots, None, False, False, 150, 170)
    for kd, vd, window, keep in ((24, 40, 70, 5), (64, 128, 70, 70), (128, 64, 33, 1), (64, 64, 130, 64), (128, 128, 64, 3),
                                 (64, 128, 5, 0), (8, 8, 1, 1)):
        # qk_prep on the step's rows: a fused row [q | k | v | gate], norms over the whole projections, values blended
        ld = H * kd + G * (kd + vd) + H
        proj = torch.randn(n, ld, device=dev)
        other = torch.randn(n, G * vd + 3, device=dev)
        qn, kn, lam, eps = torch.randn(H * kd, device=dev), torch.randn(G * kd, device=dev), 0.3, 1e-3
        for dtype in (torch.float32, torch.bfloat16):
            ks = [torch.randn(t, G, kd) for t in tot]
            vs = [torch.randn(t, G, vd) for t in tot]
            kp, vp = _paged(ks, vs, table, G, kd, vd, dtype, dev)
            cache = ops.PagedKVArgs(kp, vp, table.to(dev), 0, G, kd, vd)
            q = torch.empty(n, H, kd, device=dev)
            ops.qk_prep(proj, None, qn, kn, eps, None, 0, 1.0, step, q, cache, H, G, kd, vd, True, other, 3, lam)
            P = proj.double().cpu()
            q64, k64 = P[:, :H * kd], P[:, H * kd:(H + G) * kd]
            q64 = q64 / torch.sqrt((q64 * q64).mean(-1, keepdim=True) + eps) * qn.double().cpu()
            k64 = k64 / torch.sqrt((k64 * k64).mean(-1, keepdim=True) + eps) * kn.double().cpu()
            v64 = (1 - lam) * P[:, (H + G) * kd:(H + G) * kd + G * vd] + lam * other.double().cpu()[:, 3:]
            assert float((q.double().cpu().view(n, -1) - q64).abs().max()) < 1e-5 * max(1.0, float(q64.abs().max()))
            # what the cache must now hold: the rows before the step as they were, the step's rows from qk_prep
            at, want = 0, []
            rnd = (lambda t: t.to(torch.bfloat16).double()) if dtype == torch.bfloat16 else (lambda t: t.float().double())
            if dtype == torch.bfloat16:                # every kernel then sees the queries the tensor cores would round to
                q = q.to(torch.bfloat16).float()
            qq = q.double().cpu().view(n, -1)
            for sq, (ln, s0) in enumerate(zip(lens, starts)):
                kk = torch.cat([rnd(ks[sq][:s0]), rnd(k64[at:at + ln].view(ln, G, kd).float())]).repeat_interleave(H // G, 1)
                vv = torch.cat([rnd(vs[sq][:s0]), rnd(v64[at:at + ln].view(ln, G, vd).float())]).repeat_interleave(H // G, 1)
                sc = torch.einsum("ihd,jhd->hij", qq[at:at + ln].view(ln, H, kd), kk) * scale
                ii, jj = (s0 + torch.arange(ln))[:, None], torch.arange(tot[sq])[None]
                e = torch.exp(sc) * ((ii >= jj) & ((ii - jj < window) | (jj < keep)))
                pr = e / (1.0 + e.sum(-1, keepdim=True))
                o = torch.einsum("hij,jhr->ihr", pr, vv)
                want.append(o * torch.sigmoid(P[at:at + ln, ld - H:])[..., None])
                at += ln
            want = torch.cat(want)
            tol = 2e-5 if dtype == torch.float32 else 1e-2
            sink = torch.zeros(H, device=dev)
            for splits in (1, 3):
                out = torch.empty(n, H * vd, device=dev, dtype=dtype)
                ops.gated_attn(q, cache, sink, proj, ld - H, step, out, scale, 0, window, splits, keep)
                err = float((out.double().cpu().view(n, H, vd) - want).abs().max())
                assert err < tol * max(1.0, float(want.abs().max())), f"{kd}/{vd} window {window} keeps {keep}, {splits} shares: {err:.2e}"
            if dtype != torch.bfloat16 or kd not in (64, 128) or vd not in (64, 128):
                continue
            out = torch.empty(n, H * vd, device=dev, dtype=dtype)
            assert ops.gated_attn_mma(q, cache, sink, proj, ld - H, step, out, scale, 0, window, 3 + 2 + 1, keep)
            err = float((out.double().cpu().view(n, H, vd) - want).abs().max())
            assert err < tol * max(1.0, float(want.abs().max())), f"tensor cores, {kd}/{vd} window {window} keeps {keep}: {err:.2e}"
            last = [149, 219, 222]
            step1 = StepInfo(3, 3, None, pos[last].contiguous(), slots, torch.arange(4, dtype=torch.int32, device=dev), slots,
                             None, False, True, 1, 170)
            q1, g1 = q[last].contiguous(), proj[last].contiguous()
            for shares in (1, 2, 5):
                out1 = torch.empty(3, H * vd, device=dev, dtype=dtype)
                assert ops.gated_attn_mma_decode(q1, cache, sink, g1, ld - H, step1, out1, scale, 0, window, shares, keep)
                err = float((out1.double().cpu().view(3, H, vd) - want[last]).abs().max())
                assert err < tol * max(1.0, float(want.abs().max())), f"single tokens, {kd}/{vd}, {shares} shares: {err:.2e}"


def test_the_router_kernel_alone_against_float64():
    """Logistic scores of 32-bit logits, the `top` largest, the plain scores as weights: few rows and many (a block
    takes one, four or eight rows), few outputs and many (their groups of eight on blocks of their own), widths that are
    and are not multiples of four, 32-bit and bfloat16 rows, padding rows.  A row's logits do not depend on how many
    rows come with it: the weights of a row alone and in a batch are the same numbers."""
    from hos_b200 import ops
    dev = "cuda"
    torch.manual_seed(9)
    for n, d, n_out, top in ((1, 100, 3, 1), (5, 64, 8, 8), (17, 1024, 40, 6), (70, 250, 9, 2), (1100, 128, 16, 3),
                             (2100, 96, 33, 4), (16, 4096, 300, 5)):
        router = torch.randn(n_out, d, device=dev) * (3.0 / d ** 0.5)
        for dtype in (torch.float32, torch.bfloat16):
            h = torch.randn(n, d, device=dev).to(dtype)
            seq = torch.zeros(n, dtype=torch.int32, device=dev)
            if n > 2:
                seq[n // 2] = -1                                         # a padding row
            choice = torch.full((n * top,), -7, dtype=torch.int32, device=dev)
            weight = torch.full((n * top,), -7.0, device=dev)
            ops.moe_route(h, router, None, seq, choice, weight, top, ops.MOE_SCORING["logistic"])
            s64 = torch.sigmoid(h.double().cpu() @ router.double().cpu().T)
            choice, weight = choice.cpu().view(n, top), weight.cpu().view(n, top)
            for r in range(n):
                if n > 2 and r == n // 2:
                    assert choice[r].tolist() == [-1] * top and weight[r].tolist() == [0.0] * top
                    continue
                order = sorted(range(n_out), key=lambda e: (-float(s64[r, e]), e))
                got = choice[r].tolist()
                assert len(set(got)) == top and all(0 <= e < n_out for e in got)
                # the chosen ones are the largest (a tie within 32-bit rounding may come in either order)
                assert float(s64[r, got].min()) >= float(s64[r, order[top - 1]]) - 1e-6, (n, d, n_out, r)
                assert float((weight[r].double() - s64[r, got]).abs().max()) < 1e-5
                assert all(float(weight[r, k]) >= float(weight[r, k + 1]) for k in range(top - 1))
            if n > 1:
                c1 = torch.empty(top, dtype=torch.int32, device=dev)
                w1 = torch.empty(top, device=dev)
                ops.moe_route(h[n - 1:].clone(), router, None, seq[:1], c1, w1, top, ops.MOE_SCORING["logistic"])
                assert torch.equal(c1.cpu(), choice[n - 1]) and torch.equal(w1.cpu(), weight[n - 1]), "alone and in a batch differ"


@pytest.mark.gpu
def test_the_few_rows_expert_products_alone_against_float64():
    """A handful of (row, choice) pairs without lists or tiles: one, two or four features to a warp (the grid decides),
    widths and feature counts that end inside a warp's share and inside a round of loads, the weight on the expert's
    input or on its output, a clamp and a shift or none, a pair that chose nothing."""
    from hos_b200 import ops
    dev = "cuda"
    torch.manual_seed(21)
    for rows, top, n_experts, d, f, on_input, limit, alpha, shift in (
            (1, 4, 9, 1024, 1024, True, 0.0, 1.0, 0.0),        # few blocks: one feature to a warp
            (3, 2, 5, 1000, 1016, True, 0.0, 1.0, 0.0),        # two to a warp; rows of 125 groups
            (8, 4, 6, 520, 2408, True, 0.0, 1.0, 0.0),         # four to a warp; features end inside a block
            (2, 3, 4, 72, 40, False, 7.0, 1.7, 1.0),           # tiny, the weight on the output, clamp and shift
            (5, 2, 3, 4096, 264, False, 0.0, 1.0, 0.0)):
        pairs = rows * top
        h = torch.randn(rows, d, device=dev).to(torch.bfloat16)
        w_gu = (torch.randn(n_experts, 2 * f, d, device=dev) / d ** 0.5).to(torch.bfloat16)
        w_dn = (torch.randn(n_experts, d, f, device=dev) / f ** 0.5).to(torch.bfloat16)
        choice = torch.randint(0, n_experts, (pairs,), dtype=torch.int32, device=dev)
        if pairs > 2:
            choice[1] = -1
        weight = torch.rand(pairs, device=dev) + 0.25
        y = torch.zeros(pairs, f, dtype=torch.bfloat16, device=dev)
        out = torch.full((pairs, d), -5.0, device=dev)
        assert ops.moe_few(h, w_gu, w_dn, choice, weight, y, out, top, n_experts, limit, alpha, shift, weight_on_input=on_input)
        torch.cuda.synchronize()
        for p in range(pairs):
            e = int(choice[p])
            if e < 0:
                assert float(out[p].min()) == -5.0 and float(out[p].max()) == -5.0      # untouched
                continue
            x = h[p // top].double().cpu()
            wt = float(weight[p])
            g = w_gu[e, :f].double().cpu() @ x
            u = w_gu[e, f:].double().cpu() @ x
            if on_input:
                g, u = g * wt, u * wt
            if limit > 0:
                g, u = g.clamp(max=limit), u.clamp(-limit, limit)
            act = g * torch.sigmoid(alpha * g) * (u + shift)
            assert float((y[p].double().cpu() - act).abs().max()) < 0.02 * float(act.abs().max()) + 1e-3, (rows, d, f, p)
            down = w_dn[e].double().cpu() @ y[p].double().cpu()             # from the rounded activations the kernel read
            if not on_input:
                down = down * wt
            assert float((out[p].double().cpu() - down).abs().max()) < 1e-4 * float(down.abs().max()) + 1e-5, (rows, d, f, p)


@pytest.mark.gpu
def test_the_router_tells_apart_scores_that_round_to_the_same_number():
    """Logits of 10 to 50 have logistic scores within a few 32-bit steps of 1 (or equal to it); the chosen experts are
    still those with the largest logits, as they are with exact scores."""
    from hos_b200 import ops
    dev = "cuda"
    torch.manual_seed(5)
    n, d, n_out, top = 40, 128, 24, 5
    router = torch.randn(n_out, d, device=dev) * (6.0 / d ** 0.5)
    h = torch.randn(n, d, device=dev)
    h[:, 0] = 32.0 / (6.0 / d ** 0.5)                                      # with the router's first column: 32 added to every logit
    router[:, 0] = 6.0 / d ** 0.5
    seq = torch.zeros(n, dtype=torch.int32, device=dev)
    choice = torch.empty(n * top, dtype=torch.int32, device=dev)
    weight = torch.empty(n * top, device=dev)
    ops.moe_route(h, router, None, seq, choice, weight, top, ops.MOE_SCORING["logistic"])
    z = h.double().cpu() @ router.double().cpu().T
    assert float(z.min()) > 4.0
    choice = choice.cpu().view(n, top)
    for r in range(n):
        order = torch.argsort(z[r], descending=True)
        gap = float(z[r, order[top - 1]] - z[r, order[top]])
        if gap < 1e-3:
            continue                                                       # a close call in 32-bit logits too
        assert sorted(choice[r].tolist()) == sorted(order[:top].tolist()), r
    assert float(weight.min()) > 0.98
