"""Tofodra on the GPU against the plain oracle (tests/plain/tofodra_plain.py): every mechanism alone, whole prompts,
decoding through the cache and the state, prompts in pieces, batches against each request alone, reuse of slots, pages
and state, the edges of windows, kept keys and pages, the first tokens, far keys, long decoding, other sizes, and
generation through the engine, the replay program and the command line."""
import copy
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from tofodra_cases import CASES, assert_rows, attention, latent, make_folder, model, moe, oracle_view, retention, row_errors, tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("tofodra")
    return {k: make_folder(base, raw, seed, k) for k, (raw, seed) in CASES.items()}


def _runner(folder, dtype, **kw):
    from hos_b200.engine import Runner
    kw.setdefault("max_tokens", 4096)
    kw.setdefault("max_seq_len", 1024)
    return Runner.from_folder(folder, dtype=dtype, **kw)


def _oracle(folder, seqs):
    from plain import tofodra_plain as P
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
    steps, so every window passes wholly over decoded tokens and the matrix states are carried for as long."""
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
    """Pieces down to two tokens and one, pieces that end on a page's border and one past it: the matrix states go on
    from what the slot holds, a reading layer finds the earlier pieces' latents in the other layer's pages."""
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
    tol = 2e-5 if dtype == "float32" else 4e-2
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
    """What a freed slot's pages and its matrix states still hold must never be read: the pages are overwritten and
    the states start at zero when the slot is taken again."""
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
            if t is not None:            # a keys-only group has no values; a reading call has no arrays of its own
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
    # a request that starts with single tokens in a used slot: its states start at zero all the same
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
    from plain import tofodra_plain as P
    raw = CASES[case][0]
    cfg, w = oracle_view(folders[case])
    seq = tokens(60, 160, raw["vocab"])
    want = P.forward(cfg, w, seq)
    for key, d in (("size", 1), ("size", -1), ("keep_first", 1), ("keep_first", -1)):
        def edit(i, m):
            if m.get("mask") and m["mask"].get(key, 0) + d > 0:
                m["mask"] = dict(m["mask"], **{key: m["mask"].get(key, 0) + d})
            return m
        if not any(l["mixer"].get("mask") for l in cfg["layers"]):
            continue
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


def test_far_keys_kept_keys_and_a_long_memory(tmp_path):
    """Soft scores and a slow decay: a latent layer and a differential layer that see all keys, a reading layer, a
    differential layer with a short window that keeps the first five keys, retention that forgets a thousandth per token.
    Without the keys that lie more than 600 tokens back, or without the kept keys, the oracle's logits move by far more
    than the tolerance.  In decoding a row's keys are cut into shares that are merged (more than 256 keys)."""
    from plain import tofodra_plain as P
    raw = model(48, 60, [latent(2, 8, 4, 12, 16, 0.1, mlp=None), attention(2, 1, 8, 12, 0.15, 0.4, mlp=None),
                         attention(4, 2, 8, 12, 0.3, 0.2, window=9, keep=5, mlp=None),
                         retention((0.999, 0.99), 8, 12, rot=8, mlp=None),
                         latent(3, 4, 4, 8, 16, 0.12, kv_from=0, mlp=None)])
    folder = make_folder(tmp_path, raw, 5, "far")
    cfg, w = oracle_view(folder)
    seq = tokens(70, 644, 60)
    want = P.forward(cfg, w, seq)

    def no_far(i, m):
        return dict(m, mask={"size": 600}) if not m.get("mask") and "decay" not in m else m

    def no_kept(i, m):
        return dict(m, mask={"size": m["mask"]["size"]}) if m.get("mask") else m

    def forgets(i, m):
        return dict(m, decay=[0.9, 0.9]) if "decay" in m else m
    assert float(row_errors(P.forward(cfg, w, seq, edit=no_far)[610:], want[610:]).median()) > 1e-4
    assert float(row_errors(P.forward(cfg, w, seq, edit=no_kept)[610:], want[610:]).median()) > 2e-3
    assert float(row_errors(P.forward(cfg, w, seq, edit=forgets)[610:], want[610:]).median()) > 2e-3
    for dtype in ("float32", "bfloat16"):
        r = _runner(folder, dtype)
        (slot,) = r.admit(1)
        got = [r.step([slot], [seq[:600]], [list(range(600))]).cpu()] + [r.step([slot], [[t]]).cpu() for t in seq[600:]]
        assert_rows(torch.cat(got), want, dtype, "far keys and kept keys")
        r.release(slot)


def test_one_key_far_back_that_stands_out(tmp_path):
    """A key among hundreds made to carry the whole softmax: the query of the last positions and the key at position 3
    are scaled so that their score stands out in the latent layer and in both maps of the differential layer; a kernel
    that lost that key (a page, a share, a tile) would be off by the size of the logits."""
    from plain import tofodra_plain as P
    raw = model(32, 40, [latent(2, 8, 4, 8, 12, 0.5, mlp=None), attention(2, 1, 8, 8, 0.5, 0.3, mlp=None)])
    seq = tokens(71, 400, 40)
    seq[3] = 7
    for t in range(380, 400):
        seq[t] = 11

    def edit(t):
        t["embed"][7] *= 4.0          # the far key's token, and the asking token: large rows give large q and k
        t["embed"][11] *= 4.0
    folder = make_folder(tmp_path, raw, 6, "peak", edit=edit)
    cfg, w = oracle_view(folder)
    want = P.forward(cfg, w, seq)
    w2 = dict(w)
    cut = P.forward(cfg, w2, seq[:3] + [8] + seq[4:])
    assert float(row_errors(cut[380:], want[380:]).median()) > 1e-3, "the far key does not matter enough"
    for dtype in ("float32", "bfloat16"):
        r = _runner(folder, dtype)
        (slot,) = r.admit(1)
        got = [r.step([slot], [seq[:390]], [list(range(370, 390))]).cpu()] + [r.step([slot], [[t]]).cpu() for t in seq[390:]]
        assert_rows(torch.cat(got), want[370:], dtype, "a far key that stands out")
        r.release(slot)


def test_every_layer_alone(folders):
    """The residual stream after every layer, in 32-bit, for a prompt; then the same for the prompt's second half fed
    after its first (every mixer resumes from its cache or state)."""
    from plain import tofodra_plain as P
    for case in ("A", "B", "C", "D"):
        cfg, w = oracle_view(folders[case])
        seq = tokens(80, 90, cfg["vocab"])
        want = []
        P.forward(cfg, w, seq, taps=want)
        r = _runner(folders[case], "float32")
        (slot,) = r.admit(1)
        taps = r.hidden_states([slot], [seq])[1:]           # the first tap is the embedding
        assert len(taps) == len(want)
        for i, (g, x) in enumerate(zip(taps, want)):
            assert float(row_errors(g.cpu(), x).max()) < 1e-5, f"case {case}: after layer {i}"
        r.release(slot)
        (slot,) = r.admit(1)
        r.step([slot], [seq[:47]])
        taps = r.hidden_states([slot], [seq[47:]])[1:]
        for i, (g, x) in enumerate(zip(taps, want)):
            assert float(row_errors(g.cpu(), x[47:]).max()) < 1e-5, f"case {case}: after layer {i}, second half"
        r.release(slot)


SINGLE = {
    "latent: one head, a latent of three": latent(1, 4, 2, 5, 3, 0.6, mlp=None),
    "latent: nine heads (two head groups), values wider than keys": latent(9, 8, 4, 24, 40, 0.4, mlp=None),
    "latent: a latent wider than a block's threads": latent(2, 8, 8, 8, 272, 0.2, mlp=None),
    "retention: one head of one key number": retention((0.9,), 1, 3, mlp=None),
    "retention: heads of 200 x 40, half rotated": retention((0.99, 0.95), 200, 40, rot=100, mlp=None),
    "retention: nothing rotated, values wider than keys": retention((0.7, 0.8, 0.9), 8, 264, mlp=None),
    "attention: keys wider than values, all keys in sight": attention(3, 3, 40, 8, 0.3, 0.5, mlp=None),
    "attention: maps of 100 numbers, values of 264": attention(2, 1, 100, 264, 0.1, 0.2, window=50, keep=3, mlp=None),
    "attention: ten query heads to a kv head": attention(10, 1, 8, 8, 0.5, 0.6, window=100, keep=1, mlp=None),
    "attention: one head of one number, values of three": attention(1, 1, 1, 3, 0.9, 0.3, window=2, keep=2, mlp=None),
    "attention: kept keys beyond the prompt": attention(4, 2, 16, 16, 0.5, 0.9, window=3, keep=120, mlp=None),
    "a dense feed-forward whose clamp always bites": attention(1, 1, 8, 8, 0.2, 0.5, window=4),
    "every expert chosen, no shared one": retention((0.9, 0.8), 8, 8, rot=4, mlp=moe(4, 4, 24, scale=0.3)),
    "one expert of one": retention((0.9,), 8, 8, mlp=moe(1, 1, 40, shared=8, scale=2.0)),
    "forty experts, six chosen": latent(2, 8, 4, 8, 16, 0.4, mlp=moe(40, 6, 8, shared=72)),
    "experts wider than the model": latent(2, 8, 4, 8, 16, 0.4, mlp=moe(3, 2, 136, shared=264, scale=1.5)),
}


@pytest.mark.parametrize("name", list(SINGLE))
def test_one_layer_models_of_other_sizes(tmp_path, name):
    """Sizes that the kernels' shapes switch on, each as a model of one layer: a prompt, then pieces of one to five
    tokens, in 32-bit."""
    raw = model(40, 50, [SINGLE[name]], ff=16, limit=0.05 if "always bites" in name else 1.0)
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
    from plain import tofodra_plain as P
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
    from plain import tofodra_plain as P
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


def test_the_attention_kernels_agree_in_bfloat16(folders):
    """The tensor-core kernels against the FMA kernels on the same bfloat16 model: a prompt, a piece, single tokens."""
    from hos_b200.parts.differential_attention import DifferentialAttention
    from hos_b200.parts.latent_attention import LatentAttention
    vocab = CASES["E"][0]["vocab"]
    seq = tokens(130, 400, vocab)
    outs = []
    for use in (True, False):
        DifferentialAttention.use_tensor_cores = LatentAttention.use_tensor_cores = use
        try:
            r = _runner(folders["E"], "bfloat16")
            (slot,) = r.admit(1)
            got = [r.step([slot], [seq[:310]], [list(range(0, 310, 3))]), r.step([slot], [seq[310:380]], [list(range(70))])]
            got += [r.step([slot], [[t]]) for t in seq[380:]]
            outs.append(torch.cat(got).cpu())
            r.release(slot)
        finally:
            DifferentialAttention.use_tensor_cores = LatentAttention.use_tensor_cores = True
    assert_rows(outs[0], outs[1], "bfloat16", "the two kinds of kernel")


def test_the_small_kernels_alone_against_float64():
    """rotate_rows (both pairings, part of a head, the keys' factor, padding rows), diff_combine (with and without a
    gate, both output types), the clamped gated activation, and the router's normalised and scaled weights."""
    from hos_b200 import ops
    from hos_b200.parts.base import StepInfo
    dev = "cuda"
    torch.manual_seed(3)
    n = 37
    pos = torch.randint(0, 5000, (n,), dtype=torch.int32, device=dev)
    seq = torch.zeros(n, dtype=torch.int32, device=dev)
    seq[5] = -1                                              # a padding row is left alone
    step = StepInfo(n, 1, None, pos, seq, None, None, None, False, False, n, 5000)
    for Hq, Hk, dim, rot, style, mult in ((3, 3, 24, 8, "rotate_half", 0.25), (2, 5, 16, 16, "interleaved", 1.0),
                                          (1, 1, 6, 2, "rotate_half", 3.0), (4, 2, 10, 0, "rotate_half", 0.5)):
        ld = (Hq + Hk) * dim + 7
        x = torch.randn(n, ld, device=dev)
        freq = torch.tensor([50.0 ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)], dtype=torch.float64).float().to(dev)
        y = x.clone()
        ops.rotate_rows(y, Hq, Hk, dim, freq if rot else None, rot, ops.ROPE_STYLES[style], step, mult)
        X = x.double().cpu()
        want = X.clone()
        ang = pos.double().cpu()[:, None] * freq.double().cpu()[None]
        c, s = torch.cos(ang), torch.sin(ang)
        for h in range(Hq + Hk):
            v = X[:, h * dim:(h + 1) * dim].clone()
            if rot:
                ia = torch.arange(rot // 2) if style == "rotate_half" else torch.arange(0, rot, 2)
                ib = ia + rot // 2 if style == "rotate_half" else ia + 1
                a, b = v[:, ia].clone(), v[:, ib].clone()
                v[:, ia], v[:, ib] = a * c - b * s, b * c + a * s
            want[:, h * dim:(h + 1) * dim] = v * (mult if h >= Hq else 1.0)
        want[5] = X[5]
        # the angle itself is a 32-bit product: positions up to 5,000 leave about 3e-4 of a turn
        assert float((y.double().cpu() - want).abs().max()) < 2e-3, (Hq, Hk, dim, rot, style)
        assert torch.equal(y[:, (Hq + Hk) * dim:], x[:, (Hq + Hk) * dim:])
    seq[5] = 0
    for H, vd, gated in ((3, 24, True), (1, 5, False), (4, 128, True)):
        a = torch.randn(n, H * 2 * vd, device=dev)
        gate = torch.randn(n, H * vd + 9, device=dev)
        lam, mult, eps = 0.37, 0.6, 1e-3
        A = a.double().cpu().view(n, H, 2, vd)
        o = A[:, :, 0] - lam * A[:, :, 1]
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * mult
        if gated:
            o = o * torch.sigmoid(gate.double().cpu()[:, 9:].view(n, H, vd))
        for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 1e-2)):
            out = torch.empty(n, H * vd, device=dev, dtype=dt)
            ops.diff_combine(a, lam, mult, eps, gate if gated else None, 9, step, out, H, vd)
            assert float((out.double().cpu().view(n, H, vd) - o).abs().max()) < tol * max(1.0, float(o.abs().max()))
    gu = torch.randn(n, 2 * 50, device=dev) * 2
    for limit, alpha, shift in ((0.8, 1.702, 1.0), (0.0, 1.0, 0.0)):
        g, u = gu.double().cpu()[:, :50], gu.double().cpu()[:, 50:]
        if limit:
            g, u = g.clamp(max=limit), u.clamp(-limit, limit)
        want = g * torch.sigmoid(alpha * g) * (u + shift)
        out = torch.empty(n, 50, device=dev)
        ops.clamped_gated_act(gu, out, limit, alpha, shift)
        assert float((out.double().cpu() - want).abs().max()) < 1e-5
    h = torch.randn(n, 64, device=dev)
    router = torch.randn(10, 64, device=dev) * 0.3
    top = 4
    choice = torch.empty(n * top, dtype=torch.int32, device=dev)
    weight = torch.empty(n * top, dtype=torch.float32, device=dev)
    ops.moe_route(h, router, None, seq, choice, weight, top, ops.MOE_SCORING["logistic"], 1e-20, 1.75)
    s = torch.sigmoid(h.double().cpu() @ router.double().cpu().T)
    best = torch.topk(s, top, dim=-1)
    assert torch.equal(choice.cpu().view(n, top).long(), best.indices)
    want = best.values / (best.values.sum(-1, keepdim=True) + 1e-20) * 1.75
    assert float((weight.double().cpu().view(n, top) - want).abs().max()) < 1e-5


def test_the_clamped_form_in_the_products_epilogues():
    """The dense feed-forward's clamp, activation and product as the third activation of the gated epilogues: the
    few-rows kernel, the tcgen05 kernel in both orientations and on pairs of SMs, the plain kernel in both types,
    against float64; and the part's two ways (fused, or a kernel of its own) on the same rows."""
    from hos_b200 import ops
    from hos_b200.parts import linear
    dev = "cuda"
    torch.manual_seed(9)
    k, f, limit = 256, 384, 0.9
    w = (torch.randn(2 * f, k, device=dev) * 0.08).to(torch.bfloat16)
    for m in (1, 5, 24, 100, 300, 1100):
        x = torch.randn(m, k, device=dev).to(torch.bfloat16)
        gu = x.double().cpu() @ w.double().cpu().T
        g, u = gu[:, :f].clamp(max=limit), gu[:, f:].clamp(-limit, limit)
        want = g * torch.sigmoid(1.702 * g) * (u + 1.0)
        got = linear.matmul(x, w, epilogue=ops.EPI_GATED, act=ops.ACT_CLAMPED_SWISH, cap=limit)
        assert got.dtype == torch.bfloat16
        assert float((got.double().cpu() - want).abs().max()) < 2e-2 * max(1.0, float(want.abs().max())), f"{m} rows"
        linear.force_plain(True)
        try:
            got = linear.matmul(x, w, epilogue=ops.EPI_GATED, act=ops.ACT_CLAMPED_SWISH, cap=limit)
            got32 = linear.matmul(x.float(), w.float(), epilogue=ops.EPI_GATED, act=ops.ACT_CLAMPED_SWISH, cap=limit)
        finally:
            linear.force_plain(False)
        assert float((got.double().cpu() - want).abs().max()) < 2e-2 * max(1.0, float(want.abs().max()))
        assert float((got32.double().cpu() - want).abs().max()) < 1e-5 * max(1.0, float(want.abs().max()))
        # no clamp at all: the limit is zero
        free = gu[:, :f] * torch.sigmoid(1.702 * gu[:, :f]) * (gu[:, f:] + 1.0)
        got = linear.matmul(x, w, epilogue=ops.EPI_GATED, act=ops.ACT_CLAMPED_SWISH, cap=0.0)
        assert float((got.double().cpu() - free).abs().max()) < 2e-2 * max(1.0, float(free.abs().max()))


def test_the_dense_feed_forward_fused_and_in_two_steps(folders):
    from hos_b200.parts.feedforward import GatedMLP
    vocab = CASES["A"][0]["vocab"]
    seq = tokens(160, 200, vocab)
    want = _oracle(folders["A"], [seq])[0]
    for dtype in ("float32", "bfloat16"):
        outs = []
        for fused in (True, False):
            GatedMLP.fused = fused
            try:
                r = _runner(folders["A"], dtype)
                (slot,) = r.admit(1)
                got = [r.step([slot], [seq[:190]], [list(range(190))])] + [r.step([slot], [[t]]) for t in seq[190:]]
                outs.append(torch.cat(got).cpu())
                r.release(slot)
            finally:
                GatedMLP.fused = True
        for o in outs:
            assert_rows(o, want, dtype, "the clamped feed-forward")
