"""Tofodra without a GPU: the configuration's checks, the plan (arrangement, parts, run order, tensor names and
shapes) and properties of the oracle itself that the GPU tests rely on."""
import copy

import pytest
import torch

from tofodra_cases import CASES, make_folder, oracle_view, row_errors, tokens


def test_the_plan_names_every_tensor_once():
    from hos_b200.model import weight_specs_for
    from hos_b200.registry import config_from_dict, plan_for
    cfg = config_from_dict(CASES["A"][0])
    plan = plan_for(cfg)
    assert [l.arrangement for l in plan.layers] == ["sandwich"] * 5
    assert [l.mixer.kind for l in plan.layers] == ["decay_linear_attention", "latent_attention", "differential_attention",
                                                   "decay_linear_attention", "latent_attention"]
    assert [c.cache_from for c in plan.schedule] == [None, None, None, None, 1]
    assert plan.layers[4].mixer.params["shares_kv"] and not plan.layers[1].mixer.params["shares_kv"]
    assert plan.layers[2].mixer.params["keep_first"] == 3 and plan.layers[2].mixer.params["window"] == 70
    assert plan.layers[2].feed_forward.kind == "none" and set(plan.layers[2].norms) == {"pre_mixer", "post_mixer"}
    assert plan.layers[0].feed_forward.params["weight_scale"] == 1.7 and plan.layers[3].feed_forward.params["weight_scale"] == 1.0
    assert plan.layers[0].mixer.params["position"].params["style"] == "rotate_half"
    assert plan.layers[3].mixer.params["position"] is None
    assert plan.layers[1].mixer.params["position"].params["style"] == "interleaved"
    names = {s.name: tuple(s.shape) for s in weight_specs_for(cfg)}
    assert names["embed"] == (211, 72) and names["head"] == (211, 72) and names["final.norm"] == (72,)
    assert names["l0.mix.q"] == (72, 72) and names["l0.mix.v"] == (48, 72) and names["l0.mix.g"] == (48, 72)
    assert names["l0.mix.o"] == (72, 48) and "l0.mix.norm" not in names
    assert names["l1.mix.q"] == (72, 72) and names["l1.mix.dkv"] == (48, 72) and names["l1.mix.dkv.norm"] == (40,)
    assert names["l1.mix.uk"] == (48, 40) and names["l1.mix.uv"] == (72, 40) and names["l1.mix.o"] == (72, 72)
    assert names["l2.mix.q"] == (96, 72) and names["l2.mix.k"] == (32, 72) and names["l2.mix.v"] == (24, 72)
    assert names["l2.mix.q.b"] == (96,) and names["l2.mix.k.b"] == (32,) and names["l2.mix.v.b"] == (24,)
    assert names["l2.mix.lq1"] == (16,) and names["l2.mix.lk2"] == (16,) and names["l2.mix.g"] == (72, 72)
    assert "l2.norm2" not in names and "l2.ls2" not in names and names["l2.ls1"] == (72,) and names["l2.norm1b"] == (72,)
    assert "l4.mix.dkv" not in names and "l4.mix.dkv.norm" not in names and names["l4.mix.uk"] == (48, 40)
    assert names["l0.mlp.router"] == (5, 72) and names["l0.mlp.e4.down"] == (72, 40) and names["l0.mlp.shared.up"] == (24, 72)
    assert "l3.mlp.shared.gate" not in names and names["l1.mlp.gate"] == (56, 72) and names["l1.ls2"] == (72,)
    assert config_from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][2]["mixer"].update(kv_heads=2), "multiple"),
    (lambda c: c["layers"][4]["mixer"].update(kv_rank=48), "differ"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=4), "kv_from"),
    (lambda c: c["layers"][4]["mixer"].update(kv_from=0), "kv_from"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mixer"].pop("rot"), "rot"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][2]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][2]["mixer"]["mask"].update(size=0), "mask"),
    (lambda c: c["layers"][2]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["layers"][0].update(type="recurrence"), "type"),
    (lambda c: c["layers"][1]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["layers"][1]["mlp"].pop("limit"), "limit"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][0]["mlp"].pop("expert"), "expert"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_a_wrong_configuration_is_refused_with_the_key_named(edit, word):
    from hos_b200.errors import MissingMetaError
    from hos_b200.registry import config_from_dict
    raw = copy.deepcopy(CASES["A"][0])
    edit(raw)
    with pytest.raises(MissingMetaError) as e:
        config_from_dict(raw)
    assert word in str(e.value)


def test_a_layer_scale_is_folded_into_its_norm():
    """The multiplier per column is the norm's second tensor; bound, the norm's weight is the exact product."""
    from hos_b200.config.base import PartSpec
    from hos_b200.parts.base import Runtime
    from hos_b200.parts.norm import RMSNorm
    w = torch.randn(12).to(torch.bfloat16)
    s = torch.randn(12).to(torch.bfloat16)
    n = RMSNorm(PartSpec("rmsnorm", {"width": 12, "eps": 1e-6}, {"weight": "w", "scale": "s"}), Runtime(torch.device("cpu"), torch.bfloat16))
    assert [x.name for x in n.weight_specs()] == ["w", "s"]
    n.bind({"w": w, "s": s})
    assert torch.equal(n.weight.double(), w.double() * s.double())
    g = RMSNorm(PartSpec("rmsnorm", {"width": 12, "eps": 1e-6, "add_one": True}, {"weight": "w", "scale": "s"}),
                Runtime(torch.device("cpu"), torch.bfloat16))
    g.bind({"w": w, "s": s})
    assert float(((g.weight.double() + 1.0) - (w.double() + 1.0) * s.double()).abs().max()) < 1e-6


def test_the_oracle_feels_every_mechanism(tmp_path):
    """What the GPU tests compare with must move when a mechanism is taken away or shifted by one: every window's and
    kept run's edge, lambda, the second map, the gate, the source of a reading layer's latents, the rotations, the decay,
    the keys' factor, the clamp, the router's normalisation and factor, the layer scales."""
    from plain import tofodra_plain as P
    folder = make_folder(tmp_path, CASES["A"][0], CASES["A"][1], "A")
    cfg, w = oracle_view(folder)
    seq = tokens(1, 110, cfg["vocab"])
    want = P.forward(cfg, w, seq)
    for key, d in (("size", 1), ("size", -1), ("keep_first", 1), ("keep_first", -1)):
        def edit(i, m):
            if m.get("mask") and m["mask"].get(key, 0) + d > 0:
                m["mask"] = dict(m["mask"], **{key: m["mask"].get(key, 0) + d})
            return m
        assert float(row_errors(P.forward(cfg, w, seq, edit=edit)[80:], want[80:]).median()) > 2e-3, (key, d)

    def moved(edit=None, **changed):
        w2 = dict(w, **changed)
        return float(row_errors(P.forward(cfg, w2, seq, edit=edit), want).median())
    assert moved(**{"l2.mix.lq1": w["l2.mix.lq1"] * 0.5}) > 2e-3                       # lambda
    assert moved(edit=lambda i, m: dict(m, diff=m["diff"] + 0.1) if "diff" in m else m) > 2e-3
    assert moved(**{"l2.mix.g": torch.zeros_like(w["l2.mix.g"])}) > 2e-3               # the gate
    assert moved(**{"l2.mix.q.b": torch.zeros_like(w["l2.mix.q.b"])}) > 2e-3           # a bias
    assert moved(edit=lambda i, m: dict(m, decay=[d * 0.98 for d in m["decay"]]) if "decay" in m else m) > 2e-3
    assert moved(edit=lambda i, m: dict(m, rot=dict(m["rot"], base=m["rot"]["base"] * 2)) if i == 0 else m) > 2e-3
    assert moved(edit=lambda i, m: dict(m, rot=dict(m["rot"], base=m["rot"]["base"] * 2)) if i == 1 else m) > 2e-3
    assert moved(**{"l1.ls1": w["l1.ls1"] * 1.1}) > 2e-3 and moved(**{"l4.ls2": w["l4.ls2"] * 1.1}) > 2e-3
    assert moved(**{"l1.mix.dkv": w["l1.mix.dkv"].flip(0)}) > 2e-3                     # what the last layer reads
    cfg2 = copy.deepcopy(cfg)
    cfg2["layers"][1]["mlp"]["limit"] = 50.0
    assert float(row_errors(P.forward(cfg2, w, seq), want).median()) > 2e-3            # the clamp bites
    cfg2 = copy.deepcopy(cfg)
    cfg2["layers"][0]["mlp"]["router"]["scale"] = 1.0
    assert float(row_errors(P.forward(cfg2, w, seq), want).median()) > 2e-3            # the router's factor
    # the rotation of retention is by position: a sequence shifted by one token is not the same sequence
    h = torch.randn(6, cfg["width"], dtype=torch.float64)
    m0 = cfg["layers"][0]["mixer"]
    full = P.retention_mixer(m0, 1e-6, w, "l0.mix.", h)
    assert float((P.retention_mixer(m0, 1e-6, w, "l0.mix.", h[1:]) - full[1:]).abs().max()) > 1e-3
    # the weights of the chosen experts sum to the router's factor
    mlp = cfg["layers"][0]["mlp"]
    one = dict(w)
    for e in range(5):
        for part in ("gate", "up", "down"):
            one[f"l0.mlp.e{e}.{part}"] = w[f"l0.mlp.e0.{part}"]
    for part in ("gate", "up", "down"):
        one[f"l0.mlp.shared.{part}"] = torch.zeros_like(w[f"l0.mlp.shared.{part}"])
    same = P.routed_ff(mlp, one, "l0.mlp.", h)
    assert float((same - 1.7 * P.expert_ff(one, "l0.mlp.e0.", h)).abs().max()) < 1e-9 * float(same.abs().max())
    # prefix property: a position's logits do not depend on later tokens
    assert float(row_errors(P.forward(cfg, w, seq[:60]), want[:60]).max()) < 1e-12


def test_the_two_rotary_pairings_differ_and_turn_by_the_position():
    from plain import tofodra_plain as P
    v = torch.arange(1.0, 9.0, dtype=torch.float64)
    rot = {"base": 100.0, "dims": 4}
    a, b = P.rotate_pairs(v, 3, rot), P.rotate_halves(v, 3, rot)
    assert torch.equal(a[4:], v[4:]) and torch.equal(b[4:], v[4:]) and not torch.allclose(a, b)
    assert torch.allclose(P.rotate_pairs(v, 0, rot), v) and torch.allclose(P.rotate_halves(v, 0, rot), v)
    import math
    c, s = math.cos(3.0), math.sin(3.0)          # pair 0 turns at frequency 1
    assert abs(float(a[0]) - (1 * c - 2 * s)) < 1e-12 and abs(float(a[1]) - (2 * c + 1 * s)) < 1e-12
    assert abs(float(b[0]) - (1 * c - 3 * s)) < 1e-12 and abs(float(b[2]) - (3 * c + 1 * s)) < 1e-12
    # rotations keep dot products of equal positions and depend on the distance only
    q, k = torch.randn(8, dtype=torch.float64), torch.randn(8, dtype=torch.float64)
    rot8 = {"base": 50.0, "dims": 8}
    for f in (P.rotate_pairs, P.rotate_halves):
        assert abs(float(f(q, 9, rot8) @ f(k, 4, rot8)) - float(f(q, 15, rot8) @ f(k, 10, rot8))) < 1e-9
