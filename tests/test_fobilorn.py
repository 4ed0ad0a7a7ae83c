"""Fobilorn without a GPU: the configuration's checks, the plan (arrangement, parts, tensor names and shapes) and
properties of the oracle itself that the GPU tests rely on."""
import copy

import pytest
import torch

from fobilorn_cases import CASES, make_folder, oracle_view, row_errors, tokens


def test_the_plan_names_every_tensor_once():
    from hos_b200.model import weight_specs_for
    from hos_b200.registry import config_from_dict, plan_for
    cfg = config_from_dict(CASES["A"][0])
    plan = plan_for(cfg)
    assert [l.arrangement for l in plan.layers] == ["parallel_shared_norm"] * 4
    assert [c.cache_from for c in plan.schedule] == [None] * 4
    assert [l.mixer.params["value_mix"] and l.mixer.params["value_mix"]["role"] for l in plan.layers] == \
        [None, "source", "mixed", "mixed"]
    assert plan.layers[0].mixer.params["keep_first"] == 3 and plan.layers[3].mixer.params["window"] is None
    specs = {s.name: s for s in weight_specs_for(cfg)}
    names = {n: tuple(s.shape) for n, s in specs.items()}
    assert names["embed"] == (211, 72) and names["bigram"] == (14, 72) and names["head"] == (211, 72)
    assert names["embed.norm"] == (72,) and names["embed.norm.b"] == (72,) and names["embed.norm.alpha"] == ()
    assert names["l0.mix.q"] == (48, 72) and names["l0.mix.q.norm"] == (48,) and names["l0.mix.k.norm"] == (16,)
    assert names["l0.mix.v"] == (24, 72) and names["l0.mix.g"] == (3, 72) and names["l0.mix.o"] == (72, 72)
    assert specs["l0.mix.vmix"].optional and specs["l1.mix.vmix"].optional and not specs["l2.mix.vmix"].optional
    assert "l0.norm2" not in names and "l0.mix.sink" not in names
    assert names["l1.mlp.router"] == (5, 72) and names["l1.mlp.e4.down"] == (72, 40) and names["l1.mlp.shared.up"] == (24, 72)
    assert "l2.mlp.gate" not in names and "l3.mlp.shared.gate" not in names and names["l0.mlp.gate"] == (56, 72)
    assert config_from_dict(cfg.to_dict()) == cfg
    bare = config_from_dict(CASES["C"][0])
    assert plan_for(bare).embedding.kind == "scaled_embedding" and "bigram" not in {s.name for s in weight_specs_for(bare)}


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=16), "differ"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(keep_first=-1), "keep_first"),
    (lambda c: c["layers"][0].update(type="recurrence"), "type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="sparse"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][1]["mlp"].pop("expert"), "expert"),
    (lambda c: c["embedding"]["bigram"].pop("mul_cur"), "mul_cur"),
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


def test_a_checkpoint_may_lack_the_blending_scalar_where_it_is_not_used(tmp_path):
    """The layer whose values the others blend in, and layers that blend nothing, do not use the scalar: a checkpoint
    with or without it loads; a blending layer's is required."""
    from hos_b200.errors import WeightMismatchError
    from hos_b200.model import weight_specs_for
    from hos_b200.registry import config_from_dict
    from hos_b200.weights.loader import check_against

    class Names:
        def __init__(self, specs, drop):
            self.s = {s.name: s for s in specs if s.name not in drop}

        def names(self):
            return list(self.s)

        def info(self, n):
            return torch.bfloat16, tuple(self.s[n].shape)
    specs = weight_specs_for(config_from_dict(CASES["A"][0]))
    check_against(specs, Names(specs, ()))
    check_against(specs, Names(specs, ("l0.mix.vmix", "l1.mix.vmix")))
    with pytest.raises(WeightMismatchError):
        check_against(specs, Names(specs, ("l2.mix.vmix",)))


def test_the_oracle_feels_every_mechanism(tmp_path):
    """What the GPU tests compare with must move when a mechanism is taken away or shifted by one: the one in the
    denominator, the window's edge, the kept keys' edge, the blending of values, the pair table, the router's weight on
    the input."""
    from plain import fobilorn_plain as P
    folder = make_folder(tmp_path, CASES["A"][0], CASES["A"][1], "A")
    cfg, w = oracle_view(folder)
    seq = tokens(1, 110, cfg["vocab"])
    want = P.forward(cfg, w, seq)
    assert float(row_errors(P.forward(cfg, w, seq, sink=False), want).median()) > 2e-3
    for key, d in (("size", 1), ("size", -1), ("keep_first", 1), ("keep_first", -1)):
        def edit(m):
            if m.get("mask") and m["mask"].get(key, 0) + d > 0:
                m["mask"] = dict(m["mask"], **{key: m["mask"].get(key, 0) + d})
            return m
        assert float(row_errors(P.forward(cfg, w, seq, edit=edit)[80:], want[80:]).median()) > 2e-3, (key, d)
    w2 = dict(w)
    w2["l2.mix.vmix"] = torch.zeros((), dtype=torch.float64)
    assert float(row_errors(P.forward(cfg, w2, seq), want).median()) > 2e-3
    w3 = dict(w)
    w3["bigram"] = torch.zeros_like(w["bigram"])
    assert float(row_errors(P.forward(cfg, w3, seq), want).median()) > 2e-3
    # the weight on the input is not the weight on the output: the experts are not linear
    h = torch.randn(4, cfg["width"], dtype=torch.float64)
    mlp = cfg["layers"][1]["mlp"]
    inside = P.routed_ff(mlp, w, "l1.mlp.", h)
    outside = torch.zeros_like(h)
    for t in range(4):
        s = torch.sigmoid(h[t] @ w["l1.mlp.router"].T)
        for e in sorted(range(5), key=lambda e: (-float(s[e]), e))[:2]:
            outside[t] += s[e] * P.gated_ff(w, f"l1.mlp.e{e}.", h[t][None])[0]
    outside = outside + P.gated_ff(w, "l1.mlp.shared.", h)
    assert float((inside - outside).abs().max()) > 1e-3 * float(inside.abs().max())
    # prefix property: a position's logits do not depend on later tokens
    assert float(row_errors(P.forward(cfg, w, seq[:60]), want[:60]).max()) < 1e-12
