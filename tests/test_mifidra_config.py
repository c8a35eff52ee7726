"""Mifidra without a GPU: its configuration, the tensors its spec expects, the order in which a repeated stretch
runs, and the plain implementation's own consistency (a whole prompt against the same tokens in portions, the
mechanisms against independent restatements)."""

import copy
import math

import pytest
import torch

import plain_mifidra as plain
from tiny_mifidra import MIFIDRA, decisive_routing, draw_weights, one_layer


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_spec_expects_exactly_the_tensors_the_design_names(name):
    from gllm_b200.config import load_config
    from gllm_b200.weights.random_init import expected_tensors_of

    cfg = MIFIDRA[name]
    weights = draw_weights(cfg, seed=1)
    expected = expected_tensors_of(load_config(copy.deepcopy(cfg)))
    assert set(expected) == set(weights)
    for key, exp in expected.items():
        want = tuple(weights[key].shape)
        assert len(exp.shape) == len(want) and all(a in (-1, b) for a, b in zip(exp.shape, want)), key


def test_config_round_trip_and_errors():
    from gllm_b200.config import ConfigError, load_config
    from gllm_b200.config.mifidra_config import MifidraConfig

    cfg = load_config(copy.deepcopy(MIFIDRA["A"]))
    assert isinstance(cfg, MifidraConfig) and cfg.hidden_size == 64 and cfg.vocab_size == 200
    assert cfg.loop == (0, 2, 3) and cfg.logit_scale == 0.5
    again = load_config(cfg.to_dict())
    assert again.layers == cfg.layers and again.norm_eps == cfg.norm_eps and again.loop == cfg.loop
    assert load_config(copy.deepcopy(MIFIDRA["B"])).loop is None

    def broken(change):
        bad = copy.deepcopy(MIFIDRA["A"])
        change(bad)
        with pytest.raises(ConfigError):
            load_config(bad)

    broken(lambda c: c["layers"][1].update(type="other"))
    broken(lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3))
    broken(lambda c: c["layers"][0]["mixer"]["right"].pop("conv"))
    broken(lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=34))
    broken(lambda c: c["layers"][0].update(mlp={"kind": "sparse", "ff": 8}))
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=5))            # only 2 groups of 2 stay
    broken(lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3))
    broken(lambda c: c.update(loop={"start": 2, "stop": 2, "times": 2}))
    broken(lambda c: c.pop("norm"))


def test_spec_layers_and_running_order_follow_the_config():
    from gllm_b200.config import load_config
    from gllm_b200.config.registry import architecture_for

    spec = architecture_for("Mifidra").build_spec(load_config(copy.deepcopy(MIFIDRA["A"])))
    assert {layer.block for layer in spec.layers} == {"sandwich"}
    assert [layer.parts["mixer"].kind for layer in spec.layers] == ["parallel"] * 4
    assert [layer.parts["feed_forward"].kind if "feed_forward" in layer.parts else None for layer in spec.layers] == [
        "swiglu", "routed_experts", None, "routed_experts"]
    assert [(e.layer, e.adds_embedding) for e in spec.plan] == [
        (0, False), (1, False), (0, True), (1, False), (0, True), (1, False), (2, False), (3, False)]
    assert [(e.layer, e.adds_embedding) for e in spec.plan] == plain.layer_runs(MIFIDRA["A"])
    assert spec.head_name is None and spec.logit_scale == 0.5
    left = spec.layers[1].parts["mixer"].params["left"]
    assert left.params["value_dim"] == 40 and left.params["head_dim"] == 24 and left.params["scale"] == 0.25
    assert left.params["position"].params["rotary_dim"] == 16 and left.params["position"].params["interleaved"]
    routed = spec.layers[1].parts["feed_forward"].params
    assert (routed["experts"], routed["top"], routed["groups"], routed["groups_kept"]) == (8, 2, 4, 2)
    assert spec.layers[3].parts["feed_forward"].params["groups"] is None
    whole = architecture_for("Mifidra").build_spec(load_config(copy.deepcopy(MIFIDRA["C"])))
    assert [(e.layer, e.adds_embedding) for e in whole.plan] == [(0, False), (1, False), (0, True), (1, False)]
    once = architecture_for("Mifidra").build_spec(load_config(copy.deepcopy(MIFIDRA["D"])))
    assert [(e.layer, e.adds_embedding) for e in once.plan] == [(0, False), (1, False)]


def test_engine_frequencies_match_the_plain_ones():
    """The rotary part's table against the plain frequencies, with and without scaling, also where the ramp's ends
    fall outside the pairs (clamped) and where they coincide."""
    from gllm_b200.parts.base import POSITION_ENCODINGS, build_part
    from gllm_b200.models.mifidra import _rotary

    for rot in ({"base": 10000.0, "dims": 32},
                {"base": 20000.0, "dims": 64, "scaling": {"factor": 6.0, "original": 256, "fast": 16.0, "slow": 2.0}},
                {"base": 50.0, "dims": 10, "scaling": {"factor": 16.0, "original": 32, "fast": 4.0, "slow": 0.5}},
                {"base": 1e6, "dims": 16, "scaling": {"factor": 2.0, "original": 4096, "fast": 1e-3, "slow": 1e-4}},
                {"base": 100.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 2.0, "slow": 2.0}}):
        part = build_part(POSITION_ENCODINGS, _rotary(rot, 64))
        part.load(lambda *a: None, torch.float32, "cpu")
        inv_freq, rotary_dim, interleaved = part.rotary()
        f, mult = plain.yarn_frequencies(rot)
        assert rotary_dim == rot["dims"] and interleaved
        assert torch.allclose(inv_freq.double().cpu(), f, rtol=2e-6, atol=0)
        assert abs(part.magnitude() - mult) < 1e-7


@pytest.mark.parametrize("name", ["A", "B"])
def test_plain_whole_prompt_equals_plain_portions(name):
    cfg = MIFIDRA[name]
    w = draw_weights(cfg, seed=2)
    toks = torch.randint(0, cfg["vocab"], (23,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = plain.forward(cfg, w, toks)
    state = plain.PlainState(cfg)
    parts = [plain.forward(cfg, w, toks[a:b], state) for a, b in ((0, 5), (5, 6), (6, 8), (8, 20), (20, 23))]
    assert torch.allclose(torch.cat(parts, 0), whole, rtol=0, atol=1e-9)


def test_plain_delta_rule_against_its_closed_form():
    """Without decay and with beta 1 and orthonormal keys the state ends as sum_t k_t v_t^T, whatever was written
    under the same key before is replaced, and a read with key j returns value j."""
    dk, dv = 6, 4
    keys = torch.linalg.qr(torch.randn(dk, dk, dtype=plain.F, generator=torch.Generator().manual_seed(0)))[0]
    T = 9
    k = keys[[0, 1, 2, 0, 3, 1, 4, 5, 2]][:, None, :]
    v = torch.randn(T, 1, dv, dtype=plain.F, generator=torch.Generator().manual_seed(1))
    S = torch.zeros(1, dk, dv, dtype=plain.F)
    o = plain.delta_rule(k.clone(), k, v, torch.ones(T, 1, dk, dtype=plain.F), torch.ones(T, 1, dtype=plain.F), S)
    assert torch.allclose(o, v, atol=1e-12)                     # the read-out sees the token's own write
    last = {0: 3, 1: 5, 2: 8, 3: 4, 4: 6, 5: 7}
    want = sum(torch.outer(keys[j], v[t, 0]) for j, t in last.items())
    assert torch.allclose(S[0], want, atol=1e-12)
    # a decay acts on the rows of the state that belong to key channels, before the write
    S = torch.ones(1, dk, dv, dtype=plain.F)
    g = torch.linspace(0.1, 0.9, dk, dtype=plain.F).view(1, 1, dk)
    plain.delta_rule(torch.zeros(1, 1, dk, dtype=plain.F), torch.zeros(1, 1, dk, dtype=plain.F),
                     torch.zeros(1, 1, dv, dtype=plain.F), g, torch.ones(1, 1, dtype=plain.F), S)
    assert torch.allclose(S[0], g.view(dk, 1).expand(dk, dv))


def test_plain_routing_by_hand():
    """Eight experts in four groups of which two stay; the correction steers the choice and not the weights; a
    group of excluded experts loses even against negative choice scores."""
    router = {"experts": 8, "top": 3, "groups": {"count": 4, "keep": 2}}
    z = torch.tensor([[4.0, -4.0, 0.5, 0.4, -1.0, 3.0, 0.0, 0.1]], dtype=plain.F)
    w = {"m.router": torch.eye(8, dtype=plain.F), "m.correction": torch.tensor(
        [0.0, 0.0, 0.0, 0.0, 0.0, -2.0, -3.0, -3.0], dtype=plain.F)}
    chosen, weights = plain.route(z, w, "m", router)
    # group scores: 0.98+0.02 = 1.0 | 0.62+0.60 = 1.22 | 0.27-1.05 = -0.78 | -2.5-2.48: groups 1 and 0 stay; top 3
    # of experts 0..3 by choice score
    assert sorted(chosen[0].tolist()) == [0, 2, 3]
    s = torch.sigmoid(z[0])
    assert torch.allclose(weights[0].sort().values, s[[0, 2, 3]].sort().values)
    # all choice scores negative: the best groups' experts are still chosen over the excluded ones
    w["m.correction"] = torch.tensor([-5.0, -5.0, -9.0, -9.0, -2.0, -2.0, -9.0, -9.0], dtype=plain.F)
    chosen, _ = plain.route(z, w, "m", router)
    assert set(chosen[0].tolist()) <= {0, 1, 4, 5}


def test_decisive_routing_leaves_wide_margins():
    cfg = MIFIDRA["A"]
    w = decisive_routing(cfg, draw_weights(cfg, seed=5))
    toks = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(3)).tolist()
    margins: list = []
    plain.forward(cfg, w, toks, margins=margins)
    assert margins and min(margins) > 5e-3


def test_one_layer_helper_and_scales():
    cfg = one_layer(left_scale=0.0, right_scale=1.0)
    w = draw_weights(cfg, seed=4)
    toks = list(range(12))
    a = plain.forward(cfg, w, toks)
    w2 = dict(w)
    w2["l0.mix.left.v"] = w["l0.mix.left.v"] * 3.0            # the left half is switched off: nothing changes
    assert torch.allclose(plain.forward(cfg, w2, toks), a)
    assert math.isfinite(float(a.abs().max()))
