"""Sazisun without a GPU: its configuration, the tensors its spec expects, which plan entries read another's cache,
the random-weights mode, and the plain implementation's own consistency (mechanisms against independent
restatements, a prompt against its own prefix)."""

import copy
import json
import math
import os

import pytest
import torch

import plain_sazisun as plain
from tiny_sazisun import SAZISUN, _att, _moe, _ssd, decisive_routing, draw_weights, one_layer, tensor_shapes

F = plain.F


@pytest.mark.parametrize("name", sorted(SAZISUN))
def test_the_spec_expects_exactly_the_tensors_the_design_names(name):
    from gllm_b200.config import load_config
    from gllm_b200.weights.random_init import expected_tensors_of

    cfg = SAZISUN[name]
    shapes = tensor_shapes(cfg)
    expected = expected_tensors_of(load_config(copy.deepcopy(cfg)))
    assert set(expected) == set(shapes)
    for key, exp in expected.items():
        assert tuple(exp.shape) == tuple(shapes[key]), key


def test_config_round_trip_and_errors():
    from gllm_b200.config import ConfigError, load_config
    from gllm_b200.config.sazisun_config import SazisunConfig

    cfg = load_config(copy.deepcopy(SAZISUN["A"]))
    assert isinstance(cfg, SazisunConfig) and cfg.hidden_size == 64 and cfg.vocab_size == 200
    assert cfg.norm_eps == 1e-5 and [layer.type for layer in cfg.layers] == ["attention", "mamba2", "attention", "mamba2"]
    again = load_config(cfg.to_dict())
    assert again.layers == cfg.layers and again.norm_eps == cfg.norm_eps

    def broken(change, base="A"):
        bad = copy.deepcopy(SAZISUN[base])
        change(bad)
        with pytest.raises(ConfigError):
            load_config(bad)

    broken(lambda c: c["layers"][1].update(type="other"))
    broken(lambda c: c["layers"][0]["mixer"].update(kv_heads=3))
    broken(lambda c: c["layers"][0]["mixer"].pop("softcap"))
    broken(lambda c: c["layers"][0]["mixer"].update(softcap=0.0))
    broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18))
    broken(lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("low"))
    broken(lambda c: c["layers"][1]["mixer"].update(groups=3))
    broken(lambda c: c["layers"][1]["mixer"].update(norm_groups=5))
    broken(lambda c: c["layers"][1]["mixer"].pop("conv"))
    broken(lambda c: c["layers"][0].update(mlp={"kind": "sparse", "ff": 8}))
    broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=5))            # only 2 groups of 2 stay
    broken(lambda c: c["layers"][1]["mlp"]["router"].pop("scale"))
    broken(lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3))
    broken(lambda c: c["layers"][2]["mixer"].update(kv_from=1))                # a recurrence has no keys
    broken(lambda c: c["layers"][2]["mixer"].update(kv_from=2))                # not an earlier layer
    broken(lambda c: c["layers"][2]["mixer"].update(dim=8))                    # other widths than the keys it reads
    broken(lambda c: c["layers"][3]["mixer"].update(kv_from=2), base="C")      # layer 2 has no keys of its own
    broken(lambda c: c.pop("norm"))


def test_spec_parts_and_shared_caches_follow_the_config():
    from gllm_b200.config import load_config
    from gllm_b200.config.registry import architecture_for

    cfg = load_config(copy.deepcopy(SAZISUN["C"]))
    spec = architecture_for("Sazisun").build_spec(cfg)
    assert [e.reads_cache_of for e in spec.plan] == [None, None, 0, 0]
    assert [layer.mixer.kind for layer in spec.layers] == ["differential_attention", "state_space_duality",
                                                           "differential_attention", "differential_attention"]
    assert spec.layers[2].mixer.params["own_kv"] is False and "k" not in spec.layers[2].mixer.names
    assert spec.layers[0].mixer.params["own_kv"] is True
    assert "feed_forward" not in spec.layers[3].parts and spec.head_name is None
    moe = spec.layers[0].feed_forward.params
    assert (moe["score"], moe["group_score"], moe["expert"], moe["renormalize"]) == ("softmax", "max", "relu_squared", True)
    assert moe["scale"] == 2.0 and moe["groups"] == 4 and moe["groups_kept"] == 3 and moe["shared_gate"] is True
    rot = spec.layers[0].mixer.params["position"].params
    assert rot["interleaved"] is True and rot["rotary_dim"] == 32 and rot["scaling"]["rope_type"] == "llama3"
    # no rotation at all: no position part
    cfg_b = load_config(copy.deepcopy(SAZISUN["B"]))
    assert architecture_for("Sazisun").build_spec(cfg_b).layers[3].mixer.params["position"] is None


def test_cache_requirements_pages_states_and_readers():
    """The attention layers that own keys share one page group per distinct shape, readers get the owner's pool layer
    and write nothing, the recurrences get two state tensors each."""
    from gllm_b200.cache.manager import CacheManager
    from gllm_b200.config import load_config
    from gllm_b200.config.registry import architecture_for
    from gllm_b200.models.decoder import DecoderModel

    cfg = load_config(copy.deepcopy(SAZISUN["C"]))
    model = DecoderModel(architecture_for("Sazisun").build_spec(cfg), torch.float32, "cpu")
    reqs = model.cache_requirements()
    assert reqs[0][0].tensors == ((2, 128), (2, 64)) and reqs[0][0].window is None
    assert [s.shape for s in reqs[1][1]] == [(4, 32, 64), (2, 4 * 32 + 2 * 64)]
    assert reqs[2][2] == 0 and reqs[3][2] == 0
    cache = CacheManager(reqs, block_size=8, num_blocks=6, max_batch_size=2, max_seq_len=48, dtype=torch.float32,
                         device="cpu")
    caches = cache.mixer_caches()
    assert caches[0].writes and not caches[2].writes and not caches[3].writes
    assert caches[2].pages.data_ptr() == caches[0].pages.data_ptr() == caches[3].pages.data_ptr()
    assert len(cache.groups) == 1 and len(caches[1].states) == 2


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    from gllm_b200.config import load_config
    from gllm_b200.weights.loader import open_checkpoint
    from gllm_b200.weights.random_init import expected_tensors_of, write_random_model

    cfg = load_config(copy.deepcopy(SAZISUN["B"]))
    folder = write_random_model(str(tmp_path / "m"), cfg, seed=5)
    open_checkpoint(folder).validate(expected_tensors_of(cfg))
    with open(os.path.join(folder, "config.json")) as f:
        assert load_config(json.load(f)).layers == cfg.layers


# ------------------------------------------------------------------ the plain implementation against restatements
def test_plain_frequencies_match_a_direct_restatement():
    rot = {"base": 500.0, "dims": 12, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    f = plain.scaled_frequencies(rot)
    for i in range(6):
        raw = 500.0 ** (-2.0 * i / 12)
        wavelength = 2 * math.pi / raw
        if wavelength < 16:
            want = raw
        elif wavelength > 64:
            want = raw / 8.0
        else:
            s = (64 / wavelength - 1.0) / 3.0
            want = (1 - s) * raw / 8.0 + s * raw
        assert abs(float(f[i]) - want) < 1e-12
    assert len({round(float(x / (500.0 ** (-2.0 * i / 12))), 6) for i, x in enumerate(f)}) > 1      # some are scaled


def test_plain_recurrence_equals_its_unrolled_sum():
    """``y_t = sum_{s <= t} (prod_{s < r <= t} a_r) dt_s (C_t . B_s) x_s + D x_t``: the recurrence written as the
    sum over earlier tokens it stands for."""
    g = torch.Generator().manual_seed(0)
    T, H, P, N = 9, 2, 3, 4
    x, B, C = (torch.randn(T, *s, generator=g, dtype=F) for s in ((H, P), (1, N), (1, N)))
    dt = torch.rand(T, H, generator=g, dtype=F) + 0.1
    A_log, D = torch.randn(H, generator=g, dtype=F) * 0.3, torch.randn(H, generator=g, dtype=F)
    y = plain.ssd_scan(x, B, C, dt, A_log, D, 2)
    for h in range(H):
        a = torch.exp(-torch.exp(A_log[h]) * dt[:, h])
        for t in range(T):
            want = D[h] * x[t, h]
            for s in range(t + 1):
                want = want + a[s + 1: t + 1].prod() * dt[s, h] * (C[t, 0] @ B[s, 0]) * x[s, h]
            assert torch.allclose(y[t, h], want, atol=1e-12)


def test_plain_routing_picks_within_the_best_groups_and_scales_the_weights():
    mlp = _moe(8, 8, 3, 2.5, (4, 2))
    w = {"r.router": torch.eye(8, dtype=F)}
    #            group 0      group 1      group 2      group 3
    h = torch.tensor([[0.0, 3.0, 2.5, 0.1, 2.9, 2.8, 0.3, 0.2]], dtype=F)
    chosen, weights = plain.route(h, mlp, w, "r")
    # groups score by their best expert: group 0 (3.0) and group 2 (2.9) stay; expert 2 (2.5, group 1) is out
    assert sorted(chosen[0].tolist()) == [1, 4, 5]
    assert abs(float(weights.sum()) - 2.5) < 1e-9
    s = torch.softmax(h, -1)[0]
    assert torch.allclose(weights[0], s[chosen[0]] / s[chosen[0]].sum() * 2.5)


def test_plain_difference_of_maps_and_prefix_consistency():
    """With the second map's weight at zero a head is plain capped softmax attention; and the logits of a prefix do
    not depend on what follows (everything is causal)."""
    cfg = one_layer(_att(2, 1, 8, 6, 0.3, 4, softcap=5.0, diff=0.25), width=32, vocab=40)
    w = draw_weights(cfg, seed=2)
    w = {k: v.to(F) for k, v in w.items()}
    m = cfg["layers"][0]["mixer"]
    g = torch.Generator().manual_seed(1)
    T = 7
    q, k, v = torch.randn(T, 2, 2, 8, generator=g, dtype=F), torch.randn(T, 1, 2, 8, generator=g, dtype=F), torch.randn(T, 1, 6, generator=g, dtype=F)
    p = torch.arange(T)
    o = plain.attend(q, k, v, p, p, m, 0.0, 1e-5).view(T, 2, 6)
    for t in range(T):
        s = 5.0 * torch.tanh((k[: t + 1, 0, 0] @ q[t, 1, 0]) * 0.3 / 5.0)
        a = torch.softmax(s, 0) @ v[: t + 1, 0]
        want = a / torch.sqrt((a * a).mean() + 1e-5) * 0.75
        assert torch.allclose(o[t, 1], want, atol=1e-12)
    tokens = list(range(3, 25))
    full = plain.forward(cfg, w, tokens)
    assert torch.allclose(plain.forward(cfg, w, tokens[:9]), full[:9], atol=1e-10)


def test_decisive_routing_leaves_wide_borders():
    for name in ("A", "C"):
        cfg = SAZISUN[name]
        w = decisive_routing(cfg, draw_weights(cfg, seed=4))
        tokens = torch.arange(cfg["vocab"]).tolist()[:64]
        _, layers = plain.forward(cfg, w, tokens, return_layers=True)
        assert torch.allclose(layers[-1][:, -4:].abs(), torch.full((64, 4), 3.0, dtype=F))     # the code survives
