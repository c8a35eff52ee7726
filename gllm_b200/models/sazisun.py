"""``Sazisun`` as a ModelSpec: a token embedding; pre-norm layers whose norm is ``dynamic_tanh`` (a scaled tanh with a
weight and a bias, no statistic); the mixer is ``differential_attention`` (two softmax maps per head over the same
values, subtracted; capped scores; neighbouring rotary pairs with wavelength-dependent frequency scaling; a per-head
norm and a sigmoid gate on the result; a layer may read an earlier layer's keys and values instead of projecting its
own) or ``state_space_duality`` (a short convolution, one decay per head and token, a gated norm over groups of
columns); the feed-forward is ``swiglu`` or ``routed_experts`` (softmax scores, groups scored by their best expert,
renormalized and scaled weights, experts with a squared ReLU, a shared expert behind a sigmoid gate); the embedding
table is the output head.

Tensor names: ``embed``, ``final.norm`` (+ ``.b``, ``.alpha``); layer ``i``: ``l<i>.norm1|norm2`` (+ ``.b``,
``.alpha``), ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from gllm_b200.config.registry import register_architecture
from gllm_b200.config.sazisun_config import SazisunConfig
from gllm_b200.models.spec import LayerSpec, ModelSpec, PartSpec, PlanEntry

# the design's fixed constant: what is added to the sum the chosen experts' scores are divided by
ROUTER_SUM_EPS = 1e-20


def _norm(width: int, name: str) -> PartSpec:
    return PartSpec("dynamic_tanh", dict(size=width), {"weight": name, "bias": name + ".b", "alpha": name + ".alpha"})


def _rotary(rot: dict, dim: int) -> PartSpec | None:
    if int(rot["dims"]) == 0:
        return None
    scaling = rot.get("scaling")
    if scaling is not None:
        scaling = {"rope_type": "llama3", "factor": scaling["factor"], "low_freq_factor": scaling["low"],
                   "high_freq_factor": scaling["high"], "original_max_position_embeddings": scaling["original"]}
    return PartSpec("rotary", dict(head_dim=dim, rotary_dim=int(rot["dims"]), theta=float(rot["base"]),
                                   scaling=scaling, interleaved=True))


def _attention(width: int, eps: float, m: dict, p: str) -> PartSpec:
    own = m.get("kv_from") is None
    names = {n: f"{p}.{n}" for n in ("q", "g", "o", "lq1", "lk1", "lq2", "lk2") + (("k", "v") if own else ())}
    return PartSpec(
        "differential_attention",
        dict(hidden_size=width, heads=m["heads"], kv_heads=m["kv_heads"], dk=m["dim"], dv=m["vdim"],
             scale=float(m["scale"]), softcap=float(m["softcap"]), diff=float(m["diff"]), eps=eps,
             position=_rotary(m["rot"], int(m["dim"])), own_kv=own),
        names,
    )


def _mamba2(width: int, eps: float, m: dict, p: str) -> PartSpec:
    names = {n: f"{p}.{n}" for n in ("in", "conv", "dt_bias", "A_log", "D", "norm", "o")}
    names["conv_bias"] = f"{p}.conv.b"
    return PartSpec(
        "state_space_duality",
        dict(hidden_size=width, heads=m["heads"], head_dim=m["vdim"], states=m["state"], groups=m["groups"],
             taps=m["conv"], norm_groups=m["norm_groups"], eps=eps),
        names,
    )


def _feed_forward(width: int, mlp: dict, p: str) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", dict(hidden_size=width, intermediate_size=mlp["ff"]),
                        {n: f"{p}.{n}" for n in ("gate", "up", "down")})
    router, groups, shared = mlp["router"], mlp["router"].get("groups"), mlp.get("shared")
    names = {"router": f"{p}.router", "expert": p + ".e{index}.{part}"}
    if shared is not None:
        names["shared_gate"] = f"{p}.shared.sg"
    return PartSpec(
        "routed_experts",
        dict(hidden_size=width, intermediate_size=mlp["expert"]["ff"], experts=router["experts"], top=router["top"],
             groups=None if groups is None else int(groups["count"]),
             groups_kept=None if groups is None else int(groups["keep"]),
             score="softmax", group_score="max", renormalize=True, renormalize_eps=ROUTER_SUM_EPS,
             scale=float(router["scale"]), expert="relu_squared", shared_gate=shared is not None,
             shared=None if shared is None else PartSpec(
                 "dense", dict(hidden_size=width, intermediate_size=shared["ff"], activation="relu_squared"),
                 {"up": f"{p}.shared.up", "down": f"{p}.shared.down"})),
        names,
    )


def build_sazisun_spec(cfg: SazisunConfig) -> ModelSpec:
    width, eps = cfg.hidden_size, cfg.norm_eps
    layers, plan = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer.mixer
        mixer = _attention(width, eps, m, f"{p}.mix") if layer.type == "attention" else _mamba2(width, eps, m, f"{p}.mix")
        parts = {"mixer_norm": _norm(width, f"{p}.norm1"), "mixer": mixer}
        if layer.mlp is not None:
            parts["feed_forward_norm"] = _norm(width, f"{p}.norm2")
            parts["feed_forward"] = _feed_forward(width, layer.mlp, f"{p}.mlp")
        layers.append(LayerSpec("prenorm", parts))
        # (plan entries and layers run one to one here, so a layer index is a plan index)
        reads = m.get("kv_from") if layer.type == "attention" else None
        plan.append(PlanEntry(i, reads_cache_of=None if reads is None else int(reads)))
    return ModelSpec(
        hidden_size=width,
        vocab_size=cfg.vocab_size,
        layers=tuple(layers),
        plan=tuple(plan),
        final_norm=_norm(width, "final.norm"),
        embedding_name="embed",
        head_name=None,
        eos_token_ids=cfg.eos_token_ids,
    )


register_architecture("Sazisun", SazisunConfig, build_sazisun_spec)
