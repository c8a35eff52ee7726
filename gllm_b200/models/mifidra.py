"""``Mifidra`` as a ModelSpec: a token embedding; layers of the ``sandwich`` block (an RMS norm before and one after
each sublayer: ``x += norm_b(sublayer(norm_a(x)))``); the mixer is ``parallel``: softmax ``attention`` (grouped
heads, neighbouring rotary pairs with wavelength-dependent frequency scaling whose sine and cosine carry a
multiplier, queries and keys divided by their root mean square AFTER the rotation, key and value widths of
their own) beside ``gated_delta_rule`` (short convolutions, unit-length queries and keys, a decay per key
channel, a corrected write); the feed-forward is ``swiglu`` with biases or ``routed_experts`` (sigmoid scores, a
correction that only steers the choice, groups of experts, a shared expert); layers ``loop.start .. loop.stop-1``
run ``loop.times`` times with the same weights, every pass with caches and states of its own, the embedding
output being added to the residual before every pass but the first; the embedding table is the output head and
the logits are scaled.

Tensor names: ``embed``, ``final.norm``; layer ``i``: ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.left.*``,
``l<i>.mix.right.*``, ``l<i>.mlp.*``.
"""

from __future__ import annotations

from gllm_b200.config.mifidra_config import MifidraConfig
from gllm_b200.config.registry import register_architecture
from gllm_b200.models.spec import LayerSpec, ModelSpec, PartSpec, PlanEntry

# the design's fixed constants: what is added under the root when queries and keys of the delta rule are made
# unit vectors
UNIT_NORM_EPS = 1e-6


def _rotary(rot: dict, head_dim: int) -> PartSpec | None:
    if int(rot["dims"]) == 0:
        return None
    scaling = rot.get("scaling")
    if scaling is not None:
        scaling = {"rope_type": "yarn", "factor": scaling["factor"], "beta_fast": scaling["fast"],
                   "beta_slow": scaling["slow"], "original_max_position_embeddings": scaling["original"]}
    return PartSpec("rotary", dict(head_dim=head_dim, rotary_dim=int(rot["dims"]), theta=float(rot["base"]),
                                   scaling=scaling, interleaved=True))


def _left(width: int, eps: float, m: dict, p: str) -> PartSpec:
    return PartSpec(
        "attention",
        dict(hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
             value_dim=m["vdim"], scale=m["scale"], unit_norm_after_rotation_eps=eps, pad_heads=True,
             position=_rotary(m["rot"], int(m["dim"]))),
        {n: f"{p}.{n}" for n in ("q", "k", "v", "o")},
    )


def _right(width: int, eps: float, m: dict, p: str) -> PartSpec:
    names = {n: f"{p}.{n}" for n in ("q", "k", "v", "b", "A_log", "norm", "a1", "a2", "dt_bias", "g1", "g2", "o")}
    names.update({f"{n}_conv": f"{p}.{n}.conv" for n in ("q", "k", "v")})
    return PartSpec(
        "gated_delta_rule",
        dict(hidden_size=width, heads=m["heads"], kv_heads=m["kv_heads"], dk=m["dim"], dv=m["vdim"],
             taps=m["conv"], eps=eps, unit_eps=UNIT_NORM_EPS, q_scale=float(m["dim"]) ** -0.5,
             decay_rank=m.get("decay_rank"), gate_rank=m.get("gate_rank")),
        names,
    )


def _glu_names(p: str, bias: bool) -> dict:
    names = {n: f"{p}.{n}" for n in ("gate", "up", "down")}
    if bias:
        names.update({f"{n}_bias": f"{p}.{n}.b" for n in ("gate", "up", "down")})
    return names


def _feed_forward(width: int, mlp: dict, p: str) -> PartSpec:
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", dict(hidden_size=width, intermediate_size=mlp["ff"], bias=True), _glu_names(p, True))
    router, groups, shared = mlp["router"], mlp["router"].get("groups"), mlp.get("shared")
    names = {"router": f"{p}.router", "correction": f"{p}.correction", "expert": p + ".e{index}.{part}"}
    return PartSpec(
        "routed_experts",
        dict(hidden_size=width, intermediate_size=mlp["expert"]["ff"], experts=router["experts"], top=router["top"],
             groups=None if groups is None else int(groups["count"]),
             groups_kept=None if groups is None else int(groups["keep"]),
             score="sigmoid", renormalize=False, correction=True,
             shared=None if shared is None else PartSpec(
                 "swiglu", dict(hidden_size=width, intermediate_size=shared["ff"]), _glu_names(p + ".shared", False))),
        names,
    )


def layer_order(cfg: MifidraConfig) -> list[tuple[int, bool]]:
    """(layer, the embedding output is added before it) in running order."""
    n = len(cfg.layers)
    if cfg.loop is None:
        return [(i, False) for i in range(n)]
    start, stop, times = cfg.loop
    order = [(i, False) for i in range(start)]
    for t in range(times):
        order += [(i, t > 0 and i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def build_mifidra_spec(cfg: MifidraConfig) -> ModelSpec:
    width, eps = cfg.hidden_size, cfg.norm_eps

    def norm(weight: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(size=width, eps=eps), {"weight": weight})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer.mixer
        parts = {
            "mixer_norm": norm(f"{p}.norm1"),
            "mixer": PartSpec("parallel", dict(left=_left(width, eps, m["left"], f"{p}.mix.left"),
                                               right=_right(width, eps, m["right"], f"{p}.mix.right"),
                                               left_scale=float(m["left_scale"]), right_scale=float(m["right_scale"]))),
            "mixer_post_norm": norm(f"{p}.norm1b"),
        }
        if layer.mlp is not None:
            parts["feed_forward_norm"] = norm(f"{p}.norm2")
            parts["feed_forward"] = _feed_forward(width, layer.mlp, f"{p}.mlp")
            parts["feed_forward_post_norm"] = norm(f"{p}.norm2b")
        layers.append(LayerSpec("sandwich", parts))
    return ModelSpec(
        hidden_size=width,
        vocab_size=cfg.vocab_size,
        layers=tuple(layers),
        plan=tuple(PlanEntry(i, adds_embedding=adds) for i, adds in layer_order(cfg)),
        final_norm=norm("final.norm"),
        embedding_name="embed",
        head_name=None,
        eos_token_ids=cfg.eos_token_ids,
        logit_scale=None if cfg.logit_scale == 1.0 else cfg.logit_scale,
    )


register_architecture("Mifidra", MifidraConfig, build_mifidra_spec)
