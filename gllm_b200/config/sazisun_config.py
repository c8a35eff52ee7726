"""``Sazisun``'s own config.json keys as a typed configuration.

config.json names ``architecture`` (a string), ``vocab``, ``width``, ``norm.eps`` and ``layers``: one entry per
layer with ``type`` (which mixer: "attention" or "mamba2"), ``mixer`` (that mixer's sizes and constants) and ``mlp``
(``{"kind": "dense", "ff": n}``, ``{"kind": "moe", "expert": {"ff": n}, "router": {"experts", "top", "scale",
"groups": {"count", "keep"}}, "shared": {"ff": n}}`` or null for a layer without a feed-forward).

``attention``: ``heads``, ``kv_heads``, ``dim`` (width of one of a head's two query / key maps), ``vdim``, ``scale``,
``softcap``, ``diff``, ``rot`` (``base``, ``dims``, optionally ``scaling``: ``factor``, ``low``, ``high``,
``original``) and optionally ``kv_from``: the index of an earlier attention layer whose keys and values this layer
reads instead of projecting its own.  ``mamba2``: ``heads``, ``vdim``, ``state``, ``groups``, ``conv``,
``norm_groups``.  Every size and constant the model uses comes from here or from a tensor's shape; what a key that
may be absent would switch on is off without it (``rot.scaling``, ``kv_from``, ``router.groups``, ``mlp.shared``).
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any

from gllm_b200.config.model_config import DTYPE_NAMES, ConfigError, ModelConfig, as_eos, require

ATTENTION_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale", "softcap", "diff", "rot")
MAMBA2_KEYS = ("heads", "vdim", "state", "groups", "conv", "norm_groups")
SCALING_KEYS = ("factor", "low", "high", "original")
LAYER_TYPES = ("attention", "mamba2")
FEED_FORWARD_KINDS = ("dense", "moe")


def _positive(where: str, d: dict, *keys: str) -> None:
    for key in keys:
        if int(require(d, key)) <= 0:
            raise ConfigError(f"{where}.{key} must be positive")


def _check_attention(where: str, m: dict) -> None:
    for key in ATTENTION_KEYS:
        if key not in m:
            raise ConfigError(f"{where}.mixer lacks {key!r}")
    _positive(f"{where}.mixer", m, "heads", "kv_heads", "dim", "vdim")
    if int(m["heads"]) % int(m["kv_heads"]):
        raise ConfigError(f"{where}.mixer: heads is not a multiple of kv_heads")
    if not float(m["softcap"]) > 0:
        raise ConfigError(f"{where}.mixer.softcap must be positive")
    float(m["scale"]), float(m["diff"])
    rot = m["rot"]
    if "base" not in rot or "dims" not in rot:
        raise ConfigError(f"{where}.mixer.rot needs 'base' and 'dims'")
    dims = int(rot["dims"])
    if dims % 2 or dims < 0 or dims > int(m["dim"]):
        raise ConfigError(f"{where}.mixer.rot.dims must be even and at most dim")
    scaling = rot.get("scaling")
    if scaling is not None:
        for key in SCALING_KEYS:
            if key not in scaling:
                raise ConfigError(f"{where}.mixer.rot.scaling lacks {key!r}")
        if not float(scaling["factor"]) > 0 or float(scaling["high"]) == float(scaling["low"]):
            raise ConfigError(f"{where}.mixer.rot.scaling needs a positive factor and high != low")


def _check_mamba2(where: str, m: dict) -> None:
    for key in MAMBA2_KEYS:
        if key not in m:
            raise ConfigError(f"{where}.mixer lacks {key!r}")
    _positive(f"{where}.mixer", m, *MAMBA2_KEYS)
    if int(m["heads"]) % int(m["groups"]):
        raise ConfigError(f"{where}.mixer: heads is not a multiple of groups")
    if (int(m["heads"]) * int(m["vdim"])) % int(m["norm_groups"]):
        raise ConfigError(f"{where}.mixer: heads * vdim is not a multiple of norm_groups")


def _check_mlp(where: str, mlp: dict) -> None:
    kind = mlp.get("kind")
    if kind not in FEED_FORWARD_KINDS:
        raise ConfigError(f"{where}.mlp: unknown kind {kind!r}; known: {list(FEED_FORWARD_KINDS)}")
    if kind == "dense":
        _positive(f"{where}.mlp", mlp, "ff")
        return
    _positive(f"{where}.mlp.expert", require(mlp, "expert"), "ff")
    router = require(mlp, "router")
    _positive(f"{where}.mlp.router", router, "experts", "top")
    float(require(router, "scale"))
    experts, top = int(router["experts"]), int(router["top"])
    allowed = experts
    groups = router.get("groups")
    if groups is not None:
        _positive(f"{where}.mlp.router.groups", groups, "count", "keep")
        count, keep = int(groups["count"]), int(groups["keep"])
        if experts % count or keep > count:
            raise ConfigError(f"{where}.mlp.router.groups: the experts form 'count' equal groups of which 'keep' <= "
                              "'count' stay")
        allowed = keep * (experts // count)
    if top > allowed:
        raise ConfigError(f"{where}.mlp.router.top exceeds the experts that can be chosen")
    if mlp.get("shared") is not None:
        _positive(f"{where}.mlp.shared", mlp["shared"], "ff")


@dataclass(frozen=True)
class SazisunLayer:
    type: str
    mixer: dict[str, Any]
    mlp: dict[str, Any] | None

    @classmethod
    def from_dict(cls, index: int, d: dict) -> "SazisunLayer":
        where = f"layers[{index}]"
        kind = require(d, "type")
        if kind not in LAYER_TYPES:
            raise ConfigError(f"{where}: unknown layer type {kind!r}; known: {list(LAYER_TYPES)}")
        mixer = require(d, "mixer")
        (_check_attention if kind == "attention" else _check_mamba2)(where, mixer)
        mlp = d.get("mlp")
        if mlp is not None:
            _check_mlp(where, mlp)
        return cls(kind, copy.deepcopy(mixer), copy.deepcopy(mlp))

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": copy.deepcopy(self.mixer), "mlp": copy.deepcopy(self.mlp)}


def _check_shared_keys(layers: tuple[SazisunLayer, ...]) -> None:
    """A layer that reads another's keys and values names an earlier attention layer that projects its own and has
    the same head counts, widths and rotation."""
    for i, layer in enumerate(layers):
        j = layer.mixer.get("kv_from") if layer.type == "attention" else None
        if j is None:
            continue
        j = int(j)
        if not 0 <= j < i or layers[j].type != "attention" or layers[j].mixer.get("kv_from") is not None:
            raise ConfigError(f"layers[{i}].mixer.kv_from must name an earlier attention layer with keys of its own")
        mine, theirs = layer.mixer, layers[j].mixer
        if any(mine[k] != theirs[k] for k in ("kv_heads", "dim", "vdim", "rot")):
            raise ConfigError(f"layers[{i}] reads the keys of layers[{j}], whose kv_heads, dim, vdim or rot differ")


@dataclass(frozen=True)
class SazisunConfig(ModelConfig):
    """A decoder of pre-norm layers with a norm that takes no statistic (a scaled tanh), whose mixers are
    differential attention (optionally over an earlier layer's keys and values) or a state-space-duality
    recurrence, and whose feed-forwards are gated dense ones or routed experts; the embedding table is the head."""

    layers: tuple[SazisunLayer, ...] = field(default_factory=tuple)
    norm_eps: float = 0.0

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "SazisunConfig":
        arch = d.get("architecture") or (d.get("architectures") or [None])[0]
        layers = require(d, "layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("'layers' must be a non-empty list")
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if dtype not in DTYPE_NAMES:
            raise ConfigError(f"unsupported dtype {dtype!r}")
        vocab, width = int(require(d, "vocab")), int(require(d, "width"))
        if vocab <= 0 or width <= 0:
            raise ConfigError("'vocab' and 'width' must be positive")
        parsed = tuple(SazisunLayer.from_dict(i, layer) for i, layer in enumerate(layers))
        _check_shared_keys(parsed)
        return cls(
            architecture=str(arch), vocab_size=vocab, hidden_size=width, dtype=DTYPE_NAMES[dtype],
            eos_token_ids=as_eos(d.get("eos_token_id")), layers=parsed,
            norm_eps=float(require(require(d, "norm"), "eps")),
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [layer.to_dict() for layer in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab_size,
            "width": self.hidden_size,
            "torch_dtype": self.dtype,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
