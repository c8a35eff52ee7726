"""``Mifidra``'s own config.json keys as a typed configuration.

config.json names ``architecture`` (a string), ``vocab``, ``width``, ``norm.eps``, ``logit_scale``, ``layers``: one
entry per layer with ``type`` (which mixer: "parallel"), ``mixer`` (``left``: softmax attention, ``right``: gated
delta rule, ``left_scale``, ``right_scale``) and ``mlp`` (``{"kind": "dense", "ff": n}``,
``{"kind": "moe", "expert": {"ff": n}, "router": {"experts", "top", "groups": {"count", "keep"}}, "shared": {"ff": n}}``
or null for a layer without a feed-forward), and optionally ``loop`` (``start``, ``stop``, ``times``: layers
``start .. stop-1`` run ``times`` times in a row with the same weights).  Every size and constant the model uses
comes from here or from a tensor's shape; what a key that may be absent would switch on is off without it
(``rot.scaling``, ``router.groups``, ``mlp.shared``, ``loop``).  ``right`` may also name ``decay_rank`` and
``gate_rank``, the inner sizes of its two low-rank projections: a checkpoint's tensors give them, only the
random-weights mode needs them named.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any

from gllm_b200.config.model_config import DTYPE_NAMES, ConfigError, ModelConfig, as_eos, require

LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale", "rot")
RIGHT_KEYS = ("heads", "kv_heads", "dim", "vdim", "conv")
SCALING_KEYS = ("factor", "original", "fast", "slow")
FEED_FORWARD_KINDS = ("dense", "moe")


def _positive(where: str, d: dict, *keys: str) -> None:
    for key in keys:
        if int(require(d, key)) <= 0:
            raise ConfigError(f"{where}.{key} must be positive")


def _check_parallel(where: str, mixer: dict) -> None:
    left, right = require(mixer, "left"), require(mixer, "right")
    for side, keys, d in (("left", LEFT_KEYS, left), ("right", RIGHT_KEYS, right)):
        for key in keys:
            if key not in d:
                raise ConfigError(f"{where}.mixer.{side} lacks {key!r}")
        _positive(f"{where}.mixer.{side}", d, "heads", "kv_heads", "dim", "vdim")
        if int(d["heads"]) % int(d["kv_heads"]):
            raise ConfigError(f"{where}.mixer.{side}: heads is not a multiple of kv_heads")
    for key in ("left_scale", "right_scale"):
        float(require(mixer, key))
    rot = left["rot"]
    if "base" not in rot or "dims" not in rot:
        raise ConfigError(f"{where}.mixer.left.rot needs 'base' and 'dims'")
    dims = int(rot["dims"])
    if dims % 2 or dims < 0 or dims > int(left["dim"]):
        raise ConfigError(f"{where}.mixer.left.rot.dims must be even and at most dim")
    scaling = rot.get("scaling")
    if scaling is not None:
        for key in SCALING_KEYS:
            if key not in scaling:
                raise ConfigError(f"{where}.mixer.left.rot.scaling lacks {key!r}")
        if not float(scaling["factor"]) > 0:
            raise ConfigError(f"{where}.mixer.left.rot.scaling.factor must be positive")
    if int(right["conv"]) < 1:
        raise ConfigError(f"{where}.mixer.right.conv must be at least 1")


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
class MifidraLayer:
    type: str
    mixer: dict[str, Any]
    mlp: dict[str, Any] | None

    @classmethod
    def from_dict(cls, index: int, d: dict) -> "MifidraLayer":
        where = f"layers[{index}]"
        kind = require(d, "type")
        if kind != "parallel":
            raise ConfigError(f"{where}: unknown layer type {kind!r}; known: ['parallel']")
        mixer = require(d, "mixer")
        _check_parallel(where, mixer)
        mlp = d.get("mlp")
        if mlp is not None:
            _check_mlp(where, mlp)
        return cls(kind, copy.deepcopy(mixer), copy.deepcopy(mlp))

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": copy.deepcopy(self.mixer), "mlp": copy.deepcopy(self.mlp)}


@dataclass(frozen=True)
class MifidraConfig(ModelConfig):
    """A decoder whose layers norm every sublayer's input and result, mix tokens by softmax attention beside a
    gated delta rule, and feed forward densely or through routed experts; a stretch of layers may run several
    times, taking the embedding output in again before every further pass; the embedding table is the head."""

    layers: tuple[MifidraLayer, ...] = field(default_factory=tuple)
    norm_eps: float = 0.0
    logit_scale: float = 1.0
    # (start, stop, times) or None
    loop: tuple[int, int, int] | None = None

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "MifidraConfig":
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
        loop = d.get("loop")
        if loop is not None:
            start, stop, times = (int(require(loop, k)) for k in ("start", "stop", "times"))
            if not 0 <= start < stop <= len(layers) or times < 0:
                raise ConfigError("'loop' needs 0 <= start < stop <= number of layers and times >= 0")
            loop = (start, stop, times)
        return cls(
            architecture=str(arch), vocab_size=vocab, hidden_size=width, dtype=DTYPE_NAMES[dtype],
            eos_token_ids=as_eos(d.get("eos_token_id")),
            layers=tuple(MifidraLayer.from_dict(i, layer) for i, layer in enumerate(layers)),
            norm_eps=float(require(require(d, "norm"), "eps")),
            logit_scale=float(d.get("logit_scale", 1.0)),
            loop=loop,
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [layer.to_dict() for layer in self.layers],
            "logit_scale": self.logit_scale,
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab_size,
            "width": self.hidden_size,
            "torch_dtype": self.dtype,
        }
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
