"""Rotary position encoding with optional llama3 or yarn frequency scaling.

Frequencies ``theta ** (-2m / rotary_dim)`` for m = 0 .. rotary_dim/2 - 1 as
gllm/model/model.py:119-123; each head's first ``rotary_dim`` dims are rotated
in pairs of its two halves (gllm/model/layers/attention.py:91-118) by
``position * frequency``.  The reference rounds a cos/sin table to the model
dtype (gllm/model/model.py:126-128) and ignores ``rope_scaling``; here the
frequencies are computed in float64 on the host, rounded once to fp32, and the
angle, sine and cosine are fp32 inside the kernel.
"""

from __future__ import annotations

import math

import torch

from gllm_b200.parts.base import PositionEncoding, register_position_encoding


def scaled_inverse_frequencies(
    rotary_dim: int,
    theta: float,
    scaling: dict | None = None,
) -> list[float]:
    """Float64 frequencies, scaled as ``scaling["rope_type"]`` says ("llama3" or "yarn")."""
    half = rotary_dim // 2
    freqs = [float(theta) ** (-2.0 * m / rotary_dim) for m in range(half)]
    if not scaling:
        return freqs
    kind = scaling.get("rope_type")
    if kind == "yarn":
        # Pair m keeps its frequency below pair ``lo`` and has it divided by ``factor`` from pair ``hi`` on, with a
        # linear ramp between; lo and hi are the pairs that make ``beta_fast`` and ``beta_slow`` turns over the
        # original context: pair(t) = rotary_dim * ln(original / (2 pi t)) / (2 ln theta).
        factor = float(scaling["factor"])
        original = float(scaling["original_max_position_embeddings"])

        def pair_of(turns: float) -> float:
            return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(theta)))

        lo = max(math.floor(pair_of(float(scaling["beta_fast"]))), 0)
        hi = min(math.ceil(pair_of(float(scaling["beta_slow"]))), rotary_dim - 1)
        out = []
        for m, f in enumerate(freqs):
            ramp = min(max((m - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f / factor * ramp + f * (1.0 - ramp))
        return out
    if kind != "llama3":
        raise ValueError(f"rotary scaling {kind!r} is not supported")
    factor = float(scaling["factor"])
    low = float(scaling["low_freq_factor"])
    high = float(scaling["high_freq_factor"])
    original = float(scaling["original_max_position_embeddings"])
    out = []
    for f in freqs:
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            out.append(f)
        elif wavelength > original / low:
            out.append(f / factor)
        else:
            smooth = (original / wavelength - low) / (high - low)
            out.append((1.0 - smooth) * f / factor + smooth * f)
    return out


def rotary_magnitude(scaling: dict | None) -> float:
    """What sine and cosine are multiplied by: ``0.1 ln(factor) + 1`` under yarn scaling, 1 otherwise."""
    if scaling and scaling.get("rope_type") == "yarn":
        return 0.1 * math.log(float(scaling["factor"])) + 1.0
    return 1.0


@register_position_encoding("rotary")
class RotaryEncoding(PositionEncoding):
    graph_safe_portions = True

    def __init__(self, names=None, head_dim: int = 0, rotary_dim: int | None = None, theta: float = 10000.0,
                 scaling: dict | None = None, interleaved: bool = False):
        super().__init__(names)
        self.head_dim = int(head_dim)
        self.rotary_dim = int(rotary_dim if rotary_dim is not None else head_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self.theta = float(theta)
        self.scaling = dict(scaling) if scaling else None
        self.interleaved = bool(interleaved)
        self.inv_freq: torch.Tensor | None = None

    def load(self, get, dtype, device):
        freqs = scaled_inverse_frequencies(self.rotary_dim, self.theta, self.scaling)
        self.inv_freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(device)

    def rotary(self):
        return self.inv_freq, self.rotary_dim, self.interleaved

    def magnitude(self) -> float:
        """The multiplier of sine and cosine (1 unless the scaling kind has one)."""
        return rotary_magnitude(self.scaling)


@register_position_encoding("none")
class NoPositionEncoding(PositionEncoding):
    """Positions do not enter the mixer (keys and values are stored as they are)."""

    graph_safe_portions = True

    def __init__(self, names=None):
        super().__init__(names)
