"""Small Mifidra configurations for the tests, as raw config.json dicts, and a writer that draws their weights here
(not through the engine's random-weights mode), tensor by tensor under the names the design gives them.

The configurations differ in every size and option: with and without a repeated stretch (at the start, in the middle, over the
whole model, a single pass), layers without a feed-forward, dense and routed feed-forwards (with and without
groups, groups of one expert, with and without a shared expert, one expert per token), key and value widths that
differ on the left (both ways) and on the right, grouped / multi-query / one head per key head on both sides,
convolutions of 1 to 4 taps, rotations over the whole head, a part of it and none, with and without frequency
scaling, sizes that are no multiple of 8, low ranks that are no multiple of 8, head widths that the tensor-core
kernels take and ones they do not."""

from __future__ import annotations

import json
import math
import os

import torch
from safetensors.torch import save_file


def _left(heads, kv_heads, dim, vdim, scale, dims, base=10000.0, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}


def _right(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def _layer(left, right, mlp, left_scale=1.0, right_scale=1.0):
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


# the first two layers run three times; grouped heads on the left, key and value widths that differ; grouped
# routing with a shared expert; a dense layer; a layer without a feed-forward
MIFIDRA_A = {
    "architecture": "Mifidra", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 0.5,
    "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [
        _layer(_left(4, 2, 32, 16, 0.2, 32, scaling=(4.0, 64, 8.0, 1.0)), _right(4, 2, 16, 8, 3), _dense(96), 0.7, 0.6),
        _layer(_left(2, 1, 24, 40, 0.25, 16, base=500.0), _right(2, 2, 8, 24, 4), _moe(32, 8, 2, (4, 2), 48), 1.2, 0.4),
        _layer(_left(4, 4, 16, 16, 0.3, 16), _right(3, 1, 16, 16, 2), None, 0.5, 1.0),
        _layer(_left(2, 2, 32, 32, 0.15, 8), _right(2, 1, 32, 16, 3), _moe(24, 6, 3), 1.0, 1.0),
    ],
}
# no repeated stretch; sizes that are no multiple of 8; no rotation in one layer; a convolution of one tap; groups of
# one expert; one expert per token
MIFIDRA_B = {
    "architecture": "Mifidra", "vocab": 131, "width": 44, "norm": {"eps": 3e-6}, "logit_scale": 1.0,
    "layers": [
        _layer(_left(3, 3, 12, 20, 0.3, 0), _right(3, 3, 10, 6, 1), _moe(20, 4, 1, (4, 2)), 0.9, 0.8),
        _layer(_left(3, 1, 20, 12, 0.25, 10, base=50.0, scaling=(16.0, 32, 4.0, 0.5)), _right(2, 1, 12, 20, 4), _dense(36)),
        _layer(_left(1, 1, 36, 36, 0.2, 36), _right(1, 1, 20, 12, 2), None, 0.3, 1.5),
    ],
}
# the whole model is the repeated stretch (twice); head widths the tensor-core kernels take; wide feed-forwards
MIFIDRA_C = {
    "architecture": "Mifidra", "vocab": 160, "width": 128, "norm": {"eps": 1e-6}, "logit_scale": 0.125,
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        _layer(_left(4, 2, 64, 64, 0.125, 64, base=250000.0, scaling=(6.0, 128, 16.0, 2.0)), _right(4, 4, 32, 32, 4),
               _moe(48, 12, 3, (3, 2), 96), 0.9, 0.6),
        _layer(_left(2, 1, 128, 64, 0.09, 32), _right(2, 2, 64, 64, 3), _dense(192)),
    ],
}
# one pass of a "repeated" stretch (nothing is added then), no feed-forward anywhere
MIFIDRA_D = {
    "architecture": "Mifidra", "vocab": 150, "width": 32, "norm": {"eps": 1e-5}, "logit_scale": 2.0,
    "loop": {"start": 1, "stop": 2, "times": 1},
    "layers": [_layer(_left(2, 1, 8, 8, 0.35, 8), _right(2, 2, 8, 8, 2), None),
               _layer(_left(2, 2, 16, 8, 0.25, 4), _right(1, 1, 16, 24, 3), None)],
}
MIFIDRA = {"A": MIFIDRA_A, "B": MIFIDRA_B, "C": MIFIDRA_C, "D": MIFIDRA_D}

DECAY_RANK, GATE_RANK = 6, 12       # the low ranks come from the tensors' shapes; 6 is no multiple of 8


def one_layer(left=None, right=None, mlp=None, width=64, vocab=120, **scales) -> dict:
    """One layer with the given halves of the mixer (and a feed-forward), no repeated stretch."""
    left = left or _left(2, 1, 16, 16, 0.25, 16)
    right = right or _right(2, 2, 8, 8, 3)
    return {"architecture": "Mifidra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_scale": 1.0,
            "layers": [_layer(left, right, mlp, **scales)]}


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    w = cfg["width"]
    out = {"embed": (cfg["vocab"], w), "final.norm": (w,)}
    for i, layer in enumerate(cfg["layers"]):
        p, left, right = f"l{i}", layer["mixer"]["left"], layer["mixer"]["right"]
        out.update({f"{p}.norm1": (w,), f"{p}.norm1b": (w,)})
        h, g, d, dv = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
        out.update({f"{p}.mix.left.q": (h * d, w), f"{p}.mix.left.k": (g * d, w), f"{p}.mix.left.v": (g * dv, w),
                    f"{p}.mix.left.o": (w, h * dv)})
        h, g, d, dv, taps = right["heads"], right["kv_heads"], right["dim"], right["vdim"], right["conv"]
        r = f"{p}.mix.right"
        out.update({f"{r}.q": (g * d, w), f"{r}.q.conv": (g * d, taps), f"{r}.k": (g * d, w), f"{r}.k.conv": (g * d, taps),
                    f"{r}.v": (h * dv, w), f"{r}.v.conv": (h * dv, taps), f"{r}.b": (h, w), f"{r}.A_log": (h,),
                    f"{r}.norm": (dv,), f"{r}.a1": (DECAY_RANK, w), f"{r}.a2": (h * d, DECAY_RANK),
                    f"{r}.dt_bias": (h * d,), f"{r}.g1": (GATE_RANK, w), f"{r}.g2": (h * dv, GATE_RANK),
                    f"{r}.o": (w, h * dv)})
        mlp = layer["mlp"]
        if mlp is None:
            continue
        out.update({f"{p}.norm2": (w,), f"{p}.norm2b": (w,)})
        m = f"{p}.mlp"
        if mlp["kind"] == "dense":
            ff = mlp["ff"]
            out.update({f"{m}.gate": (ff, w), f"{m}.gate.b": (ff,), f"{m}.up": (ff, w), f"{m}.up.b": (ff,),
                        f"{m}.down": (w, ff), f"{m}.down.b": (w,)})
        else:
            ff, experts = mlp["expert"]["ff"], mlp["router"]["experts"]
            out.update({f"{m}.router": (experts, w), f"{m}.correction": (experts,)})
            for e in range(experts):
                out.update({f"{m}.e{e}.gate": (ff, w), f"{m}.e{e}.up": (ff, w), f"{m}.e{e}.down": (w, ff)})
            if mlp.get("shared"):
                ff = mlp["shared"]["ff"]
                out.update({f"{m}.shared.gate": (ff, w), f"{m}.shared.up": (ff, w), f"{m}.shared.down": (w, ff)})
    return out


def draw_weights(cfg: dict, seed: int, sharp: float = 1.0) -> dict[str, torch.Tensor]:
    """float32 tensors whose values are bfloat16 numbers.  ``sharp`` multiplies the left query projections, so
    that the softmax has a few large weights and a key that is lost or one too many shows."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2", "norm1b", "norm2b", "norm") or name == "final.norm":
            t = 1.0 + torch.randn(shape, generator=g) * 0.15
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif last == "conv":
            t = torch.randn(shape, generator=g) * 0.6
        elif last in ("A_log", "dt_bias", "b") and len(shape) == 1:
            t = torch.randn(shape, generator=g) * 0.5
        elif last == "correction":
            t = torch.randn(shape, generator=g) * 0.2
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if name.endswith(".left.q"):
                t = t * sharp
            if last in ("a2", "g2", "router"):
                t = t * 3.0                    # so that decays, gates and scores are spread out
            if name.endswith(".right.b"):
                t = t * 2.0
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


ROUTE_COLUMNS = 4


def decisive_routing(cfg: dict, weights: dict, seed: int = 3) -> dict:
    """Make every router's choice robust against rounding without making it the same for all tokens.  The last
    ``ROUTE_COLUMNS`` columns of the residual carry a code of +-3 per token that nothing overwrites (the rows of
    every projection that writes the residual are zero there); the routers read only these columns, with large
    weights, so that every score is 0, 1/2 or 1 up to 1e-4; the corrections then order the experts with gaps far
    above what a bfloat16 run changes.  Which experts score 1 depends on the token's code."""
    g = torch.Generator().manual_seed(seed)
    w, cols = cfg["width"], list(range(cfg["width"] - ROUTE_COLUMNS, cfg["width"]))
    out = dict(weights)
    codes = (torch.randint(0, 2, (cfg["vocab"], ROUTE_COLUMNS), generator=g) * 2 - 1).float() * 3.0
    out["embed"] = out["embed"].clone()
    out["embed"][:, cols] = codes
    for name in list(out):
        last = name.rsplit(".", 1)[-1]
        if last in ("o", "down") or name.endswith("down.b"):
            t = out[name].clone()
            t[cols] = 0.0
            out[name] = t
        elif last in ("norm1", "norm2"):
            t = out[name].clone()
            t[cols] = 1.0
            out[name] = t
        elif last == "router":
            t = torch.zeros_like(out[name])
            t[:, cols] = (torch.randint(0, 2, (t.shape[0], ROUTE_COLUMNS), generator=g) * 2 - 1).float() * 8.0
            out[name] = t
        elif last == "correction":
            n = out[name].numel()
            out[name] = (torch.randperm(n, generator=g).float() * 0.0625 + torch.rand(n, generator=g) * 0.02)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in out.items()}


def write_model(cfg: dict, weights: dict, folder: str) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()},
              os.path.join(folder, "model.safetensors"))
    return folder
