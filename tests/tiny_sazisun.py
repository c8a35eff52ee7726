"""Small Sazisun configurations for the tests, as raw config.json dicts, and a writer that draws their weights here
(not through the engine's random-weights mode), tensor by tensor under the names the design gives them.

The configurations differ in every size and option: attention first or a recurrence first, layers that read the keys
and values of an earlier layer (one reader, two readers, with another number of query heads), layers without a
feed-forward, dense and routed feed-forwards (with and without groups, groups of one expert, all groups kept, with
and without a shared expert, one expert per token), grouped / multi-query / one query head per key head, map and
value widths that differ both ways, rotations over the whole map, a part of it and none, with and without frequency
scaling, convolutions of 1 to 4 taps, one and several groups of the recurrence's projections and of its norm, sizes
that are no multiple of 8 and sizes the tensor-core kernels take."""

from __future__ import annotations

import json
import math
import os

import torch
from safetensors.torch import save_file


def _att(heads, kv_heads, dim, vdim, scale, dims, softcap=30.0, diff=0.3, base=10000.0, scaling=None, kv_from=None):
    rot = {"base": base, "dims": dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "softcap": softcap,
         "diff": diff, "rot": rot}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _ssd(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top, scale, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def _layer(mixer, mlp):
    return {"type": "mamba2" if "state" in mixer else "attention", "mixer": mixer, "mlp": mlp}


# attention first; grouped heads, values wider than the maps, a partial scaled rotation; a reader of layer 0's keys
SAZISUN_A = {
    "architecture": "Sazisun", "vocab": 200, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        _layer(_att(4, 2, 16, 24, 0.2, 8, scaling=(4.0, 1.0, 4.0, 64)), _dense(96)),
        _layer(_ssd(4, 16, 16, 2, 4, 2), _moe(32, 8, 2, 1.5, (4, 2), 48)),
        _layer(_att(4, 2, 16, 24, 0.25, 8, softcap=8.0, diff=0.6, scaling=(4.0, 1.0, 4.0, 64), kv_from=0),
               _moe(24, 8, 3, 2.5, (2, 1))),
        _layer(_ssd(2, 8, 24, 1, 2, 1), None),
    ],
}

# a recurrence first; sizes that are no multiple of 8; one key head for all query heads; a rotation over the whole
# map without scaling; one expert per token and no groups; a convolution of one tap (no convolution state)
SAZISUN_B = {
    "architecture": "Sazisun", "vocab": 131, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_ssd(3, 10, 12, 1, 2, 1), None),
        _layer(_att(3, 1, 10, 6, 0.35, 10, softcap=45.0, diff=0.1, base=500.0), _moe(20, 6, 1, 1.0)),
        _layer(_ssd(2, 24, 8, 2, 1, 4), _dense(40)),
        _layer(_att(1, 1, 12, 20, 0.3, 0, softcap=12.0, diff=0.5), _dense(56)),
    ],
}

# sizes the tensor-core products take; two readers of one layer's keys, one with another number of query heads;
# groups of one expert; all groups kept; a shared expert
SAZISUN_C = {
    "architecture": "Sazisun", "vocab": 256, "width": 128, "norm": {"eps": 1e-5},
    "layers": [
        _layer(_att(2, 2, 64, 64, 0.125, 32, softcap=20.0, diff=0.4, scaling=(8.0, 1.0, 2.0, 32)), _moe(64, 4, 2, 2.0, (4, 3), 64)),
        _layer(_ssd(4, 32, 64, 1, 3, 1), _moe(64, 4, 4, 0.5, (2, 2), 128)),
        _layer(_att(2, 2, 64, 64, 0.125, 32, softcap=20.0, diff=0.2, scaling=(8.0, 1.0, 2.0, 32), kv_from=0), _dense(128)),
        _layer(_att(4, 2, 64, 64, 0.1, 32, softcap=25.0, diff=0.7, scaling=(8.0, 1.0, 2.0, 32), kv_from=0), None),
    ],
}

SAZISUN = {"A": SAZISUN_A, "B": SAZISUN_B, "C": SAZISUN_C}


def one_layer(mixer, mlp=None, width=64, vocab=150, eps=1e-5):
    """A model of one layer: the mechanism alone between the embedding and the head."""
    return {"architecture": "Sazisun", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [_layer(mixer, mlp)]}


def tensor_shapes(cfg: dict) -> dict[str, tuple]:
    """Names and shapes of a configuration's tensors, as the design lays them out."""
    w, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"])}

    def norm(name):
        out[name], out[name + ".b"], out[name + ".alpha"] = (w,), (w,), ()

    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix", layer["mixer"]
        norm(f"l{i}.norm1")
        if layer["type"] == "attention":
            out[p + ".q"] = (m["heads"] * 2 * m["dim"], w)
            if m.get("kv_from") is None:
                out[p + ".k"], out[p + ".v"] = (m["kv_heads"] * 2 * m["dim"], w), (m["kv_heads"] * m["vdim"], w)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[f"{p}.{n}"] = (m["dim"],)
            out[p + ".g"], out[p + ".o"] = (m["heads"] * m["vdim"], w), (w, m["heads"] * m["vdim"])
        else:
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            out[p + ".in"] = (2 * inner + 2 * gn + m["heads"], w)
            out[p + ".conv"], out[p + ".conv.b"] = (inner + 2 * gn, m["conv"]), (inner + 2 * gn,)
            for n in ("dt_bias", "A_log", "D"):
                out[f"{p}.{n}"] = (m["heads"],)
            out[p + ".norm"], out[p + ".o"] = (inner,), (w, inner)
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        norm(f"l{i}.norm2")
        q = f"l{i}.mlp"
        if mlp["kind"] == "dense":
            out[q + ".gate"], out[q + ".up"], out[q + ".down"] = (mlp["ff"], w), (mlp["ff"], w), (w, mlp["ff"])
            continue
        out[q + ".router"] = (mlp["router"]["experts"], w)
        for e in range(mlp["router"]["experts"]):
            out[f"{q}.e{e}.up"], out[f"{q}.e{e}.down"] = (mlp["expert"]["ff"], w), (w, mlp["expert"]["ff"])
        if mlp.get("shared"):
            out[q + ".shared.up"], out[q + ".shared.down"] = (mlp["shared"]["ff"], w), (w, mlp["shared"]["ff"])
            out[q + ".shared.sg"] = (1, w)
    norm("final.norm")
    return out


def draw_weights(cfg: dict, seed: int = 0, sharp: float = 1.0) -> dict[str, torch.Tensor]:
    """Weights as bfloat16-representable fp32 tensors.  ``sharp`` multiplies the query projections (peaked maps)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last == "alpha":
            t = torch.rand((), generator=g) * 0.6 + 0.4
        elif last in ("norm1", "norm2", "norm") and len(shape) == 1:
            t = 1.0 + torch.randn(shape, generator=g) * 0.2
        elif last == "b" and len(shape) == 1:
            t = torch.randn(shape, generator=g) * 0.1
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif last == "conv":
            t = torch.randn(shape, generator=g) * 0.6
        elif last in ("A_log", "dt_bias"):
            t = torch.randn(shape, generator=g) * 0.5
        elif last == "D":
            t = 1.0 + torch.randn(shape, generator=g) * 0.3
        elif last in ("lq1", "lk1", "lq2", "lk2"):
            t = torch.randn(shape, generator=g) * 0.3
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if last == "q":
                t = t * sharp
            if last in ("router", "sg"):
                t = t * 3.0
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


ROUTE_COLUMNS = 4


def decisive_routing(cfg: dict, weights: dict, seed: int = 3, gap: float = 1.0) -> dict:
    """Make every router's choice robust against rounding without making it the same for all tokens.  The last
    ``ROUTE_COLUMNS`` columns of the residual carry a code of +-3 per token that nothing overwrites (the rows of
    every projection that writes the residual are zero there; the norms pass them with weight 1 and bias 0); the
    routers read only these columns, and their rows are drawn again until, for every code, the logits at the two
    borders a choice has (the last kept group against the first dropped one, the last chosen expert against the next)
    lie at least ``gap`` apart."""
    g = torch.Generator().manual_seed(seed)
    w, cols = cfg["width"], list(range(cfg["width"] - ROUTE_COLUMNS, cfg["width"]))
    out = dict(weights)
    codes = (torch.randint(0, 2, (cfg["vocab"], ROUTE_COLUMNS), generator=g) * 2 - 1).float() * 3.0
    out["embed"] = out["embed"].clone()
    out["embed"][:, cols] = codes
    all_codes = torch.tensor([[1.0 if (c >> j) & 1 else -1.0 for j in range(ROUTE_COLUMNS)]
                              for c in range(2 ** ROUTE_COLUMNS)])
    for name in list(out):
        last = name.rsplit(".", 1)[-1]
        if last in ("o", "down"):
            t = out[name].clone()
            t[cols] = 0.0
            out[name] = t
        elif last in ("norm1", "norm2") or name == "final.norm":
            t = out[name].clone()
            t[cols] = 1.0
            out[name] = t
        elif name.endswith((".norm1.b", ".norm2.b")):
            t = out[name].clone()
            t[cols] = 0.0
            out[name] = t
    for i, layer in enumerate(cfg["layers"]):
        mlp = layer.get("mlp")
        if not mlp or mlp["kind"] != "moe":
            continue
        r = mlp["router"]
        E, top = r["experts"], r["top"]
        count, keep = (r["groups"]["count"], r["groups"]["keep"]) if r.get("groups") else (1, 1)
        seen = torch.tanh(out[f"l{i}.norm2.alpha"] * 3.0) * all_codes          # what the router reads, per code
        for _ in range(20000):
            rows = torch.randn(E, ROUTE_COLUMNS, generator=g) * 6.0
            rows = rows.to(torch.bfloat16).to(torch.float32)
            z = seen @ rows.T                                                    # [codes, experts]
            best = z.view(-1, count, E // count).max(-1).values
            ok = True
            if keep < count:
                order = best.sort(-1, descending=True).values
                ok = bool((order[:, keep - 1] - order[:, keep] >= gap).all())
                kept = best >= order[:, keep - 1: keep]
                z = z.masked_fill(~kept[:, :, None].expand(-1, -1, E // count).reshape(-1, E), -1e9)
            allowed = int((z[0] > -1e8).sum())
            if ok and top < allowed:
                order = z.sort(-1, descending=True).values
                ok = bool((order[:, top - 1] - order[:, top] >= gap).all())
            if ok:
                break
        else:
            raise RuntimeError("no decisive router found")
        t = torch.zeros(E, w)
        t[:, cols] = rows
        out[f"l{i}.mlp.router"] = t
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in out.items()}


def write_model(cfg: dict, weights: dict, folder: str) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()},
              os.path.join(folder, "model.safetensors"))
    return folder
