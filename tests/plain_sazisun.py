"""A plain, slow restatement of the Sazisun design in float64, one function per mechanism.

It shares nothing with the package: it reads a configuration as a plain dict (the keys of config.json)
and weights as a dict of tensors by checkpoint name, and runs one request's tokens at once on the CPU.

Notation.  ``h``: a sublayer's input ``[T, width]``; ``p``: positions ``0 .. T-1``; ``T``: tokens.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def silu(x):
    return x * sigmoid(x)


def softplus(x):
    return torch.clamp(x, min=0) + torch.log1p(torch.exp(-x.abs()))


# ---------------------------------------------------------------- norm
def dynamic_tanh(x, w, pre):
    """``tanh(alpha x) * weight + b``: no statistic of the row enters."""
    return torch.tanh(w[pre + ".alpha"] * x) * w[pre] + w[pre + ".b"]


# ---------------------------------------------------------------- rotation
def scaled_frequencies(rot: dict) -> torch.Tensor:
    """``base^(-2i/dims)``, long wavelengths slowed down by ``factor``, a linear blend in between."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = base ** (-2.0 * torch.arange(dims // 2, dtype=F) / dims)
    s = rot.get("scaling")
    if not s:
        return f
    factor, low, high, original = (float(s[k]) for k in ("factor", "low", "high", "original"))
    out = f.clone()
    for i in range(dims // 2):
        wavelength = 2 * math.pi / float(f[i])
        if wavelength < original / high:
            continue
        if wavelength > original / low:
            out[i] = f[i] / factor
        else:
            t = (original / wavelength - low) / (high - low)
            out[i] = (1 - t) * f[i] / factor + t * f[i]
    return out


def rotate_pairs(x, p, rot):
    """``x [T, units, dim]``: columns (2i, 2i+1) of the first ``dims`` turn by ``p f_i``."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    a = p.to(F)[:, None] * scaled_frequencies(rot)[None, :]
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---------------------------------------------------------------- differential attention
def attention_keys_values(h, p, m, w, pre):
    """Rotated keys ``[T, G, 2, dim]`` and values ``[T, G, vdim]`` of a layer that owns them."""
    T, G, d, dv = h.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = rotate_pairs((h @ w[pre + ".k"].T).view(T, G * 2, d), p, m["rot"]).view(T, G, 2, d)
    return k, (h @ w[pre + ".v"].T).view(T, G, dv)


def difference_weight(m, w, pre):
    return (torch.exp((w[pre + ".lq1"] * w[pre + ".lk1"]).sum()) - torch.exp((w[pre + ".lq2"] * w[pre + ".lk2"]).sum())
            + float(m["diff"]))


def attend(q, k, v, q_pos, k_pos, m, lam, eps, gate=None):
    """``q [Tq, H, 2, dim]`` (rotated), ``k [Tk, G, 2, dim]`` (rotated), ``v [Tk, G, vdim]``: two capped softmax maps
    per head over the keys at positions up to the query's, their difference, the per-head norm, the gate.
    Returns ``[Tq, H * vdim]``."""
    H, G = q.shape[1], k.shape[1]
    cap, diff = float(m["softcap"]), float(m["diff"])
    visible = k_pos[None, :] <= q_pos[:, None]
    heads = []
    for hd in range(H):
        g = hd // (H // G)
        maps = []
        for part in range(2):
            s = (q[:, hd, part] @ k[:, g, part].T) * float(m["scale"])
            s = cap * torch.tanh(s / cap)
            s = s.masked_fill(~visible, -math.inf)
            maps.append(torch.softmax(s, -1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        heads.append(o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * (1.0 - diff))
    o = torch.cat(heads, -1)
    return o if gate is None else o * sigmoid(gate)


def differential_attention(h, p, m, w, pre, eps, k, v):
    """Queries of this layer over the given keys and values; gate; output projection."""
    T, H, d = h.shape[0], m["heads"], m["dim"]
    q = rotate_pairs((h @ w[pre + ".q"].T).view(T, H * 2, d), p, m["rot"]).view(T, H, 2, d)
    o = attend(q, k, v, p, p, m, difference_weight(m, w, pre), eps, gate=h @ w[pre + ".g"].T)
    return o @ w[pre + ".o"].T


# ---------------------------------------------------------------- state-space duality
def causal_conv(x, weight, bias):
    """``y[t, c] = bias[c] + sum_j weight[c, taps-1-j] x[t-j, c]``, zeros before the start."""
    T, taps = x.shape[0], weight.shape[1]
    y = bias[None, :].expand(T, -1).clone()
    for j in range(taps):
        shifted = torch.zeros_like(x)
        shifted[j:] = x[: T - j] if j else x
        y = y + shifted * weight[:, taps - 1 - j][None, :]
    return y


def ssd_scan(x, B, C, dt, A_log, D, heads_per_group):
    """``S <- exp(-exp(A_log) dt) S + dt B x^T``, ``y = S^T C + D x`` per head, token after token."""
    T, Hh, P = x.shape
    N = B.shape[-1]
    y = torch.zeros(T, Hh, P, dtype=F)
    for hd in range(Hh):
        g = hd // heads_per_group
        S = torch.zeros(N, P, dtype=F)
        for t in range(T):
            S = torch.exp(-torch.exp(A_log[hd]) * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + D[hd] * x[t, hd]
    return y


def mamba2(h, m, w, pre, eps):
    T, Hh, P, N, G = h.shape[0], m["heads"], m["vdim"], m["state"], m["groups"]
    inner = Hh * P
    proj = h @ w[pre + ".in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner: 2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[pre + ".conv"], w[pre + ".conv.b"]))
    x = xbc[:, :inner].view(T, Hh, P)
    B = xbc[:, inner: inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[pre + ".dt_bias"])
    y = ssd_scan(x, B, C, dt, w[pre + ".A_log"], w[pre + ".D"], Hh // G).reshape(T, inner)
    y = (y * silu(z)).view(T, m["norm_groups"], -1)
    y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
    return (y.reshape(T, inner) * w[pre + ".norm"]) @ w[pre + ".o"].T


# ---------------------------------------------------------------- feed-forwards
def gated_feed_forward(h, w, pre):
    return (silu(h @ w[pre + ".gate"].T) * (h @ w[pre + ".up"].T)) @ w[pre + ".down"].T


def squared_relu_expert(h, w, pre):
    return (torch.relu(h @ w[pre + ".up"].T) ** 2) @ w[pre + ".down"].T


def route(h, mlp, w, pre):
    """Chosen experts ``[T, top]`` and their weights."""
    r = mlp["router"]
    E, top = int(r["experts"]), int(r["top"])
    s = torch.softmax(h @ w[pre + ".router"].T, -1)
    allowed = torch.ones_like(s, dtype=torch.bool)
    groups = r.get("groups")
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        best = s.view(-1, count, E // count).max(-1).values
        kept = torch.zeros_like(best, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, -1).indices, True)
        allowed = kept[:, :, None].expand(-1, -1, E // count).reshape(-1, E)
    chosen = s.masked_fill(~allowed, -1.0).topk(top, -1).indices
    picked = s.gather(1, chosen)
    return chosen, picked / (picked.sum(-1, keepdim=True) + 1e-20) * float(r["scale"])


def mixture_of_experts(h, mlp, w, pre):
    chosen, weights = route(h, mlp, w, pre)
    out = torch.zeros(h.shape[0], w[pre + ".e0.down"].shape[0], dtype=F)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            out[t] += a * squared_relu_expert(h[t: t + 1], w, f"{pre}.e{e}")[0]
    if mlp.get("shared"):
        out = out + sigmoid(h @ w[pre + ".shared.sg"].T) * squared_relu_expert(h, w, pre + ".shared")
    return out


# ---------------------------------------------------------------- the model
def forward(config: dict, weights: dict, tokens, return_layers: bool = False):
    """Logits ``[T, vocab]`` (float64) of one request's tokens; with ``return_layers`` also the residual
    stream after every layer ``[layers, T, width]``."""
    w = {k: v.to(F) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    p = torch.arange(tokens.numel())
    x = w["embed"][tokens]
    kept, after = {}, []
    for i, layer in enumerate(config["layers"]):
        pre, m = f"l{i}", layer["mixer"]
        h = dynamic_tanh(x, w, pre + ".norm1")
        if layer["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = attention_keys_values(h, p, m, w, pre + ".mix")
            k, v = kept[i if m.get("kv_from") is None else int(m["kv_from"])]
            x = x + differential_attention(h, p, m, w, pre + ".mix", eps, k, v)
        elif layer["type"] == "mamba2":
            x = x + mamba2(h, m, w, pre + ".mix", eps)
        else:
            raise ValueError(layer["type"])
        mlp = layer.get("mlp")
        if mlp is not None:
            h = dynamic_tanh(x, w, pre + ".norm2")
            x = x + (gated_feed_forward(h, w, pre + ".mlp") if mlp["kind"] == "dense"
                     else mixture_of_experts(h, mlp, w, pre + ".mlp"))
        after.append(x.clone())
    logits = dynamic_tanh(x, w, "final.norm") @ w["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits
