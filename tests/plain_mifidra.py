"""A plain, slow restatement of the Mifidra design in float64, one function per mechanism.

It shares nothing with the package: it reads a configuration as a plain dict (the keys of config.json)
and weights as a dict of tensors by checkpoint name, and runs one request's tokens at once (or token after
token through ``PlainState``) on the CPU.

Notation.  ``h``: a sublayer's input ``[T, width]``; ``p``: positions; ``rms(x) = x / sqrt(mean(x^2) + eps)``.
"""

from __future__ import annotations

import math

import torch

F = torch.float64


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms(x, eps) * w


# ---------------------------------------------------------------- rotation
def yarn_frequencies(rot: dict) -> tuple[torch.Tensor, float]:
    """Frequencies of the rotated pairs and the multiplier of sine and cosine."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F)
    f = base ** (-2.0 * i / dims)
    s = rot.get("scaling")
    if not s:
        return f, 1.0
    factor, original = float(s["factor"]), float(s["original"])

    def dim_of(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(dim_of(float(s["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(s["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: torch.Tensor, p: torch.Tensor, rot: dict) -> torch.Tensor:
    """``x [T, heads, dim]``: neighbouring pairs (2i, 2i+1) of the first ``dims`` columns turn by ``p f_i``."""
    dims = int(rot["dims"])
    if dims == 0:
        return x
    f, mult = yarn_frequencies(rot)
    a = p.to(F)[:, None] * f[None, :]
    c, s = (a.cos() * mult)[:, None, :], (a.sin() * mult)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---------------------------------------------------------------- left: softmax attention
def left_project(h, p, m, w, pre, eps):
    """Rotated and normed queries ``[T, H, dim]``, keys ``[T, G, dim]`` and values ``[T, G, vdim]``."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w[pre + ".q"].T).view(T, H, d)
    k = (h @ w[pre + ".k"].T).view(T, G, d)
    v = (h @ w[pre + ".v"].T).view(T, G, dv)
    q, k = rotate_pairs(q, p, m["rot"]), rotate_pairs(k, p, m["rot"])
    return rms(q, eps), rms(k, eps), v


def left_attend(q, k, v, q_pos, k_pos, m):
    """Softmax over the keys at positions <= the query's."""
    H, G = m["heads"], m["kv_heads"]
    out = torch.zeros(q.shape[0], H, v.shape[-1], dtype=F)
    visible = k_pos[None, :] <= q_pos[:, None]
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~visible, float("-inf"))
        out[:, hd] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(q.shape[0], -1)


# ---------------------------------------------------------------- right: gated delta rule
def short_conv(x, taps_w, before):
    """``x [T, C]``, ``taps_w [C, taps]`` (last column: the current token), ``before [taps-1, C]``: the inputs
    before the first row (zeros at a sequence's start).  Returns silu(conv) and the new ``before``."""
    taps = taps_w.shape[1]
    full = torch.cat([before, x], 0)
    T = x.shape[0]
    y = torch.zeros_like(x)
    for j in range(taps):
        y = y + full[j:j + T] * taps_w[:, j]
    return y * torch.sigmoid(y), full[full.shape[0] - (taps - 1):] if taps > 1 else before


def unit(x):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def delta_rule(q, k, v, g, beta, S):
    """Per head, token after token: ``S <- g * S`` (rows = key channels), ``u = beta (v - S^T k)``,
    ``S <- S + k u^T``, ``o = S^T q``.  ``q, k, g [T, H, dk]``, ``v [T, H, dv]``, ``beta [T, H]``,
    ``S [H, dk, dv]`` (changed in place)."""
    T, H = beta.shape
    o = torch.zeros(T, H, v.shape[-1], dtype=F)
    for t in range(T):
        for hd in range(H):
            S[hd] *= g[t, hd][:, None]
            u = beta[t, hd] * (v[t, hd] - S[hd].T @ k[t, hd])
            S[hd] += torch.outer(k[t, hd], u)
            o[t, hd] = S[hd].T @ q[t, hd]
    return o


def right_mixer(h, m, w, pre, eps, state):
    """``state``: dict with ``S [H, dk, dv]`` and ``conv_q|k|v`` (the last taps-1 inputs), updated in place."""
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    outs = {}
    for n in ("q", "k", "v"):
        outs[n], state["conv_" + n] = short_conv(h @ w[f"{pre}.{n}"].T, w[f"{pre}.{n}.conv"], state["conv_" + n])
    q = unit(outs["q"].view(T, G, dk)) * dk ** -0.5
    k = unit(outs["k"].view(T, G, dk))
    rep = H // G
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
    v = outs["v"].view(T, H, dv)
    beta = torch.sigmoid(h @ w[pre + ".b"].T)
    raw = (h @ w[pre + ".a1"].T) @ w[pre + ".a2"].T + w[pre + ".dt_bias"]
    g = torch.exp(-torch.exp(w[pre + ".A_log"])[None, :, None] * torch.nn.functional.softplus(raw).view(T, H, dk))
    o = delta_rule(q, k, v, g, beta, state["S"])
    gate = torch.sigmoid((h @ w[pre + ".g1"].T) @ w[pre + ".g2"].T).view(T, H, dv)
    o = rms(o, eps) * w[pre + ".norm"] * gate
    return o.reshape(T, H * dv) @ w[pre + ".o"].T


def new_right_state(m):
    taps = int(m["conv"])
    return {"S": torch.zeros(m["heads"], m["dim"], m["vdim"], dtype=F),
            "conv_q": torch.zeros(taps - 1, m["kv_heads"] * m["dim"], dtype=F),
            "conv_k": torch.zeros(taps - 1, m["kv_heads"] * m["dim"], dtype=F),
            "conv_v": torch.zeros(taps - 1, m["heads"] * m["vdim"], dtype=F)}


# ---------------------------------------------------------------- feed-forwards
def glu(h, w, pre, bias):
    def lin(n):
        y = h @ w[f"{pre}.{n}"].T
        return y + w[f"{pre}.{n}.b"] if bias else y

    g = lin("gate")
    hidden = g * torch.sigmoid(g) * lin("up")
    y = hidden @ w[pre + ".down"].T
    return y + w[pre + ".down.b"] if bias else y


def route(h, w, pre, router, margins: list | None = None):
    """Chosen experts ``[T, top]`` and their weights (the uncorrected sigmoid scores, not renormalised).
    ``margins`` collects the smallest gap between what was just chosen and what was just not (groups and
    experts): a test whose gap is small rests on rounding."""
    E, top = int(router["experts"]), int(router["top"])
    s = torch.sigmoid(h @ w[pre + ".router"].T)
    choice = s + w[pre + ".correction"]
    groups = router.get("groups")
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = choice.view(-1, count, E // count)
        score = per.topk(min(2, E // count), -1).values.sum(-1)
        best = score.topk(keep, -1).indices
        if margins is not None and keep < count:
            ranked = score.sort(-1, descending=True).values
            margins.append(float((ranked[:, keep - 1] - ranked[:, keep]).min()))
        allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, best, True)
        choice = per.masked_fill(~allowed[:, :, None], float("-inf")).reshape(-1, E)
    chosen = choice.topk(top, -1).indices
    if margins is not None and top < E:
        ranked = choice.sort(-1, descending=True).values
        margins.append(float((ranked[:, top - 1] - ranked[:, top]).min()))
    return chosen, s.gather(1, chosen)


def moe(h, w, pre, mlp, margins: list | None = None):
    chosen, weights = route(h, w, pre, mlp["router"], margins)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            out[t] += a * glu(h[t:t + 1], w, f"{pre}.e{e}", False)[0]
    if mlp.get("shared"):
        out = out + glu(h, w, pre + ".shared", False)
    return out


# ---------------------------------------------------------------- the model
def layer_runs(cfg):
    """(layer index, whether the embedding output is added before it) in running order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(start)]
    for t in range(times):
        runs += [(i, t > 0 and i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, n)]


class PlainState:
    """What one request carries from token to token: per layer run the keys and values seen so far and the
    right mixer's state."""

    def __init__(self, cfg):
        self.runs = layer_runs(cfg)
        self.k = [None] * len(self.runs)
        self.v = [None] * len(self.runs)
        self.right = [new_right_state(cfg["layers"][i]["mixer"]["right"]) for i, _ in self.runs]
        self.length = 0


def forward(cfg, weights, tokens, state: PlainState | None = None, layers_out: list | None = None,
            margins: list | None = None, stored: torch.dtype | None = None):
    """Logits ``[T, vocab]`` (float64) of ``tokens`` continuing ``state`` (a fresh one if None).  ``stored``: what
    the sublayers read and what they return is rounded to this type (the arithmetic stays float64): how far the
    logits at a position move then says how much rounding alone matters there."""
    keep = (lambda t: t.to(stored).to(F)) if stored is not None else (lambda t: t)
    w = {k: v.to(F) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    state = state or PlainState(cfg)
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.numel()
    p = torch.arange(state.length, state.length + T)
    x0 = w["embed"][tokens]
    x = x0.clone()
    for run, (i, add_embedding) in enumerate(state.runs):
        layer, pre = cfg["layers"][i], f"l{i}"
        if add_embedding:
            x = x + x0
        h = keep(rms_norm(x, w[pre + ".norm1"], eps))
        m = layer["mixer"]
        q, k, v = left_project(h, p, m["left"], w, pre + ".mix.left", eps)
        state.k[run] = k if state.k[run] is None else torch.cat([state.k[run], k], 0)
        state.v[run] = v if state.v[run] is None else torch.cat([state.v[run], v], 0)
        k_pos = torch.arange(state.k[run].shape[0])
        left = left_attend(q, state.k[run], state.v[run], p, k_pos, m["left"]) @ w[pre + ".mix.left.o"].T
        right = right_mixer(h, m["right"], w, pre + ".mix.right", eps, state.right[run])
        mixed = keep(float(m["left_scale"]) * left + float(m["right_scale"]) * right)
        x = x + rms_norm(mixed, w[pre + ".norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp:
            h = keep(rms_norm(x, w[pre + ".norm2"], eps))
            y = keep(glu(h, w, pre + ".mlp", True) if mlp["kind"] == "dense" else moe(h, w, pre + ".mlp", mlp, margins))
            x = x + rms_norm(y, w[pre + ".norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    state.length += T
    return (rms_norm(x, w["final.norm"], eps) @ w["embed"].T) * float(cfg.get("logit_scale", 1.0))
