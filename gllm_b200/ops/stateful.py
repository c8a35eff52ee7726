"""Python entry points of the kernels for mixers that carry a state, for sigmoid-weighted attention
and for a residual kept as several streams (``csrc/recurrent.cu``, ``csrc/attention_sigmoid.cu``,
``csrc/hyper_streams.cu``).  As everywhere in ``gllm_b200.ops``: CUDA tensors only, no CPU path.

The batch is the step function's flat batch: request ``r`` owns rows ``cu_q[r] .. cu_q[r+1]-1`` and
row ``state_slots[r]`` of every state tensor.  States are fp32 and are read and written in place.
"""

from __future__ import annotations

import os

import torch

from gllm_b200.ops import _check, _cuda, _fn, _ptr, _stream, _suffix, status_word

# GLLM_B200_SIGMOID_MMA=0: the sigmoid attention of bf16 models stays on the CUDA-core kernel (for measurements)
USE_TENSOR_CORES = os.environ.get("GLLM_B200_SIGMOID_MMA", "1") != "0"


def _rows(t: torch.Tensor, name: str, dtype=None) -> None:
    _cuda(t, name, dtype, contiguous=False)
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be [tokens, columns] with contiguous columns")


# ------------------------------------------------------------------ streams
def embed_streams(tokens: torch.Tensor, table: torch.Tensor, positions: torch.Tensor | None,
                  frequencies: torch.Tensor | None, streams: int = 1, sampled: torch.Tensor | None = None,
                  token_row: torch.Tensor | None = None, scale: float = 1.0) -> torch.Tensor:
    """fp32 ``[n, streams * width]``: ``table[tokens] * scale`` plus, with ``frequencies`` (fp32
    ``[ceil(width / 2)]``), a sinusoid of the position (column 2i: sin(p f_i), column 2i+1: cos(p f_i)),
    copied into each of the ``streams`` residual streams.  A negative token id stands for
    ``sampled[token_row[i]]`` as in ``ops.embedding``."""
    _cuda(tokens, "tokens", torch.int32)
    _cuda(table, "table")
    n, (vocab, width) = tokens.numel(), table.shape
    if frequencies is not None:
        _cuda(frequencies, "frequencies", torch.float32)
        _cuda(positions, "positions", torch.int32)
        if frequencies.numel() != (width + 1) // 2:
            raise ValueError("one frequency per pair of columns is needed")
    if sampled is not None:
        _cuda(sampled, "sampled", torch.int32)
        _cuda(token_row, "token_row", torch.int32)
    out = torch.empty((n, streams * width), dtype=torch.float32, device=table.device)
    f = _fn("hyper_streams", f"gllm_embed_streams_{_suffix(table.dtype)}")
    _check(f(tokens.data_ptr(), _ptr(sampled), _ptr(token_row) if sampled is not None else None, table.data_ptr(),
             _ptr(positions) if frequencies is not None else None, _ptr(frequencies), out.data_ptr(), n, width, vocab,
             int(streams), float(scale), status_word(table.device).data_ptr(), _stream()), "embed_streams")
    return out


def stream_mix_norm(y: torch.Tensor | None, resid: torch.Tensor, mix: torch.Tensor | None, write: torch.Tensor | None,
                    read: torch.Tensor | None, weight: torch.Tensor | None, eps: float, out_dtype: torch.dtype,
                    streams: int, rows: torch.Tensor | None = None, want_norm: bool = True,
                    want_sum: bool = False):
    """The write of one sublayer and the read + RMS norm of the next on ``resid [n, streams * width]`` fp32.

    With ``y`` (a sublayer's result ``[n, width]``): every stream becomes
    ``new[t] = sum_s mix[s, t] * old[s] + write[t] * y`` (in place; with ``rows`` only those tokens are
    computed and ``resid`` stays as it is).  Then ``u = sum_t read[t] * new[t]`` (``read`` None: the plain
    sum of the streams) and the result is ``u / sqrt(mean(u^2) + eps) * weight`` in ``out_dtype``; with
    ``want_sum`` also (or only, ``want_norm`` False) ``u`` itself in fp32."""
    _cuda(resid, "resid", torch.float32)
    n, total = resid.shape
    if total % streams:
        raise ValueError("the residual's rows do not hold a whole number of streams")
    width = total // streams
    if y is not None:
        _cuda(y, "y", out_dtype)
        if tuple(y.shape) != (n, width):
            raise ValueError("the sublayer's result and the residual differ in shape")
        _cuda(mix, "mix", torch.float32)
        _cuda(write, "write", torch.float32)
        if mix.numel() != streams * streams or write.numel() != streams:
            raise ValueError("mix is [streams, streams] and write is [streams]")
    if read is not None:
        _cuda(read, "read", torch.float32)
        if read.numel() != streams:
            raise ValueError("read is [streams]")
    n_rows = n if rows is None else rows.numel()
    if rows is not None:
        _cuda(rows, "rows", torch.int32)
    out = sums = None
    if want_norm:
        _cuda(weight, "weight", torch.float32)
        if weight.numel() != width:
            raise ValueError("one norm weight per column is needed")
        out = torch.empty((n_rows, width), dtype=out_dtype, device=resid.device)
    if want_sum:
        sums = torch.empty((n_rows, width), dtype=torch.float32, device=resid.device)
    f = _fn("hyper_streams", f"gllm_stream_mix_norm_{_suffix(out_dtype)}")
    _check(f(_ptr(y), resid.data_ptr(), _ptr(mix) if y is not None else None, _ptr(write) if y is not None else None,
             _ptr(read), _ptr(weight) if want_norm else None, _ptr(out), _ptr(sums), _ptr(rows), n_rows, width,
             int(streams), float(eps), _stream()), "stream_mix_norm")
    if want_norm and want_sum:
        return out, sums
    return out if want_norm else sums


# ------------------------------------------------------------------ convolution and scan
def conv_silu(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, conv_state: torch.Tensor,
              positions: torch.Tensor, token_row: torch.Tensor) -> torch.Tensor:
    """``silu(causal_conv(x) + bias)`` per channel over each request's own tokens.  ``x [n, channels]``
    (rows may be a slice of wider rows), ``weight [channels, taps]`` fp32 whose last column multiplies
    the current token, ``conv_state [slots, taps-1, channels]`` fp32: each request's last ``taps-1``
    inputs before this step, oldest first (read only; ``selective_scan`` brings it up to date)."""
    _rows(x, "x")
    _cuda(weight, "weight", torch.float32)
    _cuda(conv_state, "conv_state", torch.float32)
    n, channels = x.shape
    taps = weight.shape[1]
    if weight.shape[0] != channels or tuple(conv_state.shape[1:]) != (max(taps - 1, 0), channels):
        raise ValueError("conv weight or state does not fit the channels")
    out = torch.empty((n, channels), dtype=x.dtype, device=x.device)
    f = _fn("recurrent", f"gllm_conv_silu_{_suffix(x.dtype)}")
    _check(f(x.data_ptr(), x.stride(0), weight.data_ptr(), _ptr(bias), conv_state.data_ptr(), positions.data_ptr(),
             token_row.data_ptr(), out.data_ptr(), n, channels, taps, _stream()), "conv_silu")
    return out


def selective_scan(xc: torch.Tensor, dt_raw: torch.Tensor, dt_bias: torch.Tensor, A: torch.Tensor,
                   proj: torch.Tensor, b_offset: int, c_offset: int, D: torch.Tensor, xz: torch.Tensor,
                   z_offset: int, ssm_state: torch.Tensor, conv_state: torch.Tensor, taps: int,
                   cu_q: torch.Tensor, state_slots: torch.Tensor, num_requests: int, max_q_len: int = 0) -> torch.Tensor:
    """Per channel c and state n, token after token of each request:
    ``dt = softplus(dt_raw + dt_bias)``, ``S[c, n] = exp(dt A[c, n]) S[c, n] + dt x B[n]``,
    ``y = sum_n S[c, n] C[n] + D[c] x``, result ``y * silu(z)``.  ``B`` and ``C`` are the columns
    ``b_offset ..`` and ``c_offset ..`` of ``proj``, ``z`` the columns ``z_offset ..`` of ``xz`` whose
    first columns are the raw (unconvolved) inputs, the last ``taps-1`` of which become the new
    ``conv_state``.  ``ssm_state [slots, channels, states]`` fp32 is updated in place.  ``max_q_len`` 1 says
    that every request brings one token: the kernel laid out for single tokens runs then."""
    _cuda(xc, "xc")
    _cuda(dt_raw, "dt_raw", torch.float32)
    _rows(proj, "proj", xc.dtype)
    _rows(xz, "xz", xc.dtype)
    for name, t in (("dt_bias", dt_bias), ("A", A), ("D", D), ("ssm_state", ssm_state), ("conv_state", conv_state)):
        _cuda(t, name, torch.float32)
    n, channels = xc.shape
    n_state = A.shape[1]
    if tuple(ssm_state.shape[1:]) != (channels, n_state) or tuple(dt_raw.shape) != (n, channels):
        raise ValueError("the scan's operands do not fit together")
    out = torch.empty((n, channels), dtype=xc.dtype, device=xc.device)
    f = _fn("recurrent", f"gllm_selective_scan_{_suffix(xc.dtype)}")
    _check(f(xc.data_ptr(), dt_raw.data_ptr(), dt_bias.data_ptr(), A.data_ptr(), proj.data_ptr(), proj.stride(0),
             int(b_offset), int(c_offset), D.data_ptr(), xz.data_ptr(), xz.stride(0), int(z_offset),
             ssm_state.data_ptr(), conv_state.data_ptr(), cu_q.data_ptr(), state_slots.data_ptr(), out.data_ptr(),
             int(num_requests), int(max_q_len), channels, n_state, int(taps), _stream()), "selective_scan")
    return out


# ------------------------------------------------------------------ matrix recurrences
GATED_LINEAR = 0      # a = f, b = 1 - f, f = lower + (1 - lower) sigmoid(raw + bias); q = silu(raw q)
EXP_GATED = 1         # exponential input gate, log-sigmoid forget gate, running maximum, normaliser
STEP_SIZED = 2        # one step size per (token, head): a = exp(A dt), b = dt * k, dt = softplus(raw + bias)


def matrix_recurrence(mode: int, q: torch.Tensor, k: torch.Tensor | None, v: torch.Tensor, gates: torch.Tensor,
                      gate_bias: torch.Tensor, lower: torch.Tensor | None, cap: float, q_scale: float,
                      state: torch.Tensor, mstate: torch.Tensor | None, cu_q: torch.Tensor,
                      state_slots: torch.Tensor, num_requests: int, heads: int, dk: int, dv: int,
                      max_q_len: int = 0, heads_per_group: int = 1) -> torch.Tensor:
    """``S <- diag(a) S + b v^T``, ``o = S^T q`` per (request, head), token after token.
    ``q, k [n, heads*dk]``, ``v [n, heads*dv]`` (rows may be slices), ``gates`` fp32 (``[n, heads*dk]``
    in mode ``GATED_LINEAR``, ``[n, 2*heads]`` = input | forget in mode ``EXP_GATED``).  ``state`` is
    ``[slots, heads, dv, dk]``, one row per value column (``dv + 1`` rows in mode ``EXP_GATED``: the last
    carries the normaliser) and ``mstate [slots, heads]`` the running maximum.  Returns fp32
    ``[n, heads * cols]``: ``cols = dv``, or ``dv + 2`` in mode ``EXP_GATED``, the two extra columns
    being ``n . q`` and ``exp(-m)``.  ``max_q_len`` 1 says that every request brings one token: the kernel laid
    out for single tokens runs then.  Mode ``STEP_SIZED`` (the recurrence of state-space duality): ``gates [n, heads]``
    are raw step sizes, ``gate_bias [heads]`` their bias, ``lower [heads]`` holds ``A = -exp(A_log)``;
    ``dt = softplus(gates + gate_bias)``, ``a = exp(A dt)`` for the whole head, ``b = dt * k``; ``q`` and ``k`` are
    ``[n, (heads / heads_per_group) * dk]``: ``heads_per_group`` neighbouring heads share them."""
    _rows(q, "q")
    _rows(v, "v", q.dtype)
    if k is not None:
        _rows(k, "k", q.dtype)
    _rows(gates, "gates", torch.float32)
    _cuda(gate_bias, "gate_bias", torch.float32)
    _cuda(state, "state", torch.float32)
    n = q.shape[0]
    extra = 1 if mode == EXP_GATED else 0
    if tuple(state.shape[1:]) != (heads, dv + extra, dk):
        raise ValueError("the recurrence's state does not fit its heads")
    if heads_per_group != 1 and mode != STEP_SIZED:
        raise ValueError("only the step-sized recurrence shares queries and keys between heads")
    if mode == EXP_GATED:
        _cuda(mstate, "mstate", torch.float32)
        if k is None or gates.shape[1] != 2 * heads:
            raise ValueError("the exponential-gate recurrence takes keys and two gates per head")
    elif mode == STEP_SIZED:
        _cuda(lower, "lower", torch.float32)
        if (k is None or gates.shape[1] != heads or gate_bias.numel() != heads or lower.numel() != heads
                or heads % heads_per_group or q.shape[1] != heads // heads_per_group * dk or k.shape[1] != q.shape[1]):
            raise ValueError("the step-sized recurrence takes keys, one step size, bias and rate per head, and queries "
                             "and keys of heads / heads_per_group groups")
    else:
        _cuda(lower, "lower", torch.float32)
    cols = dv + 2 * extra
    out = torch.empty((n, heads * cols), dtype=torch.float32, device=q.device)
    # the scalar gates and the running maximum of every token, made by a small kernel before the recurrence
    work = torch.empty((n, 4 * heads), dtype=torch.float32, device=q.device) if mode == EXP_GATED else None
    f = _fn("recurrent", f"gllm_matrix_recurrence_{_suffix(q.dtype)}")
    _check(f(int(mode), q.data_ptr(), q.stride(0), _ptr(k), k.stride(0) if k is not None else 0, v.data_ptr(),
             v.stride(0), gates.data_ptr(), gates.stride(0), gate_bias.data_ptr(), _ptr(lower), float(cap),
             float(q_scale), state.data_ptr(), _ptr(mstate), _ptr(work), cu_q.data_ptr(), state_slots.data_ptr(),
             out.data_ptr(), out.stride(0), int(num_requests), int(max_q_len), heads, dk, dv, int(heads_per_group),
             _stream()), "matrix_recurrence")
    return out


def gated_group_norm(y: torch.Tensor, z: torch.Tensor, weight: torch.Tensor, groups: int, eps: float,
                     skip: torch.Tensor | None = None, x: torch.Tensor | None = None, head_width: int = 0) -> torch.Tensor:
    """``u = (y + skip[head] * x) * silu(z)`` (the skip term with ``skip`` ``[heads]`` fp32 and ``x``, head ``c //
    head_width`` owning column ``c``), then every one of ``groups`` equal parts of a row divided by its own root mean
    square (eps inside the root), times ``weight``: a norm whose gate comes BEFORE it.  ``y`` fp32 ``[n, width]``;
    ``z``, ``x`` of the activation type (rows may be slices).  Returns ``[n, width]`` of the activation type."""
    _rows(y, "y", torch.float32)
    _rows(z, "z")
    _cuda(weight, "weight", torch.float32)
    n, width = y.shape
    if z.shape != y.shape or weight.numel() != width or groups < 1 or width % groups:
        raise ValueError("gated_group_norm's operands do not fit together")
    if skip is not None:
        _cuda(skip, "skip", torch.float32)
        _rows(x, "x", z.dtype)
        if x.shape != y.shape or head_width < 1 or skip.numel() * head_width != width:
            raise ValueError("the skip term needs one factor per head and the recurrence's input")
    out = torch.empty((n, width), dtype=z.dtype, device=y.device)
    f = _fn("recurrent", f"gllm_gated_group_norm_{_suffix(z.dtype)}")
    _check(f(y.data_ptr(), y.stride(0), _ptr(x) if skip is not None else None, x.stride(0) if skip is not None else 0,
             _ptr(skip), int(head_width), z.data_ptr(), z.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0),
             n, int(groups), width // groups, float(eps), _stream()), "gated_group_norm")
    return out


def conv_state_advance(x: torch.Tensor, conv_state: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor,
                       num_requests: int) -> None:
    """Bring ``conv_state [slots, taps-1, channels]`` (every request's last inputs of a short convolution, oldest
    first) up to date with this step's inputs ``x [n, channels]`` (rows may be slices)."""
    _rows(x, "x")
    _cuda(conv_state, "conv_state", torch.float32)
    if conv_state.shape[2] != x.shape[1]:
        raise ValueError("the convolution's state does not fit the channels")
    f = _fn("recurrent", f"gllm_conv_state_advance_{_suffix(x.dtype)}")
    _check(f(x.data_ptr(), x.stride(0), conv_state.data_ptr(), cu_q.data_ptr(), state_slots.data_ptr(),
             int(num_requests), x.shape[1], conv_state.shape[1] + 1, _stream()), "conv_state_advance")


def head_norm(o: torch.Tensor, heads: int, dv: int, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
              with_denominator: bool = False, denominator_eps: float = 0.0,
              gate: torch.Tensor | None = None) -> torch.Tensor:
    """Each head of ``o`` (fp32 ``[n, heads * cols]`` as ``matrix_recurrence`` returns it) divided by
    its root mean square over its ``dv`` values, times ``weight`` (``[dv]``: shared by the heads;
    ``[heads * dv]``: one per column), times ``sigmoid(gate)`` when given.  ``with_denominator``: the
    head is first divided by ``max(|o[dv]|, o[dv+1]) + denominator_eps``."""
    _cuda(o, "o", torch.float32)
    _cuda(weight, "weight", torch.float32)
    n = o.shape[0]
    cols = o.shape[1] // heads
    if weight.numel() not in (dv, heads * dv) or cols < dv + (2 if with_denominator else 0):
        raise ValueError("head_norm's operands do not fit together")
    if gate is not None:
        _rows(gate, "gate", out_dtype)
    out = torch.empty((n, heads * dv), dtype=out_dtype, device=o.device)
    f = _fn("recurrent", f"gllm_head_norm_{_suffix(out_dtype)}")
    _check(f(o.data_ptr(), o.stride(0), cols, int(with_denominator), float(denominator_eps), weight.data_ptr(),
             dv if weight.numel() == heads * dv and heads > 1 else 0, _ptr(gate),
             gate.stride(0) if gate is not None else 0, out.data_ptr(), out.stride(0), n, heads, dv, float(eps),
             _stream()), "head_norm")
    return out


# ------------------------------------------------------------------ gated delta rule
def delta_prep(x: torch.Tensor, conv_weight: torch.Tensor, conv_state: torch.Tensor, positions: torch.Tensor,
               token_row: torch.Tensor, cu_q: torch.Tensor, state_slots: torch.Tensor, num_requests: int,
               decay_raw: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor, beta_raw: torch.Tensor, heads: int,
               kv_heads: int, dk: int, dv: int, unit_eps: float, q_scale: float, max_q_len: int = 0):
    """What the delta rule's recurrence takes, in fp32, from the projections of a step's tokens.

    ``x [n, >= channels]`` (rows may be slices): the q | k | v projections (``token_row``: each token's state slot), ``channels = 2 * kv_heads * dk +
    heads * dv``; each channel passes a causal convolution over the request's own tokens (``conv_weight
    [channels, taps]`` fp32, last column = the current token; ``conv_state [slots, taps-1, channels]`` fp32 holds
    every request's last inputs, oldest first, and is brought up to date) and SiLU; every q and k head becomes
    ``x / sqrt(sum(x^2) + unit_eps)``, q also times ``q_scale``.  ``decay_raw [n, heads * dk]`` and ``beta_raw
    [n, heads]`` are fp32: ``g = exp(-exp(A_log[h]) * softplus(decay_raw + dt_bias))``, ``beta = sigmoid(beta_raw)``.
    ``max_q_len`` 1 says that every request brings one token: the state is then brought up to date by the same
    kernel.  Returns ``(qk [n, 2 * kv_heads * dk], v [n, heads * dv], g [n, heads * dk], beta [n, heads])``."""
    _rows(x, "x")
    _rows(decay_raw, "decay_raw", torch.float32)
    _rows(beta_raw, "beta_raw", torch.float32)
    for name, t in (("conv_weight", conv_weight), ("conv_state", conv_state), ("dt_bias", dt_bias), ("A_log", A_log)):
        _cuda(t, name, torch.float32)
    n = x.shape[0]
    qk_cols, channels = 2 * kv_heads * dk, 2 * kv_heads * dk + heads * dv
    taps = conv_weight.shape[1]
    if (x.shape[1] < channels or conv_weight.shape[0] != channels
            or tuple(conv_state.shape[1:]) != (max(taps - 1, 0), channels) or decay_raw.shape[1] != heads * dk
            or beta_raw.shape[1] != heads or dt_bias.numel() != heads * dk or A_log.numel() != heads):
        raise ValueError("the delta rule's operands do not fit together")
    dev = x.device
    qk = torch.empty((n, qk_cols), dtype=torch.float32, device=dev)
    v = torch.empty((n, heads * dv), dtype=torch.float32, device=dev)
    g = torch.empty((n, heads * dk), dtype=torch.float32, device=dev)
    beta = torch.empty((n, heads), dtype=torch.float32, device=dev)
    f = _fn("delta_rule", f"gllm_delta_prep_{_suffix(x.dtype)}")
    _check(f(x.data_ptr(), x.stride(0), conv_weight.data_ptr(), conv_state.data_ptr(), positions.data_ptr(),
             token_row.data_ptr(), cu_q.data_ptr(), state_slots.data_ptr(), int(num_requests), decay_raw.data_ptr(),
             decay_raw.stride(0), dt_bias.data_ptr(), A_log.data_ptr(), beta_raw.data_ptr(), beta_raw.stride(0),
             qk.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), n, heads, kv_heads, dk, dv, taps,
             float(unit_eps), float(q_scale), int(max_q_len), _stream()), "delta_prep")
    return qk, v, g, beta


def delta_rule(qk: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor, state: torch.Tensor,
               cu_q: torch.Tensor, state_slots: torch.Tensor, num_requests: int, heads: int, kv_heads: int, dk: int,
               dv: int, max_q_len: int = 0) -> torch.Tensor:
    """Per (request, head), token after token: ``S <- diag(g) S``, ``u = beta (v - S^T k)``, ``S <- S + k u^T``,
    ``o = S^T q`` (the read-out sees the token's own write).  Operands as ``delta_prep`` returns them; head ``h``
    uses the q and k of head ``h // (heads / kv_heads)``.  ``state [slots, heads, dv, dk]`` fp32 (one row per value
    column) is updated in place.  Returns fp32 ``[n, heads * dv]``."""
    for name, t in (("qk", qk), ("v", v), ("g", g), ("beta", beta), ("state", state)):
        _cuda(t, name, torch.float32)
    n = qk.shape[0]
    if (tuple(state.shape[1:]) != (heads, dv, dk) or qk.shape[1] != 2 * kv_heads * dk or v.shape[1] != heads * dv
            or g.shape[1] != heads * dk or beta.shape[1] != heads):
        raise ValueError("the delta rule's operands do not fit together")
    out = torch.empty((n, heads * dv), dtype=torch.float32, device=qk.device)
    f = _fn("delta_rule", "gllm_delta_rule")
    _check(f(qk.data_ptr(), v.data_ptr(), g.data_ptr(), beta.data_ptr(), state.data_ptr(), cu_q.data_ptr(),
             state_slots.data_ptr(), out.data_ptr(), int(num_requests), heads, kv_heads, dk, dv, int(max_q_len),
             _stream()), "delta_rule")
    return out


# ------------------------------------------------------------------ sigmoid attention
def qk_norm_store(qkv: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, eps: float, temp_coef: float,
                  temp_every: float, positions: torch.Tensor, slot_mapping: torch.Tensor | None,
                  cache_pages: torch.Tensor | None, heads: int, kv_heads: int, dk: int, dv: int,
                  block_size: int) -> torch.Tensor:
    """In place on ``qkv [n, heads*dk + kv_heads*dk + kv_heads*dv]``: RMS norm of every query and key
    head (weights ``[dk]``), queries times ``1 + temp_coef * ln(floor((p+1) / temp_every) + 1)``; the
    normed keys and the values go into ``cache_pages [pages, block_size * kv_heads * (dk + dv)]`` at
    ``slot_mapping``."""
    _cuda(qkv, "qkv")
    _cuda(q_weight, "q_weight", torch.float32)
    _cuda(k_weight, "k_weight", torch.float32)
    n = qkv.shape[0]
    if qkv.shape[1] != heads * dk + kv_heads * (dk + dv) or q_weight.numel() != dk or k_weight.numel() != dk:
        raise ValueError("qkv width or the norm weights do not fit the heads")
    num_pages = 0
    if slot_mapping is not None:
        _cuda(slot_mapping, "slot_mapping", torch.int32)
        _cuda(cache_pages, "cache_pages", qkv.dtype)
        num_pages = cache_pages.shape[0]
        if cache_pages.shape[1] != block_size * kv_heads * (dk + dv):
            raise ValueError("the cache pages do not hold keys and values of these widths")
    f = _fn("attention_sigmoid", f"gllm_qk_norm_store_{_suffix(qkv.dtype)}")
    _check(f(qkv.data_ptr(), qkv.stride(0), q_weight.data_ptr(), k_weight.data_ptr(), float(eps), float(temp_coef),
             float(temp_every), positions.data_ptr(), _ptr(slot_mapping),
             _ptr(cache_pages) if slot_mapping is not None else None, n, heads, kv_heads, dk, dv, int(block_size),
             num_pages, status_word(qkv.device).data_ptr(), _stream()), "qk_norm_store")
    return qkv


_mma = None
SPLIT_KEYS = 256          # keys per CTA when single tokens' contexts are cut (a multiple of the key tile of 64)
MAX_SPLITS = 16           # what the kernel that adds the partial results takes


def _mma_fns():
    global _mma
    if _mma is None:
        from ctypes import c_float, c_int, c_int64, c_void_p as P

        from gllm_b200.ops.build import load_module

        lib = load_module("attention_sigmoid_mma")
        f = lib.gllm_attention_sigmoid_mma
        f.argtypes = [P, c_int64, P, c_int64, P, c_int64, P, P, c_int, P, P, P, P, c_int, c_int, c_int, c_int, c_int,
                      c_int, c_int, c_int, c_float, c_int, c_int, P, P]
        f.restype = c_int
        lib.gllm_attention_sigmoid_mma_supports.argtypes = [c_int, c_int]
        lib.gllm_attention_sigmoid_mma_tokens_per_tile.argtypes = [c_int, c_int]
        _mma = (f, lib.gllm_attention_sigmoid_mma_supports, lib.gllm_attention_sigmoid_mma_tokens_per_tile)
    return _mma


def sigmoid_attention_takes_tensor_cores(dtype: torch.dtype, dk: int, dv: int) -> bool:
    """True for the sizes the tensor-core kernel is built for (bf16; widths 32, 64, 96 or 128)."""
    return dtype == torch.bfloat16 and all(d in (32, 64, 96, 128) for d in (dk, dv))


def _sigmoid_attention_mma(qkv, cache_pages, block_table, head_bias, heads, kv_heads, dk, dv, block_size, scale, batch, out):
    """The tensor-core kernel.  Steps whose tiles do not fill the GPU (single tokens over long contexts)
    cut every request's keys into ranges of at least ``SPLIT_KEYS`` keys, one CTA each; the partial results are
    added in ascending order."""
    from gllm_b200 import ops

    f, _, tokens_per_tile = _mma_fns()
    n = qkv.shape[0]
    qt = tokens_per_tile(heads, kv_heads)
    group = heads // kv_heads
    head_tiles = kv_heads * (group if 64 % group or group > 64 else 1)
    tiles = -(-batch.max_q_len // qt) * head_tiles * batch.num_requests
    sms = torch.cuda.get_device_properties(qkv.device).multi_processor_count
    splits, tiles_per_split = 1, 0
    # a captured prompt portion is replayed for other contexts: under capture the ranges cover what a block-table
    # row can hold, not just the captured step's longest sequence (single tokens are captured per sequence bucket)
    longest = batch.max_seq_len
    if batch.max_q_len > 1 and torch.cuda.is_current_stream_capturing():
        longest = max(longest, block_table.shape[1] * block_size)
    if tiles < 4 * sms and longest > 2 * SPLIT_KEYS:
        want = min(MAX_SPLITS, -(-8 * sms // tiles))          # five CTAs fit an SM: keep them all streaming
        tiles_per_split = max(SPLIT_KEYS // 64, -(-(-(-longest // 64)) // want))
        splits = -(-(-(-longest // 64)) // tiles_per_split)
    partial = None
    if splits > 1:
        partial = batch.workspace.get("sigmoid_attention_partial", splits * n * heads * dv, torch.float32)
    code = f(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), _ptr(partial), n * heads * dv,
             cache_pages.data_ptr(), block_table.data_ptr(), block_table.stride(0), batch.cu_q.data_ptr(),
             batch.context_lens.data_ptr(), batch.state_slots.data_ptr(), _ptr(head_bias), batch.num_requests,
             batch.max_q_len, heads, kv_heads, dk, dv, int(block_size), cache_pages.shape[0], float(scale), splits,
             tiles_per_split, status_word(qkv.device).data_ptr(), _stream())
    _check(code, "sigmoid_attention_mma")
    if splits > 1:
        ops.SplitSum(partial.view(splits, n, heads * dv), out.dtype).tensor(out)
    return out


def sigmoid_attention(qkv: torch.Tensor, cache_pages: torch.Tensor, block_table: torch.Tensor,
                      positions: torch.Tensor, token_row: torch.Tensor, head_bias: torch.Tensor | None, heads: int,
                      kv_heads: int, dk: int, dv: int, block_size: int, scale: float, batch=None) -> torch.Tensor:
    """``out[i, h] = sum_{j <= p_i} sigmoid(q . k_j * scale + head_bias[h]) v_j`` over the request's
    cached keys and values (this step's own included); queries are the first ``heads * dk`` columns of
    ``qkv``.  Returns ``[n, heads * dv]``.  With ``batch`` (the StepContext: per-request lengths and slots) bf16
    inputs of the sizes it takes run on the tensor-core kernel, everything else on the CUDA cores in fp32."""
    _cuda(qkv, "qkv")
    _cuda(cache_pages, "cache_pages", qkv.dtype)
    _cuda(block_table, "block_table", torch.int32, contiguous=False)
    if head_bias is not None:
        _cuda(head_bias, "head_bias", torch.float32)
    n = qkv.shape[0]
    out = torch.empty((n, heads * dv), dtype=qkv.dtype, device=qkv.device)
    if (batch is not None and sigmoid_attention_takes_tensor_cores(qkv.dtype, dk, dv) and qkv.stride(0) % 8 == 0
            and (block_size * dk) % 8 == 0 and USE_TENSOR_CORES):
        return _sigmoid_attention_mma(qkv, cache_pages, block_table, head_bias, heads, kv_heads, dk, dv, block_size,
                                      scale, batch, out)
    f = _fn("attention_sigmoid", f"gllm_attention_sigmoid_{_suffix(qkv.dtype)}")
    _check(f(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), cache_pages.data_ptr(),
             block_table.data_ptr(), block_table.stride(0), positions.data_ptr(), token_row.data_ptr(),
             _ptr(head_bias), n, heads, kv_heads, dk, dv, int(block_size), cache_pages.shape[0], float(scale),
             status_word(qkv.device).data_ptr(), _stream()), "sigmoid_attention")
    return out
