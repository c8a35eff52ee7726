"""Selective state-space mixers: Mamba's first form (``selective_scan``) and its second, state-space duality
(``state_space_duality``, below).

``selective_scan``:

``[x | z] = W_in h``; ``x`` passes a short causal convolution per channel (with bias) and SiLU;
``[dt | B | C] = W_x x``; ``dt = softplus(W_dt dt + b)`` per channel; ``A = -exp(A_log)``;
``S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n``, ``y_c = sum_n S[c, n] C_n + D_c x_c``; the
result is ``W_o (y * silu(z))``.  Per request it keeps the scan state ``[inner, states]`` and the
convolution's last ``taps - 1`` inputs, both fp32; step sizes, decays and the state are fp32 whatever
the activations' type.  The products run on the engine's product kernels, the convolution and the scan
on ``csrc/recurrent.cu``.
"""

from __future__ import annotations

import torch

from gllm_b200 import ops
from gllm_b200.ops import stateful
from gllm_b200.parts.base import Mixer, StateRequirement, TensorExpectation, register_mixer


@register_mixer("selective_scan")
class SelectiveScanMixer(Mixer):
    graph_safe_portions = True

    def __init__(self, names, hidden_size: int, inner: int, states: int, dt_rank: int, taps: int):
        super().__init__(names)
        self.hidden_size, self.inner, self.n_state = int(hidden_size), int(inner), int(states)
        self.dt_rank, self.taps = int(dt_rank), int(taps)
        if not 1 <= self.taps <= 16 or self.n_state > 256:
            raise ValueError("the scan kernels take 1..16 convolution taps and up to 256 states per channel")
        self.w_in = self.w_x = self.w_dt = self.w_o = None
        self.conv_w = self.conv_b = self.dt_b = self.A = self.D = None

    def kernel_needs(self):
        return {"modules": {"recurrent"}}

    def state_requirement(self):
        return (StateRequirement((self.inner, self.n_state), torch.float32),
                StateRequirement((max(self.taps - 1, 0), self.inner), torch.float32))

    def expected_tensors(self):
        n = self.names
        return {
            n["in"]: TensorExpectation((2 * self.inner, self.hidden_size)),
            n["conv"]: TensorExpectation((self.inner, self.taps), "vector"),
            n["conv_bias"]: TensorExpectation((self.inner,), "bias"),
            n["x"]: TensorExpectation((self.dt_rank + 2 * self.n_state, self.inner)),
            n["dt"]: TensorExpectation((self.inner, self.dt_rank)),
            n["dt_bias"]: TensorExpectation((self.inner,), "bias"),
            n["A_log"]: TensorExpectation((self.inner, self.n_state), "vector"),
            n["D"]: TensorExpectation((self.inner,), "vector"),
            n["o"]: TensorExpectation((self.hidden_size, self.inner)),
        }

    def load(self, get, dtype, device):
        n = self.names
        self.w_in, self.w_x, self.w_dt, self.w_o = (get(n[k], "matrix") for k in ("in", "x", "dt", "o"))
        self.conv_w, self.conv_b = get(n["conv"], "vector"), get(n["conv_bias"], "bias")
        self.dt_b, self.D = get(n["dt_bias"], "bias"), get(n["D"], "vector")
        self.A = (-torch.exp(get(n["A_log"], "vector"))).contiguous()

    def forward(self, x, ctx, cache):
        ssm_state, conv_state = cache.states
        xz = ops.linear(x, self.w_in)
        xc = stateful.conv_silu(xz[:, : self.inner], self.conv_w, self.conv_b, conv_state, ctx.positions, ctx.token_row)
        proj = ops.linear(xc, self.w_x)
        dt_raw = ops.linear(proj[:, : self.dt_rank], self.w_dt, out_dtype=torch.float32)
        y = stateful.selective_scan(xc, dt_raw, self.dt_b, self.A, proj, self.dt_rank, self.dt_rank + self.n_state,
                                    self.D, xz, self.inner, ssm_state, conv_state, self.taps, ctx.cu_q,
                                    ctx.state_slots, ctx.num_requests, max_q_len=ctx.max_q_len)
        return ops.linear(y, self.w_o, split_ok=True, add_into=getattr(ctx, "residual_sink", None))


@register_mixer("state_space_duality")
class StateSpaceDuality(Mixer):
    """The second form: one decay per head and token, a state matrix per head.

    ``[z | x | B | C | dt] = W_in h`` with ``inner = heads * head_dim`` columns for ``z`` and ``x``, ``groups *
    states`` for ``B`` and ``C`` and ``heads`` for ``dt``; ``x``, ``B`` and ``C`` together pass a short causal
    convolution per channel (with bias) and SiLU; ``dt = softplus(dt + dt_bias)`` (no clamp); per head ``h`` (using
    ``B`` and ``C`` of group ``h // (heads / groups)``):

        S <- exp(-exp(A_log[h]) dt) S + dt B x^T          y = S^T C + D[h] x

    then ``y * silu(z)`` is RMS-normed in ``norm_groups`` equal parts of the row (the gate comes BEFORE the norm),
    multiplied by a weight and projected by ``W_o``.  Per request it keeps ``S [heads, head_dim, states]`` and the
    convolution's last ``taps - 1`` inputs, both fp32; step sizes, decays, the state, the read-out and the norm are
    fp32 whatever the activations' type (the step sizes come out of their product in fp32).  The recurrence is the
    matrix recurrence of ``csrc/recurrent.cu`` in its step-sized mode.
    """

    graph_safe_portions = True

    def __init__(self, names, hidden_size: int, heads: int, head_dim: int, states: int, groups: int, taps: int,
                 norm_groups: int, eps: float):
        super().__init__(names)
        self.hidden_size, self.heads, self.head_dim = int(hidden_size), int(heads), int(head_dim)
        self.n_state, self.groups, self.taps = int(states), int(groups), int(taps)
        self.norm_groups, self.eps = int(norm_groups), float(eps)
        self.inner = self.heads * self.head_dim
        self.channels = self.inner + 2 * self.groups * self.n_state
        if self.heads % self.groups or self.inner % self.norm_groups:
            raise ValueError("heads must be a multiple of groups, and heads * head_dim of norm_groups")
        if not 1 <= self.taps <= 16 or not 1 <= self.n_state <= 512:
            raise ValueError("the kernels take 1..16 convolution taps and up to 512 states per head")
        self.w_in = self.w_dt = self.w_o = None
        self.conv_w = self.conv_b = self.dt_b = self.A = self.D = self.norm_w = None

    def kernel_needs(self):
        return {"modules": {"recurrent"}}

    def state_requirement(self):
        return (StateRequirement((self.heads, self.head_dim, self.n_state), torch.float32),
                StateRequirement((max(self.taps - 1, 0), self.channels), torch.float32))

    def expected_tensors(self):
        n = self.names
        return {
            n["in"]: TensorExpectation((self.inner + self.channels + self.heads, self.hidden_size)),
            n["conv"]: TensorExpectation((self.channels, self.taps), "vector"),
            n["conv_bias"]: TensorExpectation((self.channels,), "bias"),
            n["dt_bias"]: TensorExpectation((self.heads,), "bias"),
            n["A_log"]: TensorExpectation((self.heads,), "vector"),
            n["D"]: TensorExpectation((self.heads,), "vector"),
            n["norm"]: TensorExpectation((self.inner,), "vector"),
            n["o"]: TensorExpectation((self.hidden_size, self.inner)),
        }

    def load(self, get, dtype, device):
        n = self.names
        w_in = get(n["in"], "matrix")
        # the step sizes leave their product in fp32: a product of their own
        self.w_in = w_in[: self.inner + self.channels].contiguous()
        self.w_dt = w_in[self.inner + self.channels:].contiguous()
        self.w_o = get(n["o"], "matrix").contiguous()
        self.conv_w, self.conv_b = get(n["conv"], "vector"), get(n["conv_bias"], "bias")
        self.dt_b, self.D, self.norm_w = get(n["dt_bias"], "bias"), get(n["D"], "vector"), get(n["norm"], "vector")
        self.A = (-torch.exp(get(n["A_log"], "vector"))).contiguous()

    def forward(self, x, ctx, cache):
        ssm_state, conv_state = cache.states
        inner, gn = self.inner, self.groups * self.n_state
        zxbc = ops.as_tensor(ops.linear(x, self.w_in))
        dt_raw = ops.linear(x, self.w_dt, out_dtype=torch.float32)
        raw = zxbc[:, inner:]
        xbc = stateful.conv_silu(raw, self.conv_w, self.conv_b, conv_state, ctx.positions, ctx.token_row)
        if self.taps > 1:
            stateful.conv_state_advance(raw, conv_state, ctx.cu_q, ctx.state_slots, ctx.num_requests)
        y = stateful.matrix_recurrence(stateful.STEP_SIZED, xbc[:, inner + gn:], xbc[:, inner: inner + gn],
                                       xbc[:, :inner], dt_raw, self.dt_b, self.A, 0.0, 1.0, ssm_state, None, ctx.cu_q,
                                       ctx.state_slots, ctx.num_requests, self.heads, self.n_state, self.head_dim,
                                       max_q_len=ctx.max_q_len, heads_per_group=self.heads // self.groups)
        normed = stateful.gated_group_norm(y, zxbc[:, :inner], self.norm_w, self.norm_groups, self.eps, skip=self.D,
                                           x=xbc[:, :inner], head_width=self.head_dim)
        return ops.linear(normed, self.w_o, split_ok=True, add_into=getattr(ctx, "residual_sink", None))
