"""A mixer whose state is a matrix per head that is corrected, not only added to: the gated delta rule
(``csrc/delta_rule.cu``), kept in fp32 per request.

``q = W_q h``, ``k = W_k h`` (``kv_heads`` heads of ``dk``), ``v = W_v h`` (``heads`` of ``dv``; head ``h`` uses
the q and k of head ``h // (heads / kv_heads)``).  Each channel of q, k and v passes a short causal convolution over
time (``taps`` taps, no bias, zeros before the sequence's start) and SiLU; q and k become unit vectors per head,
``x / sqrt(sum(x^2) + unit_eps)``, q also times ``q_scale``.  Per head ``beta = sigmoid(W_b h)`` and, per head and
key channel, a decay ``g = exp(-exp(A_log[head]) * softplus(W_a2 (W_a1 h) + dt_bias))``.  Token after token

    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

(the read-out sees the token's own write).  Each head's ``o`` is divided by its root mean square over ``dv`` (eps
inside the root), multiplied by a weight of ``dv`` values shared by the heads and by ``sigmoid(W_g2 (W_g1 h))``, then
``W_o``.  Two states per request: ``S [heads, dv, dk]`` (from zero) and the convolution's last ``taps - 1`` inputs.
fp32 whatever the activation type: the convolution's sum, SiLU, the unit norms, beta, softplus, the decay, the
state, the read-out and the head norm; the projections run in the activation type, those that feed the recurrence's
gates (``W_b``, ``W_a2``) with fp32 output.
"""

from __future__ import annotations

import torch

from gllm_b200 import ops
from gllm_b200.ops import stateful
from gllm_b200.parts.base import Mixer, StateRequirement, TensorExpectation, register_mixer


def _round8(n: int) -> int:
    return -(-n // 8) * 8


def _pad_rows(w: torch.Tensor, rows: int) -> torch.Tensor:
    return torch.nn.functional.pad(w, (0, 0, 0, rows - w.shape[0]))


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Mixer):
    graph_safe_portions = True

    def __init__(self, names, hidden_size: int, heads: int, kv_heads: int, dk: int, dv: int, taps: int, eps: float,
                 unit_eps: float = 1e-6, q_scale: float | None = None, decay_rank: int | None = None,
                 gate_rank: int | None = None):
        """``decay_rank`` / ``gate_rank``: the inner sizes of the two low-rank projections; None takes them from
        the checkpoint's tensors."""
        super().__init__(names)
        self.hidden_size, self.heads, self.kv_heads = int(hidden_size), int(heads), int(kv_heads)
        self.dk, self.dv, self.taps = int(dk), int(dv), int(taps)
        if self.heads % self.kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if not (1 <= self.dk <= 512 and self.dv >= 1 and 1 <= self.taps <= 16):
            raise ValueError("the delta rule takes up to 512 key channels per head and up to 16 taps")
        self.eps, self.unit_eps = float(eps), float(unit_eps)
        self.q_scale = float(q_scale) if q_scale is not None else self.dk ** -0.5
        self.decay_rank = int(decay_rank) if decay_rank is not None else None
        self.gate_rank = int(gate_rank) if gate_rank is not None else None
        self.channels = 2 * self.kv_heads * self.dk + self.heads * self.dv
        self.w_in = self.w_b = self.w_a2 = self.w_g2 = self.w_o = None
        self.conv = self.dt_bias = self.A_log = self.norm = None
        self._a1_at = self._g1_at = 0

    def kernel_needs(self):
        return {"modules": {"delta_rule", "recurrent"}}

    def state_requirement(self):
        return (StateRequirement((self.heads, self.dv, self.dk), torch.float32),
                StateRequirement((max(self.taps - 1, 0), self.channels), torch.float32))

    def expected_tensors(self):
        n, w = self.names, self.hidden_size
        qk, hv, hk = self.kv_heads * self.dk, self.heads * self.dv, self.heads * self.dk
        ra = -1 if self.decay_rank is None else self.decay_rank
        rg = -1 if self.gate_rank is None else self.gate_rank
        return {
            n["q"]: TensorExpectation((qk, w)), n["q_conv"]: TensorExpectation((qk, self.taps), "bias"),
            n["k"]: TensorExpectation((qk, w)), n["k_conv"]: TensorExpectation((qk, self.taps), "bias"),
            n["v"]: TensorExpectation((hv, w)), n["v_conv"]: TensorExpectation((hv, self.taps), "bias"),
            n["b"]: TensorExpectation((self.heads, w)),
            n["A_log"]: TensorExpectation((self.heads,), "bias"),
            n["norm"]: TensorExpectation((self.dv,), "vector"),
            n["a1"]: TensorExpectation((ra, w)), n["a2"]: TensorExpectation((hk, ra)),
            n["dt_bias"]: TensorExpectation((hk,), "bias"),
            n["g1"]: TensorExpectation((rg, w)), n["g2"]: TensorExpectation((hv, rg)),
            n["o"]: TensorExpectation((w, hv)),
        }

    def load(self, get, dtype, device):
        n = self.names
        a1, g1, a2, g2 = (get(n[k], "matrix") for k in ("a1", "g1", "a2", "g2"))
        if a2.shape[1] != a1.shape[0] or g2.shape[1] != g1.shape[0]:
            raise ValueError("the two halves of a low-rank projection differ in their inner size")
        # one product for everything that reads h in the activation type: q | k | v | a1 | g1, every section but
        # the first three starting at a multiple of 8 columns (zero rows between) so that the products that follow
        # can read their slice of the result in place
        qkv = torch.cat([get(n[k], "matrix") for k in ("q", "k", "v")], 0)
        ra, rg = _round8(a1.shape[0]), _round8(g1.shape[0])
        self._a1_at = _round8(self.channels)
        self._g1_at = self._a1_at + ra
        self.w_in = torch.cat([_pad_rows(qkv, self._a1_at), _pad_rows(a1, ra), _pad_rows(g1, rg)], 0).contiguous()
        self.w_a2 = torch.nn.functional.pad(a2, (0, ra - a2.shape[1])).contiguous()
        self.w_g2 = torch.nn.functional.pad(g2, (0, rg - g2.shape[1])).contiguous()
        self.w_b, self.w_o = get(n["b"], "matrix").contiguous(), get(n["o"], "matrix").contiguous()
        self.conv = torch.cat([get(n[k], "bias") for k in ("q_conv", "k_conv", "v_conv")], 0).contiguous()
        self.dt_bias, self.A_log, self.norm = get(n["dt_bias"], "bias"), get(n["A_log"], "bias"), get(n["norm"], "vector")

    def forward(self, x, ctx, cache):
        memory, conv_state = cache.states
        proj = ops.linear(x, self.w_in)
        ra, rg = self.w_a2.shape[1], self.w_g2.shape[1]
        # what feeds the recurrence's gates leaves its product in fp32
        decay_raw = ops.linear(proj[:, self._a1_at:self._a1_at + ra], self.w_a2, out_dtype=torch.float32)
        beta_raw = ops.linear(x, self.w_b, out_dtype=torch.float32)
        gate = ops.linear(proj[:, self._g1_at:self._g1_at + rg], self.w_g2)
        qk, v, g, beta = stateful.delta_prep(proj, self.conv, conv_state, ctx.positions, ctx.token_row, ctx.cu_q,
                                             ctx.state_slots, ctx.num_requests, decay_raw, self.dt_bias, self.A_log,
                                             beta_raw, self.heads, self.kv_heads, self.dk, self.dv, self.unit_eps,
                                             self.q_scale, max_q_len=ctx.max_q_len)
        o = stateful.delta_rule(qk, v, g, beta, memory, ctx.cu_q, ctx.state_slots, ctx.num_requests, self.heads,
                                self.kv_heads, self.dk, self.dv, max_q_len=ctx.max_q_len)
        normed = stateful.head_norm(o, self.heads, self.dv, self.norm, self.eps, x.dtype, gate=gate)
        return ops.linear(normed, self.w_o, split_ok=True, add_into=getattr(ctx, "residual_sink", None))
