"""Routed experts: every token is served by ``top`` of ``experts`` small gated feed-forwards
``down(silu(gate(x)) * up(x))`` (no biases), optionally beside a shared expert that serves every token.

Router logits ``z = W_router x`` in fp32; scores ``s = sigmoid(z)``.  The choice is made on ``s + correction``
(a stored vector that steers the choice only), with ``groups``: only among the experts of the ``groups_kept``
best of ``groups`` equal groups of neighbouring experts, a group's score being the sum of its two largest choice
scores.  The result is ``sum_e s_e * expert_e(x)`` over the chosen experts (weights divided by their sum with
``renormalize``) plus the shared expert's.  The (token, expert) pairs are sorted by expert on the device and the
experts' products run over tiles of one expert each: in bf16, with sizes it takes, on the tcgen05 kernel of the dense
products in its grouped form (tiles of 128 rows, ``csrc/gemm_bf16.cu``), otherwise on a CUDA-core kernel (tiles of
16 rows, ``csrc/moe.cu``); nothing about the choice reaches the host.

Options for other designs: ``score`` "softmax" (scores are the softmax of the logits over all experts);
``group_score`` "max" (a group's score is its largest choice score); ``renormalize_eps`` (added to the sum the
weights are divided by); ``scale`` (the weights are multiplied by it last); ``expert`` "relu_squared": experts
without a gate, ``down(max(up(x), 0) ** 2)``; ``shared_gate``: the shared expert's result is multiplied by
``sigmoid(w_sg . x)``, one number per token (its row rides on the router's product).
"""

from __future__ import annotations

import torch

from gllm_b200 import ops
from gllm_b200.ops import moe
from gllm_b200.parts.base import FEED_FORWARDS, FeedForward, TensorExpectation, build_part, register_feed_forward


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    graph_safe_portions = True

    def __init__(self, names, hidden_size: int, intermediate_size: int, experts: int, top: int,
                 groups: int | None = None, groups_kept: int | None = None, score: str = "sigmoid",
                 renormalize: bool = False, correction: bool = False, shared=None, group_score: str = "top2",
                 renormalize_eps: float = 0.0, scale: float = 1.0, expert: str = "gated_silu",
                 shared_gate: bool = False):
        """``names``: ``router``, ``correction`` (with ``correction``), ``shared_gate`` (with ``shared_gate``) and
        ``expert``, a pattern with ``{index}`` and ``{part}`` (gate | up | down).  ``shared``: the PartSpec of a
        feed-forward that runs for every token."""
        super().__init__(names)
        if score not in ("sigmoid", "softmax"):
            raise ValueError(f"unknown router score {score!r}; known: ['sigmoid', 'softmax']")
        if group_score not in ("top2", "max"):
            raise ValueError(f"unknown group score {group_score!r}; known: ['top2', 'max']")
        if expert not in ("gated_silu", "relu_squared"):
            raise ValueError(f"unknown expert form {expert!r}; known: ['gated_silu', 'relu_squared']")
        if shared_gate and shared is None:
            raise ValueError("a gate of the shared expert needs a shared expert")
        self.score, self.group_score, self.gated = score, group_score, expert == "gated_silu"
        self.renormalize_eps, self.scale, self.has_shared_gate = float(renormalize_eps), float(scale), bool(shared_gate)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.experts, self.top = int(experts), int(top)
        self.groups = int(groups) if groups else 1
        self.groups_kept = int(groups_kept) if groups else 1
        if (self.experts % self.groups or not 1 <= self.groups_kept <= self.groups
                or not 1 <= self.top <= self.groups_kept * (self.experts // self.groups)):
            raise ValueError("the experts form equal groups, and 'top' experts must be left to choose from")
        self.renormalize, self.has_correction = bool(renormalize), bool(correction)
        self.shared = build_part(FEED_FORWARDS, shared) if shared is not None else None
        self.w_router = self.correction = self.w_gate_up = self.w_down = None
        self.tensor_cores = False

    def kernel_needs(self):
        needs = {"modules": {"moe"}}      # (the tensor-core products are the dense ones' module, which bf16 loads)
        if self.shared is not None:
            for key, values in self.shared.kernel_needs().items():
                needs.setdefault(key, set()).update(values)
        return needs

    def _expert(self, index: int, part: str) -> str:
        return self.names["expert"].format(index=index, part=part)

    def expected_tensors(self):
        h, i = self.hidden_size, self.intermediate_size
        exp = {self.names["router"]: TensorExpectation((self.experts, h))}
        if self.has_correction:
            exp[self.names["correction"]] = TensorExpectation((self.experts,), "bias")
        if self.has_shared_gate:
            exp[self.names["shared_gate"]] = TensorExpectation((1, h))
        for e in range(self.experts):
            if self.gated:
                exp[self._expert(e, "gate")] = TensorExpectation((i, h))
            exp[self._expert(e, "up")] = TensorExpectation((i, h))
            exp[self._expert(e, "down")] = TensorExpectation((h, i))
        if self.shared is not None:
            exp.update(self.shared.expected_tensors())
        return exp

    def load(self, get, dtype, device):
        self.w_router = get(self.names["router"], "matrix").contiguous()
        if self.has_shared_gate:
            # the gate's one row rides on the router's product (both read the same input, both leave it in fp32)
            self.w_router = torch.cat([self.w_router, get(self.names["shared_gate"], "matrix")], 0).contiguous()
        if self.has_correction:
            self.correction = get(self.names["correction"], "bias").contiguous()
        # [experts, 2 * ff, width]: an expert's gate rows, then its up rows (for the tensor-core products: blocks of
        # 64 gate rows and the 64 up rows of the same features); [experts, width, ff]
        self.tensor_cores = moe.tensor_cores_take(dtype, self.hidden_size, self.intermediate_size, self.gated)
        stack = ops.interleave_gate_up if self.tensor_cores else (lambda gate, up: torch.cat([gate, up], 0))
        if self.gated:
            self.w_gate_up = torch.stack([stack(get(self._expert(e, "gate"), "matrix"),
                                                get(self._expert(e, "up"), "matrix"))
                                          for e in range(self.experts)]).contiguous()
        else:           # experts without a gate: the up weights alone, [experts, ff, width]
            self.w_gate_up = torch.stack([get(self._expert(e, "up"), "matrix")
                                          for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([get(self._expert(e, "down"), "matrix") for e in range(self.experts)]).contiguous()
        if self.shared is not None:
            self.shared.load(get, dtype, device)

    def forward(self, x, ctx):
        logits = ops.linear(x, self.w_router, out_dtype=torch.float32)
        gate = logits[:, self.experts] if self.has_shared_gate else None
        ids, weights = moe.route(logits[:, : self.experts], self.correction, self.top, self.groups, self.groups_kept,
                                 self.renormalize, score=self.score, group_score=self.group_score,
                                 renormalize_eps=self.renormalize_eps, scale=self.scale)
        shared = None
        if self.shared is not None:
            sink, ctx.residual_sink = getattr(ctx, "residual_sink", None), None
            shared = ops.as_tensor(self.shared.forward(x, ctx))
            ctx.residual_sink = sink
        return moe.apply_experts(x, ids, weights, self.w_gate_up, self.w_down, shared, self.tensor_cores,
                                 gated=self.gated, shared_gate=gate)
