"""RMSNorm fused with the residual add.

``y = x / sqrt(mean(x^2) + eps) * w`` as gllm/model/layers/norm.py:20-22, with
eps inside the root and the weight multiplying directly.  The reference
computes the statistic in the input dtype; here it is fp32 always, over the
fp32 residual stream.  The add that the reference does separately before each
norm (gllm/model/transformer.py:58-59,72) happens in the same kernel.
"""

from __future__ import annotations

import torch

from gllm_b200 import ops
from gllm_b200.parts.base import Norm, TensorExpectation, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe_portions = True

    def __init__(self, names, size: int, eps: float, unit_offset: bool = False):
        super().__init__(names)
        self.size = int(size)
        self.eps = float(eps)
        # True: the stored weight is an offset from one, y = x_hat * (1 + w)
        self.unit_offset = bool(unit_offset)
        self.weight: torch.Tensor | None = None

    def expected_tensors(self):
        return {self.names["weight"]: TensorExpectation((self.size,), "vector")}

    def load(self, get, dtype, device):
        self.weight = get(self.names["weight"], "vector")

    def pending(self, value):
        """``value`` (a sublayer's result) as what the NEXT norm's kernel norms with this norm's weight and adds
        to the residual: the norm after a sublayer of a layer that norms both sides of it."""
        if self.unit_offset:
            raise ValueError("a norm whose weight is stored around zero cannot follow a sublayer")
        return ops.Pending(None if value is ops.ADDED else value, self.weight, self.eps)

    def forward(self, branch, resid, dtype, rows=None):
        return ops.add_rmsnorm(branch, resid, self.weight, self.eps, dtype, rows=rows, unit_offset=self.unit_offset)


@register_norm("dynamic_tanh")
class DynamicTanh(Norm):
    """``y = tanh(alpha * x) * weight + bias`` with one learned number ``alpha``: a norm that computes no mean and
    no variance, fused with the residual add like the RMS norm (``csrc/dyt_norm.cu``).  Tensor names: ``weight``,
    ``bias`` (one value per column), ``alpha`` (a single number)."""

    graph_safe_portions = True

    def __init__(self, names, size: int):
        super().__init__(names)
        self.size = int(size)
        self.weight = self.bias = self.alpha = None

    def kernel_needs(self):
        return {"modules": {"dyt_norm"}}

    def expected_tensors(self):
        return {
            self.names["weight"]: TensorExpectation((self.size,), "vector"),
            self.names["bias"]: TensorExpectation((self.size,), "bias"),
            self.names["alpha"]: TensorExpectation((), "vector"),
        }

    def load(self, get, dtype, device):
        self.weight, self.bias = get(self.names["weight"], "vector"), get(self.names["bias"], "bias")
        self.alpha = get(self.names["alpha"], "vector").reshape(1).contiguous()

    def forward(self, branch, resid, dtype, rows=None):
        return ops.add_dyt(branch, resid, self.alpha, self.weight, self.bias, dtype, rows=rows)
