"""Causal grouped-query attention over the paged cache.

The reference (gllm/model/layers/attention.py:122-182) runs three separate
projections, rotates q and k, scatters the new k, v into a flat cache, gathers
the whole padded context back out and calls a dense softmax(QK^T/sqrt(D)+bias)V.
Here: one product with the fused [q;k;v] weight, one kernel that rotates q and
k and stores k, v into their pages, one attention kernel that reads the pages
through the block table, one output product.  Query head ``h`` uses kv head
``h // (heads / kv_heads)`` (gllm/ops/attention/reference_attention.py:19-30).
"""

from __future__ import annotations

import math

import torch

from gllm_b200 import ops
from gllm_b200.parts.base import (
    POSITION_ENCODINGS,
    KVPageRequirement,
    Mixer,
    TensorExpectation,
    build_part,
    register_mixer,
)


@register_mixer("attention")
class Attention(Mixer):
    graph_safe_portions = True

    def __init__(self, names, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position=None, window: int | None = None, scale: float | None = None, bias: bool = False,
                 output_bias: bool = False, qk_norm_eps: float | None = None, qk_norm_unit_offset: bool = False,
                 qk_norm_whole: bool = False, values_from_keys: bool = False, value_dim: int | None = None,
                 unit_norm_after_rotation_eps: float | None = None, pad_heads: bool = False):
        """``bias``: the q, k and v projections add a bias (tensor names ``q_bias``, ``k_bias``, ``v_bias``);
        ``output_bias``: so does the output projection (``o_bias``).  ``qk_norm_eps``: every head of q and of k
        is RMS-normed over its ``head_dim`` values before the rotation, with one weight each for all query heads
        and all key heads (``q_norm``, ``k_norm``).  Llama has none of the three (the reference's projections
        have no bias, gllm/model/layers/attention.py:139-142); they are here for architectures that do.
        ``qk_norm_whole``: the norm of ``qk_norm_eps`` runs over the WHOLE q projection (all heads at once) and
        the whole k projection, with one weight per column (``q_norm``: heads * head_dim values).
        ``values_from_keys``: there is no v projection; the values are the keys as projected, before their norm
        and rotation.
        ``unit_norm_after_rotation_eps``: AFTER the rotation every query and key head is divided by its root mean
        square over ``head_dim`` (eps inside the root, no weight).  ``value_dim``: the width of a value head when
        it differs from ``head_dim`` (the width of a query or key head); ``pad_heads``: query, key and value heads
        are all stored ``cache_dim`` wide, the next width the tensor-core kernels take (or the larger of the two
        widths, rounded up to 8, beyond those), with zero rows appended to the projection weights and zero columns
        to the output projection: scores and results are what the unpadded heads give.  Different key and value
        widths need ``pad_heads``."""
        super().__init__(names)
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if head_dim <= 0 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is not supported: the attention kernels take head sizes up to 256")
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.window = int(window) if window else None
        # the reference divides scores by head_dim ** 0.5 (reference_attention.py:40)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.head_dim)
        self.position = build_part(POSITION_ENCODINGS, position) if position is not None else None
        self.bias, self.output_bias = bool(bias), bool(output_bias)
        self.qk_norm_eps = float(qk_norm_eps) if qk_norm_eps is not None else None
        self.qk_norm_unit_offset = bool(qk_norm_unit_offset)
        self.qk_norm_whole = bool(qk_norm_whole) and self.qk_norm_eps is not None
        self.values_from_keys = bool(values_from_keys)
        self.value_dim = int(value_dim) if value_dim is not None else self.head_dim
        self.unit_norm_eps = float(unit_norm_after_rotation_eps) if unit_norm_after_rotation_eps is not None else None
        self.pad_heads = bool(pad_heads)
        self.cache_dim = self._cache_dim()
        if self.cache_dim != self.head_dim or self.value_dim != self.head_dim or self.unit_norm_eps is not None:
            if self.qk_norm_eps is not None or self.values_from_keys or self.bias:
                raise ValueError("padded heads and the norm after the rotation go without biases, without a norm "
                                 "before the rotation and with a v projection")
        if (self.qk_norm_whole or self.values_from_keys) and (self.bias or self.qk_norm_unit_offset):
            raise ValueError("a norm over whole projections and values taken from the keys go without biases and "
                             "with plain norm weights")
        if self.values_from_keys and self.qk_norm_eps is not None and not self.qk_norm_whole:
            raise ValueError("values taken from the keys go with the norm over whole projections (or none)")
        self.w_qkv: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None
        self.b_qkv: torch.Tensor | None = None
        self.b_o: torch.Tensor | None = None
        self.w_q_norm: torch.Tensor | None = None
        self.w_k_norm: torch.Tensor | None = None

    # head widths the tensor-core attention kernels are built for
    KERNEL_WIDTHS = (32, 64, 128)

    def _cache_dim(self) -> int:
        widest = max(self.head_dim, self.value_dim)
        if not self.pad_heads:
            if self.value_dim != self.head_dim:
                raise ValueError("key and value heads of different widths need pad_heads")
            return self.head_dim
        fitting = [w for w in self.KERNEL_WIDTHS if w >= widest]
        width = fitting[0] if fitting else -(-widest // 8) * 8
        if width > 256:
            raise ValueError("the attention kernels take head sizes up to 256")
        return width

    def kv_requirement(self):
        return KVPageRequirement.keys_and_values(self.num_kv_heads, self.cache_dim, self.window)

    def kernel_needs(self):
        needs = {"attention_head_dims": {self.cache_dim}}
        if self._rotates_with_norm():
            needs["modules"] = {"rope_norm"}
        return needs

    def _rotates_with_norm(self) -> bool:
        magnitude = self.position.magnitude() if hasattr(self.position, "magnitude") else 1.0
        return self.unit_norm_eps is not None or magnitude != 1.0

    def expected_tensors(self):
        qd, kd = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        vd, od = self.num_kv_heads * self.value_dim, self.num_heads * self.value_dim
        exp = {
            self.names["q"]: TensorExpectation((qd, self.hidden_size)),
            self.names["k"]: TensorExpectation((kd, self.hidden_size)),
        }
        if not self.values_from_keys:
            exp[self.names["v"]] = TensorExpectation((vd, self.hidden_size))
        exp[self.names["o"]] = TensorExpectation((self.hidden_size, od))
        if self.bias:
            exp[self.names["q_bias"]] = TensorExpectation((qd,), "bias")
            exp[self.names["k_bias"]] = TensorExpectation((kd,), "bias")
            exp[self.names["v_bias"]] = TensorExpectation((kd,), "bias")
        if self.output_bias:
            exp[self.names["o_bias"]] = TensorExpectation((self.hidden_size,), "bias")
        if self.qk_norm_eps is not None:
            exp[self.names["q_norm"]] = TensorExpectation((qd if self.qk_norm_whole else self.head_dim,), "vector")
            exp[self.names["k_norm"]] = TensorExpectation((kd if self.qk_norm_whole else self.head_dim,), "vector")
        if self.position is not None:
            exp.update(self.position.expected_tensors())
        return exp

    def load(self, get, dtype, device):
        projections = ("q", "k") if self.values_from_keys else ("q", "k", "v")
        if self.cache_dim != self.head_dim or self.cache_dim != self.value_dim:
            # every head gets zero rows up to cache_dim; the output projection zero columns to match
            def padded(name, heads, width):
                w = get(self.names[name], "matrix").view(heads, width, self.hidden_size)
                return torch.nn.functional.pad(w, (0, 0, 0, self.cache_dim - width)).reshape(-1, self.hidden_size)

            self.w_qkv = torch.cat([padded("q", self.num_heads, self.head_dim),
                                    padded("k", self.num_kv_heads, self.head_dim),
                                    padded("v", self.num_kv_heads, self.value_dim)], dim=0).contiguous()
            w_o = get(self.names["o"], "matrix").view(self.hidden_size, self.num_heads, self.value_dim)
            self.w_o = torch.nn.functional.pad(w_o, (0, self.cache_dim - self.value_dim)).reshape(
                self.hidden_size, -1).contiguous()
        else:
            self.w_qkv = torch.cat([get(self.names[n], "matrix") for n in projections], dim=0).contiguous()
            self.w_o = get(self.names["o"], "matrix").contiguous()
        if self.bias:
            self.b_qkv = torch.cat([get(self.names[n], "bias") for n in ("q_bias", "k_bias", "v_bias")]).contiguous()
        if self.output_bias:
            self.b_o = get(self.names["o_bias"], "bias").contiguous()
        if self.qk_norm_eps is not None:
            self.w_q_norm = get(self.names["q_norm"], "vector").contiguous()
            self.w_k_norm = get(self.names["k_norm"], "vector").contiguous()
        if self.position is not None:
            self.position.load(get, dtype, device)

    def forward(self, x, ctx, cache):
        qkv = ops.linear(x, self.w_qkv, split_ok=True, bias=self.b_qkv)
        if self.qk_norm_whole or self.values_from_keys:
            qd, kd = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
            qkv = ops.qk_rownorm(qkv, self.w_q_norm, self.w_k_norm, self.qk_norm_eps or 0.0, qd, kd,
                                 values_from_keys=self.values_from_keys)
        elif self.qk_norm_eps is not None:
            qkv = ops.as_tensor(qkv)
            ops.rmsnorm_heads(qkv, self.w_q_norm, self.qk_norm_eps, 0, self.num_heads, self.head_dim,
                              self.qk_norm_unit_offset)
            ops.rmsnorm_heads(qkv, self.w_k_norm, self.qk_norm_eps, self.num_heads, self.num_kv_heads, self.head_dim,
                              self.qk_norm_unit_offset)
        view = ctx.groups[cache.group]
        rotary = self.position.rotary() if self.position is not None else None
        if self.position is not None and rotary is None:
            qkv = ops.as_tensor(qkv)
            self.position.apply(qkv, ctx, self.num_heads, self.num_kv_heads, self.head_dim)
        inv_freq, rotary_dim, interleaved = rotary if rotary is not None else (None, 0, False)
        pages = cache.kv_pages()
        if self._rotates_with_norm():
            qkv = ops.rope_norm_store(
                qkv, ctx.positions, inv_freq, self.position.magnitude() if rotary is not None else 1.0,
                view.slot_mapping if cache.writes else None, pages, self.num_heads, self.num_kv_heads,
                self.cache_dim, rotary_dim, interleaved, self.head_dim if self.unit_norm_eps is not None else 0,
                self.unit_norm_eps or 0.0,
            )
        else:
            qkv = ops.rope_store(
                qkv, ctx.positions, inv_freq,
                view.slot_mapping if cache.writes else None,
                pages, self.num_heads, self.num_kv_heads, self.cache_dim, rotary_dim, interleaved,
            )
        attn = ops.paged_attention(
            qkv, pages, view.block_table, ctx.positions, ctx.token_row, self.num_heads, self.scale,
            window=self.window, batch=ctx,
        )
        return ops.linear(attn, self.w_o, split_ok=True, add_into=getattr(ctx, "residual_sink", None), bias=self.b_o)
