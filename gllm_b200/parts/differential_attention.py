"""Differential attention over the paged cache.

Every query head has TWO query maps and every key head two key maps (stored head by head as ``[map 1, map 2]``, each
``dk`` wide); map ``m`` of a query head attends with a causal softmax over map ``m`` of its key head, both over the
same values, and the head's result is their difference:

    s_m(i, j) = cap * tanh(q_m,i . k_m,j * scale / cap)        a_m = softmax_j(s_m) V
    o = a_1 - lambda * a_2,    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff      (one number per layer)
    o <- o / sqrt(mean(o^2) + eps) * (1 - diff)                                      (per head, no weight)

The concatenated heads are multiplied by ``sigmoid(W_g h)`` (a gate that reads the mixer's input) and projected by
``W_o``.  The first ``rotary_dim`` columns of every map are rotated.  ``own_kv`` False: the layer has no key and
value projections and attends over the pages of the plan entry it reads (``PlanEntry.reads_cache_of``).  One fused
product ``[q | k | v | g]``, one kernel that rotates and stores, one attention kernel whose epilogue does the
difference, the norm and the gate (``csrc/attention_diff.cu``), one output product.
"""

from __future__ import annotations

import torch

from gllm_b200 import ops
from gllm_b200.ops import differential
from gllm_b200.parts.base import (
    POSITION_ENCODINGS,
    KVPageRequirement,
    Mixer,
    TensorExpectation,
    build_part,
    register_mixer,
)


@register_mixer("differential_attention")
class DifferentialAttention(Mixer):
    graph_safe_portions = True

    def __init__(self, names, hidden_size: int, heads: int, kv_heads: int, dk: int, dv: int, scale: float,
                 softcap: float, diff: float, eps: float, position=None, own_kv: bool = True):
        """``names``: ``q``, ``k``, ``v`` (with ``own_kv``), ``g``, ``o`` and the four vectors ``lq1``, ``lk1``,
        ``lq2``, ``lk2`` (``dk`` values each).  ``position``: the PartSpec of a rotary encoding over ``dk`` columns."""
        super().__init__(names)
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if not (0 < dk <= 256 and 0 < dv <= 256):
            raise ValueError("the differential-attention kernels take map and value widths up to 256")
        if not softcap > 0:
            raise ValueError("the cap of the scores must be positive")
        self.hidden_size, self.heads, self.kv_heads = int(hidden_size), int(heads), int(kv_heads)
        self.dk, self.dv = int(dk), int(dv)
        self.scale, self.softcap, self.diff, self.eps = float(scale), float(softcap), float(diff), float(eps)
        self.own_kv = bool(own_kv)
        self.position = build_part(POSITION_ENCODINGS, position) if position is not None else None
        if self.position is not None and getattr(type(self.position), "kind", None) != "rotary":
            raise ValueError("differential attention takes a rotary position encoding (or none)")
        self.w_in = self.w_o = None
        self.lam = 0.0

    def kernel_needs(self):
        return {"modules": {"attention_diff", "attention_diff_mma"}}

    def kv_requirement(self):
        return KVPageRequirement(((self.kv_heads, 2 * self.dk), (self.kv_heads, self.dv)), None)

    def _sections(self) -> list[tuple[str, int]]:
        out = [("q", self.heads * 2 * self.dk)]
        if self.own_kv:
            out += [("k", self.kv_heads * 2 * self.dk), ("v", self.kv_heads * self.dv)]
        return out + [("g", self.heads * self.dv)]

    def expected_tensors(self):
        exp = {self.names[n]: TensorExpectation((rows, self.hidden_size)) for n, rows in self._sections()}
        exp[self.names["o"]] = TensorExpectation((self.hidden_size, self.heads * self.dv))
        for n in ("lq1", "lk1", "lq2", "lk2"):
            exp[self.names[n]] = TensorExpectation((self.dk,), "bias")
        if self.position is not None:
            exp.update(self.position.expected_tensors())
        return exp

    def load(self, get, dtype, device):
        self.w_in = torch.cat([get(self.names[n], "matrix") for n, _ in self._sections()], dim=0).contiguous()
        self.w_o = get(self.names["o"], "matrix").contiguous()
        lq1, lk1, lq2, lk2 = (get(self.names[n], "bias") for n in ("lq1", "lk1", "lq2", "lk2"))
        # one number per layer, formed in fp32
        self.lam = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum()) + self.diff)
        if self.position is not None:
            self.position.load(get, dtype, device)

    def forward(self, x, ctx, cache):
        view = ctx.groups[cache.group]
        proj = ops.as_tensor(ops.linear(x, self.w_in))
        inv_freq, rotary_dim, interleaved = self.position.rotary() if self.position is not None else (None, 0, False)
        stores = self.own_kv and cache.writes
        differential.diff_rope_store(proj, ctx.positions, inv_freq, rotary_dim, interleaved,
                                     view.slot_mapping if stores else None, cache.pages, self.heads, self.kv_heads,
                                     self.dk, self.dv, self.own_kv, cache.block_size)
        gate_at = proj.shape[1] - self.heads * self.dv
        attn = differential.differential_attention(
            proj, proj[:, gate_at:], cache.pages, view.block_table, ctx.positions, ctx.token_row, self.heads,
            self.kv_heads, self.dk, self.dv, cache.block_size, self.scale, self.softcap, self.lam, self.eps,
            1.0 - self.diff, batch=ctx)
        return ops.linear(attn, self.w_o, split_ok=True, add_into=getattr(ctx, "residual_sink", None))
