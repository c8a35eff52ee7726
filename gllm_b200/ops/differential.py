"""Python entry points of the differential-attention kernels (``csrc/attention_diff.cu``).  As everywhere in
``gllm_b200.ops``: CUDA tensors only, no CPU path."""

from __future__ import annotations

import os

import torch

from gllm_b200.ops import _check, _cuda, _fn, _ptr, _stream, _suffix, status_word

# GLLM_B200_DIFF_MMA=0: the differential attention of bf16 models stays on the CUDA-core kernel (for measurements)
USE_TENSOR_CORES = os.environ.get("GLLM_B200_DIFF_MMA", "1") != "0"
# keys per CTA at least when single tokens' contexts are cut (a multiple of the key tile of 64), and the most ranges
SPLIT_KEYS = int(os.environ.get("GLLM_B200_DIFF_SPLIT_KEYS", "256"))
MAX_SPLITS = int(os.environ.get("GLLM_B200_DIFF_MAX_SPLITS", "16"))

_mma = None


def _mma_fns():
    global _mma
    if _mma is None:
        from ctypes import c_float, c_int, c_int64, c_void_p as P

        from gllm_b200.ops.build import load_module

        lib = load_module("attention_diff_mma")
        f = lib.gllm_attention_diff_mma
        f.argtypes = [P, c_int64, P, c_int64, P, c_int64, P, P, c_int, P, P, c_int, P, P, P, c_int, c_int, c_int, c_int,
                      c_int, c_int, c_int, c_int, c_float, c_float, c_float, c_float, c_float, c_int, c_int, P, P]
        f.restype = c_int
        lib.gllm_attention_diff_mma_supports.argtypes = [c_int, c_int]
        lib.gllm_attention_diff_mma_tokens_per_tile.argtypes = [c_int, c_int]
        _mma = (f, lib.gllm_attention_diff_mma_supports, lib.gllm_attention_diff_mma_tokens_per_tile)
    return _mma


def takes_tensor_cores(dtype: torch.dtype, dk: int, dv: int) -> bool:
    """True for the sizes the tensor-core kernel is built for (bf16; maps 32, 64 or 128 wide, values 32, 64, 96 or
    128)."""
    return dtype == torch.bfloat16 and dk in (32, 64, 128) and dv in (32, 64, 96, 128)


def _differential_attention_mma(q, gate, cache_pages, block_table, heads, kv_heads, dk, dv, block_size, scale, softcap,
                                lam, eps, out_scale, batch, out):
    """The tensor-core kernel and its combining kernel.  Steps whose tiles do not fill the GPU (single tokens over
    long contexts) cut every request's keys into ranges of at least ``SPLIT_KEYS`` keys, one CTA each."""
    f, _, tokens_per_tile = _mma_fns()
    n = q.shape[0]
    qt = tokens_per_tile(heads, kv_heads)
    group = heads // kv_heads
    head_tiles = 2 * kv_heads * (group if 64 % group or group > 64 else 1)
    tiles = -(-batch.max_q_len // qt) * head_tiles * batch.num_requests
    sms = torch.cuda.get_device_properties(q.device).multi_processor_count
    splits, tiles_per_split = 1, 0
    # a captured prompt portion is replayed for other contexts: under capture the ranges cover what a block-table
    # row can hold, not just the captured step's longest sequence (single tokens are captured per sequence bucket)
    longest = batch.max_seq_len
    if batch.max_q_len > 1 and torch.cuda.is_current_stream_capturing():
        longest = max(longest, block_table.shape[1] * block_size)
    if tiles < 4 * sms and longest > 2 * SPLIT_KEYS:
        want = min(MAX_SPLITS, -(-8 * sms // tiles))
        tiles_per_split = max(SPLIT_KEYS // 64, -(-(-(-longest // 64)) // want))
        splits = -(-(-(-longest // 64)) // tiles_per_split)
    partial = batch.workspace.get("differential_attention_partial", splits * 2 * n * heads * dv, torch.float32)
    stats = batch.workspace.get("differential_attention_stats", splits * 2 * n * heads * 2, torch.float32)
    code = f(q.data_ptr(), q.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, out.data_ptr(),
             out.stride(0), partial.data_ptr(), stats.data_ptr(), n, cache_pages.data_ptr(), block_table.data_ptr(),
             block_table.stride(0), batch.cu_q.data_ptr(), batch.context_lens.data_ptr(), batch.state_slots.data_ptr(),
             batch.num_requests, batch.max_q_len, heads, kv_heads, dk, dv, int(block_size), cache_pages.shape[0],
             float(scale), float(softcap), float(lam), float(eps), float(out_scale), splits, tiles_per_split,
             status_word(q.device).data_ptr(), _stream())
    _check(code, "differential_attention_mma")
    return out


def diff_rope_store(proj: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor | None, rotary_dim: int,
                    interleaved: bool, slot_mapping: torch.Tensor | None, cache_pages: torch.Tensor | None, heads: int,
                    kv_heads: int, dk: int, dv: int, own_kv: bool, block_size: int) -> torch.Tensor:
    """In place on ``proj [n, >= heads*2*dk (+ kv_heads*(2*dk + dv))]``: every query map (two per head, ``dk`` wide)
    has its first ``rotary_dim`` columns turned by ``position * inv_freq``; with ``own_kv`` the key maps that follow
    are turned the same way and go, with the values behind them, into ``cache_pages [pages, block_size * kv_heads *
    (2*dk + dv)]`` at ``slot_mapping`` (a page holds ``[kv_heads, block_size, 2*dk]`` keys, then ``[kv_heads,
    block_size, dv]`` values)."""
    _cuda(proj, "proj", contiguous=False)
    if proj.dim() != 2 or proj.stride(1) != 1:
        raise ValueError("proj must be [tokens, columns] with contiguous columns")
    _cuda(positions, "positions", torch.int32)
    n = proj.shape[0]
    need = heads * 2 * dk + (kv_heads * (2 * dk + dv) if own_kv else 0)
    if proj.shape[1] < need:
        raise ValueError("the projection is narrower than its query (and key and value) columns")
    if rotary_dim:
        _cuda(inv_freq, "inv_freq", torch.float32)
        if inv_freq.numel() != rotary_dim // 2:
            raise ValueError("inv_freq must hold rotary_dim/2 frequencies")
    num_pages = 0
    store = own_kv and slot_mapping is not None
    if store:
        _cuda(slot_mapping, "slot_mapping", torch.int32)
        _cuda(cache_pages, "cache_pages", proj.dtype)
        num_pages = cache_pages.shape[0]
        if cache_pages.shape[1] != block_size * kv_heads * (2 * dk + dv):
            raise ValueError("the cache pages do not hold two key maps and values of these widths")
    f = _fn("attention_diff", f"gllm_diff_rope_store_{_suffix(proj.dtype)}")
    _check(f(proj.data_ptr(), proj.stride(0), positions.data_ptr(), _ptr(inv_freq) if rotary_dim else None,
             _ptr(slot_mapping) if store else None, _ptr(cache_pages) if store else None, n, heads, kv_heads, dk, dv,
             int(rotary_dim), int(interleaved), int(own_kv), int(block_size), num_pages,
             status_word(proj.device).data_ptr(), _stream()), "diff_rope_store")
    return proj


def differential_attention(q: torch.Tensor, gate: torch.Tensor | None, cache_pages: torch.Tensor,
                           block_table: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor, heads: int,
                           kv_heads: int, dk: int, dv: int, block_size: int, scale: float, softcap: float,
                           lam: float, eps: float, out_scale: float, batch=None) -> torch.Tensor:
    """Per token and head, with the head's two rotated query maps ``q1, q2`` (``q [n, heads*2*dk]``, rows may be
    slices) and the cached key maps and values of its key head: ``a_m = softmax_j(cap * tanh(q_m . k_m,j * scale /
    cap)) V`` over the keys at positions up to the token's, ``o = a_1 - lam * a_2``, ``o`` divided by its root mean
    square over ``dv`` (eps inside the root), times ``out_scale``, times ``sigmoid(gate)`` (``gate [n, heads*dv]``,
    optional).  Returns ``[n, heads * dv]``.  With ``batch`` (the StepContext: per-request lengths, slots and the
    step's scratch) bf16 inputs of the sizes it takes run on the tensor-core kernel, everything else on the CUDA
    cores in fp32."""
    _cuda(q, "q", contiguous=False)
    _cuda(cache_pages, "cache_pages", q.dtype)
    _cuda(block_table, "block_table", torch.int32, contiguous=False)
    if q.dim() != 2 or q.stride(1) != 1 or q.shape[1] < heads * 2 * dk:
        raise ValueError("q must be [tokens, >= heads*2*dk] with contiguous columns")
    if gate is not None:
        _cuda(gate, "gate", q.dtype, contiguous=False)
        if gate.stride(1) != 1 or gate.shape[1] < heads * dv:
            raise ValueError("gate must be [tokens, >= heads*dv] with contiguous columns")
    if cache_pages.shape[1] != block_size * kv_heads * (2 * dk + dv):
        raise ValueError("the cache pages do not hold two key maps and values of these widths")
    n = q.shape[0]
    out = torch.empty((n, heads * dv), dtype=q.dtype, device=q.device)
    if (batch is not None and USE_TENSOR_CORES and takes_tensor_cores(q.dtype, dk, dv) and q.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and getattr(batch, "workspace", None) is not None):
        return _differential_attention_mma(q, gate, cache_pages, block_table, heads, kv_heads, dk, dv, block_size, scale,
                                           softcap, lam, eps, out_scale, batch, out)
    f = _fn("attention_diff", f"gllm_attention_diff_{_suffix(q.dtype)}")
    _check(f(q.data_ptr(), q.stride(0), _ptr(gate), gate.stride(0) if gate is not None else 0, out.data_ptr(),
             out.stride(0), cache_pages.data_ptr(), block_table.data_ptr(), block_table.stride(0), positions.data_ptr(),
             token_row.data_ptr(), n, heads, kv_heads, dk, dv, int(block_size), cache_pages.shape[0], float(scale),
             float(softcap), float(lam), float(eps), float(out_scale), status_word(q.device).data_ptr(), _stream()),
           "differential_attention")
    return out
