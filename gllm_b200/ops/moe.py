"""Python entry points of the routed-expert kernels (``csrc/moe.cu``).  As everywhere in ``gllm_b200.ops``: CUDA
tensors only, no CPU path; everything that varies between steps of equal shape (which experts were chosen, how
many tiles they fill) stays on the device, so a step can be captured in a CUDA graph."""

from __future__ import annotations

import torch

from gllm_b200.ops import _check, _cuda, _fn, _ptr, _stream, _suffix

TILE_ROWS = 16        # rows of one tile of the expert products: an expert's pairs are padded to a multiple of it
TENSOR_CORE_TILE_ROWS = 128     # the same for the tcgen05 products (the rows of one accumulator tile)


def route(logits: torch.Tensor, correction: torch.Tensor | None, top: int, groups: int = 1, groups_kept: int = 1,
          renormalize: bool = False, score: str = "sigmoid", group_score: str = "top2", renormalize_eps: float = 0.0,
          scale: float = 1.0):
    """From fp32 router logits ``[n, experts]`` to the chosen experts ``[n, top]`` int32 and their weights fp32.
    Scores ``s = sigmoid(logits)`` (``score`` "softmax": the softmax over all experts); the choice is made on
    ``s + correction`` among the experts of the ``groups_kept`` best of ``groups`` equal groups of neighbours (a
    group's score: the sum of its two largest choice scores, with ``group_score`` "max" its largest); the weights are
    the chosen ``s``, divided by their sum (plus ``renormalize_eps``) with ``renormalize``, times ``scale``."""
    if score not in ("sigmoid", "softmax") or group_score not in ("top2", "max"):
        raise ValueError("router scores are 'sigmoid' or 'softmax', group scores 'top2' or 'max'")
    _cuda(logits, "logits", torch.float32, contiguous=False)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("router logits must be [tokens, experts] with contiguous columns")
    if correction is not None:
        _cuda(correction, "correction", torch.float32)
        if correction.numel() != logits.shape[1]:
            raise ValueError("one correction value per expert is needed")
    n, experts = logits.shape
    ids = torch.empty((n, top), dtype=torch.int32, device=logits.device)
    weights = torch.empty((n, top), dtype=torch.float32, device=logits.device)
    _check(_fn("moe", "gllm_moe_route")(logits.data_ptr(), logits.stride(0), _ptr(correction), ids.data_ptr(),
                                        weights.data_ptr(), n, experts, int(top), int(groups), int(groups_kept),
                                        int(renormalize), int(score == "softmax"), int(group_score == "max"),
                                        float(renormalize_eps), float(scale), _stream()), "moe_route")
    return ids, weights


def align(ids: torch.Tensor, experts: int, tile_rows: int = TILE_ROWS, want_rows: bool = False):
    """The (token, slot) pairs sorted by expert in tiles of ``tile_rows`` rows: ``(sorted [max_tiles * tile_rows]``
    (pair index or -1), ``tile_expert [max_tiles]``, ``num_tiles [1])``, all int32 on the device; with
    ``want_rows`` also ``row_of_pair [pairs]``, the row each pair got."""
    _cuda(ids, "ids", torch.int32)
    pairs = ids.numel()
    max_tiles = -(-pairs // tile_rows) + min(experts, pairs)
    sorted_pairs = torch.empty(max_tiles * tile_rows, dtype=torch.int32, device=ids.device)
    tile_expert = torch.empty(max_tiles, dtype=torch.int32, device=ids.device)
    num_tiles = torch.empty(1, dtype=torch.int32, device=ids.device)
    row_of_pair = torch.empty(pairs, dtype=torch.int32, device=ids.device) if want_rows else None
    _check(_fn("moe", "gllm_moe_align")(ids.data_ptr(), sorted_pairs.data_ptr(), tile_expert.data_ptr(),
                                        num_tiles.data_ptr(), _ptr(row_of_pair), pairs, int(experts), int(tile_rows),
                                        max_tiles, _stream()), "moe_align")
    if want_rows:
        return sorted_pairs, tile_expert, num_tiles, row_of_pair
    return sorted_pairs, tile_expert, num_tiles


def gather_rows(x: torch.Tensor, top: int, row_of_pair: torch.Tensor, rows: int) -> torch.Tensor:
    """``out[row_of_pair[p]] = x[p // top]`` (bf16, ``[rows, width]``): the tokens' rows in the order of the sorted
    pairs.  Rows that no pair owns are left as they are: the products' rows do not mix, and nobody reads theirs."""
    _cuda(x, "x", torch.bfloat16, contiguous=False)
    _cuda(row_of_pair, "row_of_pair", torch.int32)
    out = torch.empty((rows, x.shape[1]), dtype=x.dtype, device=x.device)
    _check(_fn("moe", "gllm_moe_gather_bf16")(x.data_ptr(), x.stride(0), row_of_pair.data_ptr(), out.data_ptr(),
                                              row_of_pair.numel(), int(top), x.shape[1], _stream()), "moe_gather")
    return out


def tensor_cores_take(dtype: torch.dtype, width: int, ff: int, gated: bool = True) -> bool:
    """Whether the experts' products run on the tcgen05 kernel: bf16, rows that start on 16 bytes, and (for gated
    experts) gate and up rows stacked in blocks of 64."""
    return dtype == torch.bfloat16 and width % 8 == 0 and ff % (64 if gated else 8) == 0


def expert_product(a: torch.Tensor, rows_per_input: int, weight: torch.Tensor, plan, n_pairs: int, gated: bool,
                   relu_squared: bool = False):
    """``out[pair] = a[pair // rows_per_input] @ weight[expert of pair].T`` for the pairs of ``plan`` (what
    ``align`` returned).  ``weight [experts, rows, k]``; ``gated``: its rows are gate rows then up rows and the
    result is ``silu(gate) * up`` in the activation type ``[n_pairs, rows / 2]``; ``relu_squared`` (experts without a
    gate): ``max(result, 0) ** 2`` in the activation type ``[n_pairs, rows]``; otherwise fp32 ``[n_pairs, rows]``."""
    _cuda(a, "a", contiguous=False)
    _cuda(weight, "weight", a.dtype)
    if a.dim() != 2 or a.stride(1) != 1 or weight.dim() != 3 or weight.shape[2] != a.shape[1]:
        raise ValueError("the expert product takes rows of contiguous columns and weights [experts, rows, k]")
    sorted_pairs, tile_expert, num_tiles = plan
    rows, k = weight.shape[1], weight.shape[2]
    if gated and (rows % 2 or relu_squared):
        raise ValueError("gate and up rows come in equal numbers, and the gate is the activation")
    n_cols = rows // 2 if gated else rows
    out = torch.empty((n_pairs, n_cols), dtype=a.dtype if gated or relu_squared else torch.float32, device=a.device)
    f = _fn("moe", f"gllm_moe_gemm_{_suffix(a.dtype)}")
    _check(f(a.data_ptr(), a.stride(0), int(rows_per_input), weight.data_ptr(), weight.stride(0),
             n_cols * k if gated else 0, sorted_pairs.data_ptr(), tile_expert.data_ptr(), num_tiles.data_ptr(),
             out.data_ptr(), tile_expert.numel(), n_cols, k, TILE_ROWS, int(relu_squared), _stream()), "moe_gemm")
    return out


def combine(y: torch.Tensor, weights: torch.Tensor, shared: torch.Tensor | None, out_dtype: torch.dtype,
            row_of_pair: torch.Tensor | None = None, shared_gate: torch.Tensor | None = None) -> torch.Tensor:
    """``out[t] = sum_s weights[t, s] * y[t * top + s] (+ shared[t])``, summed in slot order in fp32; with
    ``row_of_pair`` the pair's result is row ``row_of_pair[t * top + s]`` of ``y``; with ``shared_gate`` (fp32, one
    logit per token; may be a column of a wider matrix) the shared result is multiplied by its sigmoid."""
    _cuda(y, "y", torch.float32)
    _cuda(weights, "weights", torch.float32)
    n, top = weights.shape
    width = y.shape[1]
    if row_of_pair is not None:
        _cuda(row_of_pair, "row_of_pair", torch.int32)
    if (y.shape[0] != n * top and row_of_pair is None) or (row_of_pair is not None and row_of_pair.numel() != n * top):
        raise ValueError("one result row per (token, slot) pair is needed")
    if shared is not None:
        _cuda(shared, "shared", out_dtype)
        if tuple(shared.shape) != (n, width):
            raise ValueError("the shared expert's result does not fit")
    gate_stride = 0
    if shared_gate is not None:
        _cuda(shared_gate, "shared_gate", torch.float32, contiguous=False)
        if shared is None or shared_gate.dim() != 1 or shared_gate.numel() != n:
            raise ValueError("the shared expert's gate is one logit per token")
        gate_stride = shared_gate.stride(0)
    out = torch.empty((n, width), dtype=out_dtype, device=y.device)
    _check(_fn("moe", f"gllm_moe_combine_{_suffix(out_dtype)}")(y.data_ptr(), weights.data_ptr(), _ptr(shared),
                                                               out.data_ptr(), _ptr(row_of_pair), n, top, width,
                                                               _ptr(shared_gate), gate_stride, _stream()), "moe_combine")
    return out


def relu_squared_rows(x: torch.Tensor) -> torch.Tensor:
    """``max(x, 0) ** 2`` of fp32 ``x``, rounded to bf16: between the two tensor-core products of experts without
    a gate."""
    _cuda(x, "x", torch.float32)
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    _check(_fn("moe", "gllm_moe_relu_sq_bf16")(x.data_ptr(), out.data_ptr(), x.numel(), _stream()), "moe_relu_sq")
    return out


def apply_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, w_gate_up: torch.Tensor,
                  w_down: torch.Tensor, shared: torch.Tensor | None, tensor_cores: bool, gated: bool = True,
                  shared_gate: torch.Tensor | None = None) -> torch.Tensor:
    """``out[t] = sum_s weights[t, s] * expert_{ids[t, s]}(x[t]) (+ shared[t])`` with ``expert_e(x) = w_down[e]
    (silu(gate) * up)``.  ``tensor_cores``: ``w_gate_up [experts, 2 * ff, width]`` is stacked per expert by
    ``interleave_gate_up``; the tokens' rows are copied into the order of the sorted pairs, both products read and
    write rows in that order on the tcgen05 kernel, and the weighted sum looks every pair's row up.  Otherwise
    ``w_gate_up`` holds an expert's gate rows, then its up rows, and the CUDA-core kernel runs.  ``gated`` False:
    experts without a gate, ``expert_e(x) = w_down[e] relu(w_up[e] x)^2`` with ``w_gate_up [experts, ff, width]`` the
    up weights.  ``shared_gate``: see ``combine``."""
    experts, (_, top), pairs = w_gate_up.shape[0], ids.shape, ids.numel()
    if not tensor_cores:
        plan = align(ids, experts)
        hidden = expert_product(x, top, w_gate_up, plan, pairs, gated=gated, relu_squared=not gated)
        y = expert_product(hidden, 1, w_down, plan, pairs, gated=False)
        return combine(y, weights, shared, x.dtype, shared_gate=shared_gate)
    from gllm_b200.ops import gemm_bf16

    _, tile_expert, num_tiles, row_of_pair = align(ids, experts, TENSOR_CORE_TILE_ROWS, want_rows=True)
    wide = pairs > 2048
    xs = gather_rows(x, top, row_of_pair, tile_expert.numel() * TENSOR_CORE_TILE_ROWS)
    hidden = gemm_bf16.linear_grouped(xs, w_gate_up, tile_expert, num_tiles, gated=gated, wide=wide)
    if not gated:
        hidden = relu_squared_rows(hidden)
    y = gemm_bf16.linear_grouped(hidden, w_down, tile_expert, num_tiles, gated=False, wide=wide)
    return combine(y, weights, shared, x.dtype, row_of_pair, shared_gate=shared_gate)
