"""Single-kernel workloads: each builds synthetic inputs, runs one kernel of the
engine a few times with an L2 flush between runs, and reports its time beside
the bytes or flops it has to move.  ``python bench.py --kernel NAME`` runs one;
the same command under ``ncu`` gives the profiles kept under ``profiles/``."""

from __future__ import annotations

import math

import torch


def _flush_l2(buf):
    buf.zero_()


def _time(fn, iters: int, flush) -> float:
    """Median device time of ``fn`` in microseconds."""
    times = []
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    for _ in range(iters):
        _flush_l2(flush)
        # keep the GPU busy while the host queues the launches, so the events bracket device time only
        torch.cuda._sleep(400_000)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end) * 1e3)
    times.sort()
    return times[len(times) // 2]


def _paged_cache(batch, context, hkv, d, block_size, extra_tokens=0, sequential=0):
    """A pool holding ``batch`` requests of ``context`` tokens on scattered pages
    (``sequential``: each request's pages lie one after another instead)."""
    pages_per_req = -(-(context + extra_tokens) // block_size)
    num_pages = batch * pages_per_req + 1
    g = torch.Generator(device="cuda").manual_seed(0)
    pool = torch.randn((num_pages, 2, hkv, block_size, d), generator=g, device="cuda", dtype=torch.float32)
    pool = pool.to(torch.bfloat16)
    perm = torch.randperm(num_pages - 1, generator=g, device="cuda").to(torch.int32)
    if sequential:
        perm = torch.arange(num_pages - 1, device="cuda", dtype=torch.int32)
    table = perm[: batch * pages_per_req].view(batch, pages_per_req).contiguous()
    return pool, table


def attention_decode(batch=64, context=2048, hq=32, hkv=8, d=64, block_size=16, iters=5, peaks=None, sequential=0,
                     stream=1):
    from gllm_b200.ops import attention_bf16

    pool, table = _paged_cache(batch, context, hkv, d, block_size, sequential=sequential)
    qkv = torch.randn(batch, (hq + 2 * hkv) * d, device="cuda").to(torch.bfloat16)
    positions = torch.full((batch,), context - 1, dtype=torch.int32, device="cuda")
    rows = torch.arange(batch, dtype=torch.int32, device="cuda")
    out = torch.empty(batch, hq * d, dtype=torch.bfloat16, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    class _WS:
        def __init__(self):
            self.b = {}

        def get(self, name, n, dt):
            if name not in self.b:
                self.b[name] = torch.empty(n, dtype=dt, device="cuda")
            return self.b[name]

    ws = _WS()
    fn = lambda: attention_bf16.decode_attention(qkv, qkv.shape[1], pool, table, positions, rows, hq,
                                                 1.0 / math.sqrt(d), 0, context, ws, out,
                                                 kernel="stream" if stream else "split")
    us = _time(fn, iters, flush)
    nbytes = batch * context * 2 * hkv * d * 2
    gbs = nbytes / us / 1e3
    return {"kernel": "attention_decode (stream + merge)" if stream else "attention_decode (split + merge)", "us": round(us, 2), "bytes": nbytes,
            "achieved_gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4),
            "shape": dict(batch=batch, context=context, heads=hq, kv_heads=hkv, head_dim=d, block_size=block_size)}


def attention_prefill(tokens=2048, context=0, hq=32, hkv=8, d=64, block_size=16, iters=5, peaks=None, tmem=1):
    from gllm_b200.ops import attention_bf16

    pool, table = _paged_cache(1, context + tokens, hkv, d, block_size)
    qkv = torch.randn(tokens, (hq + 2 * hkv) * d, device="cuda").to(torch.bfloat16)
    cu = torch.tensor([0, tokens], dtype=torch.int32, device="cuda")
    ctx = torch.tensor([context], dtype=torch.int32, device="cuda")
    slots = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.empty(tokens, hq * d, dtype=torch.bfloat16, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    kernel = attention_bf16.prefill_attention_tmem if tmem else attention_bf16.prefill_attention
    fn = lambda: kernel(qkv, qkv.shape[1], pool, table, cu, ctx, slots, 1, tokens, hq, 1.0 / math.sqrt(d), 0, out)
    us = _time(fn, iters, flush)
    flops = 4.0 * d * hq * (tokens * context + tokens * (tokens + 1) / 2)
    tf = flops / us / 1e6
    return {"kernel": "attention_prefill (tcgen05)" if tmem else "attention_prefill (mma.sync)", "us": round(us, 2), "flops": flops, "achieved_tflops": round(tf, 1),
            "frac_of_bf16_peak": round(tf / peaks["bf16_tflops"], 4),
            "shape": dict(tokens=tokens, context=context, heads=hq, kv_heads=hkv, head_dim=d, block_size=block_size)}


def linear(m=8, n=16384, k=2048, iters=5, peaks=None, out_fp32=False, gated=0, split=0, acc=0):
    """x [m, k] times a [n, k] weight.  ``gated``: the weight is a gate/up stack (n = 2 x features) and
    the epilogue writes SiLU(gate) * up.  ``split``: a product cut along K leaves its splits unsummed,
    as the decode step's products do (their consumers add them).  ``acc``: the product adds itself into
    an fp32 matrix (the residual stream), as the products that end a branch do for up to 64 tokens."""
    from gllm_b200 import ops

    x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
    out = torch.empty(m, n, dtype=torch.float32 if out_fp32 else torch.bfloat16, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    resid = torch.zeros(m, n, dtype=torch.float32, device="cuda")
    if gated:
        fn = lambda: ops.linear_gated(x, w)
    elif acc:
        fn = lambda: ops.linear(x, w, split_ok=True, add_into=resid)
    elif split:
        fn = lambda: ops.linear(x, w, split_ok=True)
    else:
        fn = lambda: ops.linear(x, w, out_dtype=out.dtype, out=out)
    us = _time(fn, iters, flush)
    nbytes = (m * k + n * k) * 2 + out.numel() * out.element_size()
    flops = 2.0 * m * n * k
    gbs, tf = nbytes / us / 1e3, flops / us / 1e6
    name = "linear (gated epilogue)" if gated else ("linear (adds into the residual)" if acc else
                                                     ("linear (unsummed splits)" if split else "linear"))
    return {"kernel": name, "us": round(us, 2), "achieved_gbs": round(gbs, 1), "achieved_tflops": round(tf, 1),
            "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4), "frac_of_bf16_peak": round(tf / peaks["bf16_tflops"], 4),
            "shape": dict(m=m, n=n, k=k)}


def linear_f32(m=2048, n=8192, k=2048, iters=5, peaks=None):
    """The true 32-bit product (FFMA, no tensor-core mode) of the float32 path."""
    from gllm_b200 import ops

    x = torch.randn(m, k, device="cuda")
    w = torch.randn(n, k, device="cuda") * 0.02
    out = torch.empty(m, n, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    us = _time(lambda: ops.linear(x, w, out=out), iters, flush)
    nbytes = (m * k + n * k + m * n) * 4
    flops = 2.0 * m * n * k
    return {"kernel": "linear_f32 (FFMA)", "us": round(us, 2), "achieved_tflops": round(flops / us / 1e6, 1),
            "achieved_gbs": round(nbytes / us / 1e3, 1), "frac_of_hbm_peak": round(nbytes / us / 1e3 / peaks["hbm_gbs"], 4),
            "shape": dict(m=m, n=n, k=k)}


def decode_step(batch=8, context=2048, layers=2, iters=3, peaks=None):
    """Whole decode steps of a model with the Llama 3.2 1B layer sizes and ``layers`` layers, every kernel
    launched on its own (no CUDA graph), so that a profiler lists them one by one."""
    import os
    import shutil
    import tempfile

    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine
    from gllm_b200.config import load_config
    from gllm_b200.config.presets import load_preset
    from gllm_b200.weights import write_random_model

    raw = load_preset("llama-3.2-1b")
    raw["num_hidden_layers"] = layers
    tmp = tempfile.mkdtemp(prefix="gllm_b200_kernel_bench_")
    try:
        folder = write_random_model(os.path.join(tmp, "model"), load_config(raw), seed=0, std=0.02)
        params = GeneratorParams(block_size=16, max_batch_size=max(batch, 8), max_seq_len=4096, model_dtype="bfloat16",
                                 cuda_graphs=False)
        engine = LLMEngine(folder, params, device="cuda:0")
    finally:
        shutil.rmtree(tmp, ignore_errors=True)
    g = torch.Generator().manual_seed(0)
    vocab = engine.config.vocab_size
    states = [engine.submit(GenerationRequest(prompt_token_ids=torch.randint(0, vocab, (context,), generator=g).tolist(),
                                              max_new_tokens=64, temperature=0.0, ignore_eos=True)) for _ in range(batch)]
    while any(s.num_computed < len(s.prompt_token_ids) for s in states):
        engine.step()
    for _ in range(3):
        engine.step()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(iters):
        engine.step()
    end.record()
    torch.cuda.synchronize()
    us = start.elapsed_time(end) * 1e3 / iters
    return {"kernel": "decode_step (no graph)", "us": round(us, 2), "shape": dict(batch=batch, context=context, layers=layers)}


def add_rmsnorm(rows=8, hidden=2048, splits=8, post=0, iters=5, peaks=None):
    """resid += (sum of ``splits`` fp32 partial products, 0: a summed bf16 branch), then RMSNorm: the
    kernel between two products of a layer.  ``post``: the branch is RMS-normed with a weight of its own
    before it is added (the norm after a sublayer of a layer that norms both sides of it)."""
    from gllm_b200 import ops

    resid = torch.randn(rows, hidden, device="cuda")
    weight = torch.ones(hidden, device="cuda")
    parts = torch.randn(max(splits, 1), rows, hidden, device="cuda")
    branch = ops.SplitSum(parts, torch.bfloat16) if splits else parts[0].to(torch.bfloat16)
    if post:
        branch = ops.Pending(branch, torch.ones(hidden, device="cuda"), 1e-5)
    out = torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    us = _time(lambda: ops.add_rmsnorm(branch, resid, weight, 1e-5, torch.bfloat16, out=out), iters, flush)
    nbytes = rows * hidden * ((4 * splits if splits else 2) + 4 + 4 + 2) + hidden * 4 * (2 if post else 1)
    gbs = nbytes / us / 1e3
    return {"kernel": "add_rmsnorm (normed branch)" if post else "add_rmsnorm", "us": round(us, 2), "bytes": nbytes,
            "achieved_gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4),
            "shape": dict(rows=rows, hidden=hidden, splits=splits)}


def argmax(rows=8, vocab=128256, iters=5, peaks=None):
    from gllm_b200 import ops

    logits = torch.randn(rows, vocab, device="cuda")
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    us = _time(lambda: ops.argmax(logits, out=out), iters, flush)
    nbytes = rows * vocab * 4
    gbs = nbytes / us / 1e3
    return {"kernel": "argmax", "us": round(us, 2), "bytes": nbytes, "achieved_gbs": round(gbs, 1),
            "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 4), "shape": dict(rows=rows, vocab=vocab)}


# ------------------------------------------------------------------ kernels of the mixers with a state
class _Scratch:
    def __init__(self):
        self.b = {}

    def get(self, name, n, dt):
        if name not in self.b or self.b[name].numel() < n:
            self.b[name] = torch.empty(n, dtype=dt, device="cuda")
        return self.b[name][:n]


class _Batch:
    """What the kernels read of a step: ``requests`` requests of ``q_len`` tokens after ``context`` cached ones."""

    def __init__(self, requests, q_len, context):
        self.num_requests, self.max_q_len, self.max_seq_len = requests, q_len, context + q_len
        self.cu_q = (torch.arange(requests + 1, dtype=torch.int32, device="cuda") * q_len).contiguous()
        self.context_lens = torch.full((requests,), context, dtype=torch.int32, device="cuda")
        self.state_slots = torch.arange(requests, dtype=torch.int32, device="cuda")
        self.positions = (context + torch.arange(q_len, dtype=torch.int32, device="cuda")).repeat(requests).contiguous()
        self.token_row = torch.arange(requests, dtype=torch.int32, device="cuda").repeat_interleave(q_len).contiguous()
        self.workspace = _Scratch()


def _result(name, us, peaks, shape, nbytes=None, flops=None):
    out = {"kernel": name, "us": round(us, 2), "shape": shape}
    if nbytes is not None:
        gbs = nbytes / us / 1e3
        out.update(bytes=int(nbytes), achieved_gbs=round(gbs, 1), frac_of_hbm_peak=round(gbs / peaks["hbm_gbs"], 4))
    if flops is not None:
        tf = flops / us / 1e6
        out.update(flops=flops, achieved_tflops=round(tf, 2), frac_of_bf16_peak=round(tf / peaks["bf16_tflops"], 4))
    return out


def sigmoid_attention(tokens=2048, batch=1, context=0, hq=32, hkv=8, dk=64, dv=64, block_size=16, iters=5, peaks=None,
                      mma=1):
    """``batch`` requests of ``tokens`` new tokens over ``context`` cached ones (tokens=1: a decode step)."""
    from gllm_b200.ops import stateful

    stateful.USE_TENSOR_CORES = bool(mma)
    pages_per_req = -(-(context + tokens) // block_size)
    num_pages = batch * pages_per_req + 1
    g = torch.Generator(device="cuda").manual_seed(0)
    pool = torch.randn((num_pages, block_size * hkv * (dk + dv)), generator=g, device="cuda").to(torch.bfloat16)
    table = torch.randperm(num_pages - 1, generator=g, device="cuda").to(torch.int32).view(batch, pages_per_req).contiguous()
    qkv = torch.randn(batch * tokens, hq * dk + hkv * (dk + dv), device="cuda").to(torch.bfloat16)
    bias = torch.full((hq,), -4.0, device="cuda")
    b = _Batch(batch, tokens, context)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fn = lambda: stateful.sigmoid_attention(qkv, pool, table, b.positions, b.token_row, bias, hq, hkv, dk, dv, block_size,
                                            dk ** -0.5, batch=b)
    us = _time(fn, iters, flush)
    flops = 2.0 * (dk + dv) * hq * batch * (tokens * context + tokens * (tokens + 1) / 2)
    nbytes = batch * (context + tokens) * hkv * (dk + dv) * 2 + qkv.numel() * 2
    return _result("sigmoid_attention (mma.sync)" if mma else "sigmoid_attention (CUDA cores)", us, peaks,
                   dict(tokens=tokens, batch=batch, context=context, heads=hq, kv_heads=hkv, dk=dk, dv=dv), nbytes, flops)


def latent_attention(tokens=2048, batch=1, context=0, heads=16, rank=512, rot=64, block_size=16, iters=5, peaks=None,
                     mma=1, split_keys=0):
    """``batch`` requests of ``tokens`` new tokens over ``context`` cached ones (tokens=1: a decode step) through
    the latent attention kernel (with its merge when the keys are cut into ranges).  FLOPs: both products over the
    visible keys; bytes: every request's cached vectors once, the queries and the result."""
    from gllm_b200.ops import latent

    latent.USE_TENSOR_CORES = bool(mma)
    if split_keys:
        latent.SPLIT_KEYS = split_keys          # the shortest range of keys a CTA takes
    dk = rank + rot
    pages_per_req = -(-(context + tokens) // block_size)
    num_pages = batch * pages_per_req + 1
    g = torch.Generator(device="cuda").manual_seed(0)
    pool = torch.randn((num_pages, block_size * dk), generator=g, device="cuda").to(torch.bfloat16)
    table = torch.randperm(num_pages - 1, generator=g, device="cuda").to(torch.int32).view(batch, pages_per_req).contiguous()
    q_head = 128 + rot
    rows = torch.randn(batch * tokens, heads * q_head + 8 * (-(-heads // 8)), device="cuda").to(torch.bfloat16)
    qa = torch.randn(batch * tokens, heads * rank, device="cuda").to(torch.bfloat16)
    b = _Batch(batch, tokens, context)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fn = lambda: latent.attention_latent(qa, rows, q_head, 128, heads * q_head, pool, table, b.positions, b.token_row,
                                         heads, rank, rot, block_size, dk ** -0.5, batch=b)
    us = _time(fn, iters, flush)
    flops = 2.0 * (dk + rank) * heads * batch * (tokens * context + tokens * (tokens + 1) / 2)
    nbytes = batch * (context + tokens) * dk * 2 + qa.numel() * 4 + batch * tokens * heads * rot * 2
    return _result("latent_attention (mma.sync)" if mma else "latent_attention (CUDA cores)", us, peaks,
                   dict(tokens=tokens, batch=batch, context=context, heads=heads, rank=rank, rot=rot), nbytes, flops)


def head_linear(tokens=2048, heads=16, inner=128, outer=512, iters=5, peaks=None, mma=1):
    """One product per head, ``[tokens, inner] x [outer, inner]^T`` for each of ``heads`` heads in one launch."""
    from gllm_b200.ops import latent

    latent.USE_TENSOR_CORES = bool(mma)
    x = torch.randn(tokens, heads * inner, device="cuda").to(torch.bfloat16)
    w = (torch.randn(heads, outer, inner, device="cuda") * 0.05).to(torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    us = _time(lambda: latent.head_linear(x, inner, w), iters, flush)
    return _result("head_linear (mma.sync)" if mma else "head_linear (CUDA cores)", us, peaks,
                   dict(tokens=tokens, heads=heads, inner=inner, outer=outer),
                   (x.numel() + w.numel() + tokens * heads * outer) * 2, 2.0 * tokens * heads * inner * outer)


def matrix_recurrence(tokens=2048, batch=1, heads=16, dk=64, dv=128, mode=0, iters=5, peaks=None):
    """mode 0: gated linear attention; mode 1: the matrix memory with exponential gates."""
    from gllm_b200.ops import stateful

    n = batch * tokens
    q = torch.randn(n, heads * dk, device="cuda").to(torch.bfloat16)
    k = torch.randn(n, heads * dk, device="cuda").to(torch.bfloat16)
    v = torch.randn(n, heads * dv, device="cuda").to(torch.bfloat16)
    gates = torch.randn(n, heads * dk if mode == 0 else 2 * heads, device="cuda")
    gbias = torch.zeros(gates.shape[1], device="cuda")
    lower = torch.rand(heads * dk, device="cuda") * 0.9
    state = torch.zeros(batch + 1, heads, dv + mode, dk, device="cuda")
    mstate = torch.zeros(batch + 1, heads, device="cuda")
    b = _Batch(batch, tokens, 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fn = lambda: stateful.matrix_recurrence(mode, q, k if mode else None, v, gates, gbias, None if mode else lower, 12.0,
                                            dk ** -0.5, state, mstate if mode else None, b.cu_q, b.state_slots, batch,
                                            heads, dk, dv, max_q_len=tokens)
    us = _time(fn, iters, flush)
    nbytes = 2 * batch * heads * dk * (dv + mode) * 4 + n * heads * ((2 + mode) * dk * 2 + dv * 2 + dv * 4) + gates.numel() * 4
    flops = 4.0 * n * heads * dk * dv
    return _result("matrix_recurrence (exponential gates)" if mode else "matrix_recurrence (gated linear)", us, peaks,
                   dict(tokens=tokens, batch=batch, heads=heads, dk=dk, dv=dv), nbytes, flops)


def selective_scan(tokens=2048, batch=1, channels=4096, states=16, dt_rank=128, taps=4, iters=5, peaks=None):
    from gllm_b200.ops import stateful

    n = batch * tokens
    xz = torch.randn(n, 2 * channels, device="cuda").to(torch.bfloat16)
    xc = torch.randn(n, channels, device="cuda").to(torch.bfloat16)
    proj = torch.randn(n, dt_rank + 2 * states, device="cuda").to(torch.bfloat16)
    dt_raw = torch.randn(n, channels, device="cuda")
    dt_b, D = torch.zeros(channels, device="cuda"), torch.ones(channels, device="cuda")
    A = -torch.rand(channels, states, device="cuda") - 0.1
    ssm = torch.zeros(batch + 1, channels, states, device="cuda")
    conv = torch.zeros(batch + 1, taps - 1, channels, device="cuda")
    b = _Batch(batch, tokens, 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fn = lambda: stateful.selective_scan(xc, dt_raw, dt_b, A, proj, dt_rank, dt_rank + states, D, xz, channels, ssm, conv,
                                         taps, b.cu_q, b.state_slots, batch, max_q_len=tokens)
    us = _time(fn, iters, flush)
    nbytes = 2 * batch * channels * states * 4 + n * (channels * (2 + 4 + 2 + 2) + 2 * states * 2)
    return _result("selective_scan", us, peaks, dict(tokens=tokens, batch=batch, channels=channels, states=states), nbytes,
                   9.0 * n * channels * states)


def conv_silu(tokens=2048, batch=1, channels=4096, taps=4, iters=5, peaks=None):
    from gllm_b200.ops import stateful

    n = batch * tokens
    xz = torch.randn(n, 2 * channels, device="cuda").to(torch.bfloat16)
    w, bias = torch.randn(channels, taps, device="cuda"), torch.zeros(channels, device="cuda")
    conv = torch.zeros(batch + 1, taps - 1, channels, device="cuda")
    b = _Batch(batch, tokens, 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    us = _time(lambda: stateful.conv_silu(xz[:, :channels], w, bias, conv, b.positions, b.token_row), iters, flush)
    return _result("conv_silu", us, peaks, dict(tokens=tokens, batch=batch, channels=channels, taps=taps),
                   n * channels * 4)


def stream_mix_norm(rows=2048, hidden=2048, streams=4, iters=5, peaks=None):
    from gllm_b200.ops import stateful

    resid = torch.randn(rows, streams * hidden, device="cuda")
    y = torch.randn(rows, hidden, device="cuda").to(torch.bfloat16)
    mix = torch.eye(streams, device="cuda").contiguous()
    vec = torch.ones(streams, device="cuda")
    weight = torch.ones(hidden, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    us = _time(lambda: stateful.stream_mix_norm(y, resid, mix, vec, vec, weight, 1e-5, torch.bfloat16, streams), iters, flush)
    return _result("stream_mix_norm", us, peaks, dict(rows=rows, hidden=hidden, streams=streams),
                   rows * hidden * (8 * streams + 4))


def delta_rule(tokens=2048, batch=1, heads=16, dk=64, dv=128, taps=4, prep=0, iters=5, peaks=None):
    """The gated delta rule's recurrence over ``batch`` requests of ``tokens`` tokens (tokens=1: a decode step);
    ``prep=1`` times the kernel before it instead (convolution, SiLU, unit norms, decays, beta)."""
    from gllm_b200.ops import stateful

    n = batch * tokens
    channels = 2 * heads * dk + heads * dv
    b = _Batch(batch, tokens, 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    shape = dict(tokens=tokens, batch=batch, heads=heads, dk=dk, dv=dv)
    x = torch.randn(n, channels, device="cuda").to(torch.bfloat16)
    conv_w = torch.randn(channels, taps, device="cuda") * 0.5
    conv_state = torch.zeros(batch + 1, taps - 1, channels, device="cuda")
    raw, braw = torch.randn(n, heads * dk, device="cuda"), torch.randn(n, heads, device="cuda")
    dt_bias, A_log = torch.zeros(heads * dk, device="cuda"), torch.full((heads,), -3.0, device="cuda")
    run_prep = lambda: stateful.delta_prep(x, conv_w, conv_state, b.positions, b.token_row, b.cu_q, b.state_slots, batch,
                                           raw, dt_bias, A_log, braw, heads, heads, dk, dv, 1e-6, dk ** -0.5)
    if prep:
        us = _time(run_prep, iters, flush)
        nbytes = n * (channels * 2 + heads * dk * 4 + heads * 4) + n * (channels + heads * dk + heads) * 4
        return _result("delta_prep", us, peaks, dict(shape, taps=taps), nbytes)
    qk, v, g, beta = run_prep()
    state = torch.zeros(batch + 1, heads, dv, dk, device="cuda")
    fn = lambda: stateful.delta_rule(qk, v, g, beta, state, b.cu_q, b.state_slots, batch, heads, heads, dk, dv,
                                     max_q_len=tokens)
    us = _time(fn, iters, flush)
    nbytes = 2 * batch * heads * dk * dv * 4 + n * heads * (3 * dk + 2 * dv + 1) * 4
    return _result("delta_rule", us, peaks, shape, nbytes, 6.0 * n * heads * dk * dv)


def routed_experts(tokens=2048, width=2048, ff=1024, experts=16, top=4, groups=4, keep=3, mma=1, iters=5, peaks=None):
    """Routing, sorting the pairs by expert, both expert products and the weighted sum of ``tokens`` tokens
    (``mma=0``: the CUDA-core products)."""
    from gllm_b200 import ops
    from gllm_b200.ops import moe

    x = (torch.randn(tokens, width, device="cuda") * 0.5).to(torch.bfloat16)
    w_gu = (torch.randn(experts, 2 * ff, width, device="cuda") * width ** -0.5).to(torch.bfloat16)
    w_d = (torch.randn(experts, width, ff, device="cuda") * ff ** -0.5).to(torch.bfloat16)
    logits = torch.randn(tokens, experts, device="cuda")
    correction = torch.zeros(experts, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    tensor_cores = bool(mma) and moe.tensor_cores_take(torch.bfloat16, width, ff)
    if tensor_cores:
        w_gu = torch.stack([ops.interleave_gate_up(w[:ff], w[ff:]) for w in w_gu]).contiguous()

    def fn():
        ids, weights = moe.route(logits, correction, top, groups, keep)
        return moe.apply_experts(x, ids, weights, w_gu, w_d, None, tensor_cores)

    us = _time(fn, iters, flush)
    used = min(experts, tokens * top)
    nbytes = used * 3 * ff * width * 2 + tokens * width * 4 + tokens * top * (ff * 4 + width * 8)
    return _result("routed_experts", us, peaks, dict(tokens=tokens, width=width, ff=ff, experts=experts, top=top), nbytes,
                   6.0 * tokens * top * ff * width)


def differential_attention(tokens=2048, batch=1, context=0, hq=16, hkv=4, dk=64, dv=128, block_size=16, iters=5,
                           peaks=None, mma=1):
    """``batch`` requests of ``tokens`` new tokens over ``context`` cached ones (tokens=1: a decode step): both maps,
    the difference, the per-head norm and the gate."""
    from gllm_b200.ops import differential

    differential.USE_TENSOR_CORES = bool(mma)
    pages_per_req = -(-(context + tokens) // block_size)
    num_pages = batch * pages_per_req + 1
    g = torch.Generator(device="cuda").manual_seed(0)
    pool = torch.randn((num_pages, block_size * hkv * (2 * dk + dv)), generator=g, device="cuda").to(torch.bfloat16)
    table = torch.randperm(num_pages - 1, generator=g, device="cuda").to(torch.int32).view(batch, pages_per_req).contiguous()
    proj = torch.randn(batch * tokens, hq * 2 * dk + hq * dv, device="cuda").to(torch.bfloat16)
    b = _Batch(batch, tokens, context)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    fn = lambda: differential.differential_attention(proj, proj[:, hq * 2 * dk:], pool, table, b.positions, b.token_row,
                                                     hq, hkv, dk, dv, block_size, dk ** -0.5, 30.0, 0.4, 1e-5, 0.7,
                                                     batch=b)
    us = _time(fn, iters, flush)
    flops = 2.0 * 2 * (dk + dv) * hq * batch * (tokens * context + tokens * (tokens + 1) / 2)
    nbytes = batch * (context + tokens) * hkv * (2 * dk + dv) * 2 + proj.numel() * 2 + batch * tokens * hq * dv * 2
    return _result("differential_attention (mma.sync)" if mma else "differential_attention (CUDA cores)", us, peaks,
                   dict(tokens=tokens, batch=batch, context=context, heads=hq, kv_heads=hkv, dk=dk, dv=dv), nbytes, flops)


def step_sized_recurrence(tokens=2048, batch=1, heads=64, dk=128, dv=64, groups=1, norm=0, iters=5, peaks=None):
    """The recurrence of state-space duality (``norm=1``: the gated norm over the whole row behind it instead)."""
    from gllm_b200.ops import stateful

    n, inner = batch * tokens, heads * dv
    xbc = torch.randn(n, inner + 2 * groups * dk, device="cuda").to(torch.bfloat16)
    z = torch.randn(n, inner, device="cuda").to(torch.bfloat16)
    dt = torch.randn(n, heads, device="cuda")
    dt_bias, A, D = torch.zeros(heads, device="cuda"), -torch.rand(heads, device="cuda"), torch.ones(heads, device="cuda")
    w = torch.ones(inner, device="cuda")
    state = torch.zeros(batch + 1, heads, dv, dk, device="cuda")
    b = _Batch(batch, tokens, 0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    gn = groups * dk
    rec = lambda: stateful.matrix_recurrence(stateful.STEP_SIZED, xbc[:, inner + gn:], xbc[:, inner:inner + gn],
                                             xbc[:, :inner], dt, dt_bias, A, 0.0, 1.0, state, None, b.cu_q, b.state_slots,
                                             batch, heads, dk, dv, max_q_len=tokens, heads_per_group=heads // groups)
    if norm:
        y = rec()
        fn = lambda: stateful.gated_group_norm(y, z, w, 1, 1e-5, skip=D, x=xbc[:, :inner], head_width=dv)
        us = _time(fn, iters, flush)
        return _result("gated_group_norm", us, peaks, dict(tokens=tokens, batch=batch, width=inner),
                       n * inner * (4 + 2 + 2 + 2) + inner * 4)
    us = _time(rec, iters, flush)
    nbytes = 2 * batch * heads * dk * dv * 4 + n * (xbc.shape[1] * 2 + heads * 4 + inner * 4)
    return _result("matrix_recurrence (step sizes)", us, peaks, dict(tokens=tokens, batch=batch, heads=heads, dk=dk, dv=dv),
                   nbytes, 4.0 * n * heads * dk * dv)


def add_dyt(rows=2048, hidden=2048, iters=5, peaks=None):
    from gllm_b200 import ops

    resid = torch.randn(rows, hidden, device="cuda")
    branch = torch.randn(rows, hidden, device="cuda").to(torch.bfloat16)
    alpha, w, bias = torch.ones(1, device="cuda"), torch.ones(hidden, device="cuda"), torch.zeros(hidden, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    us = _time(lambda: ops.add_dyt(branch, resid, alpha, w, bias, torch.bfloat16), iters, flush)
    return _result("add_dyt", us, peaks, dict(rows=rows, hidden=hidden), rows * hidden * (4 + 4 + 2 + 2) + hidden * 8)


def ungated_experts(tokens=2048, width=2048, ff=2048, experts=16, top=4, groups=8, keep=4, mma=1, iters=5, peaks=None):
    """Softmax routing, sorting the pairs by expert, both products of experts without a gate (``down(relu(up x)^2)``)
    and the weighted sum of ``tokens`` tokens (``mma=0``: the CUDA-core products)."""
    from gllm_b200.ops import moe

    x = (torch.randn(tokens, width, device="cuda") * 0.5).to(torch.bfloat16)
    w_up = (torch.randn(experts, ff, width, device="cuda") * width ** -0.5).to(torch.bfloat16)
    w_d = (torch.randn(experts, width, ff, device="cuda") * ff ** -0.5).to(torch.bfloat16)
    logits = torch.randn(tokens, experts, device="cuda")
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    tensor_cores = bool(mma) and moe.tensor_cores_take(torch.bfloat16, width, ff, gated=False)

    def fn():
        ids, weights = moe.route(logits, None, top, groups, keep, True, score="softmax", group_score="max",
                                 renormalize_eps=1e-20, scale=2.5)
        return moe.apply_experts(x, ids, weights, w_up, w_d, None, tensor_cores, gated=False)

    us = _time(fn, iters, flush)
    used = min(experts, tokens * top)
    nbytes = used * 2 * ff * width * 2 + tokens * width * 4 + tokens * top * (ff * 6 + width * 8)
    return _result("ungated_experts", us, peaks, dict(tokens=tokens, width=width, ff=ff, experts=experts, top=top), nbytes,
                   4.0 * tokens * top * ff * width)


KERNELS = {
    "differential_attention": differential_attention,
    "step_sized_recurrence": step_sized_recurrence,
    "add_dyt": add_dyt,
    "ungated_experts": ungated_experts,
    "attention_decode": attention_decode,
    "attention_prefill": attention_prefill,
    "linear": linear,
    "linear_f32": linear_f32,
    "decode_step": decode_step,
    "add_rmsnorm": add_rmsnorm,
    "argmax": argmax,
    "sigmoid_attention": sigmoid_attention,
    "latent_attention": latent_attention,
    "head_linear": head_linear,
    "matrix_recurrence": matrix_recurrence,
    "selective_scan": selective_scan,
    "conv_silu": conv_silu,
    "stream_mix_norm": stream_mix_norm,
    "delta_rule": delta_rule,
    "routed_experts": routed_experts,
}


def run(name: str, peaks: dict, overrides: dict) -> dict:
    if name not in KERNELS:
        raise SystemExit(f"unknown kernel {name!r}; known: {sorted(KERNELS)}")
    return KERNELS[name](peaks=peaks, **overrides)
