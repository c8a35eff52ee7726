"""Mifidra on the GPU against the plain implementation: each kernel of its mechanisms alone, each half of the mixer
alone, whole prompts against token by token decoding and portions of every size, mixed batches over a pool so small
that pages and state slots are used again, a key far away and at the edges of pages and key blocks, the first
tokens, long decoding through the decode graphs, sizes of every kind, and greedy generation through the engine."""

import copy
import math
import os

import numpy as np
import pytest
import torch

import plain_mifidra as plain
from replay_helpers import (BF16_TOL_MAX, BF16_TOL_MEAN, FP32_TOL, LENGTHS, compare, mixed_steps, replay, rounded,
                            run_steps, sequences, single_request_steps)
from tiny_mifidra import (MIFIDRA, _left, _moe, _right, decisive_routing, draw_weights, one_layer,
                          write_model)

pytestmark = pytest.mark.gpu

PAGE = {"A": 4, "B": 8, "C": 16, "D": 16}
F = plain.F


def tolerance(dtype):
    return (FP32_TOL, None) if dtype == "float32" else (BF16_TOL_MAX, BF16_TOL_MEAN)


def make(cfg, tmp_path, dtype, seed=7, max_tokens=512, block_size=16, max_live=4, sharp=None, weights=None):
    from gllm_b200.engine.replay import build_runner

    sharp = (1.5 if dtype == "float32" else 1.0) if sharp is None else sharp
    if weights is None:
        weights = decisive_routing(cfg, draw_weights(cfg, seed=seed, sharp=sharp))
    folder = write_model(cfg, weights, str(tmp_path / "model"))
    _, runner = build_runner(folder, dtype, max_tokens, block_size=block_size, max_live=max_live)
    return weights, folder, runner


def steps_of(tokens, cuts, rid="r", first_step=0, end=True):
    """One request fed in portions of the given sizes; every logit is wanted."""
    steps, index, p = [], [], 0
    for i, n in enumerate(cuts):
        last = p + n == len(tokens)
        steps.append({"step": first_step + i, "entries": [{"id": rid, "tokens": tokens[p:p + n], "want": list(range(n))}],
                      "end": [rid] if (last and end) else []})
        index += [(first_step + i, k, rid, p + k) for k in range(n)]
        p += n
    assert p == len(tokens)
    return steps, index


def compare_beside_rounding(results, index, want, moved, tol_max):
    """As ``compare``, for a bfloat16 run of a model in which rounding alone moves some positions' logits by more
    than the general bound (a head whose read-out is next to nothing before it is divided by its root mean square):
    ``moved`` are the plain logits with the sublayers' inputs and results rounded to bfloat16, and a position may
    differ by the general bound or four times what that rounding moved it."""
    scale = max(1.0, max(float(p.abs().max()) for p in want.values()))
    noisy = 0
    for step, row, key, position in index:
        err = float(np.abs(results[step][row].astype(np.float64) - want[key][position].numpy()).max())
        room = 4.0 * float((moved[key][position] - want[key][position]).abs().max())
        noisy += room > tol_max * scale
        assert err <= max(tol_max * scale, room), (step, row, key, position, err, room)
    assert noisy <= len(index) // 10          # the wider bound is the exception


def tokens_of(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# ------------------------------------------------------------------ the kernels of each mechanism alone
def _batch(lengths, starts, slots):
    """The flat batch's index tensors for requests bringing ``lengths`` tokens from positions ``starts``; a token's
    row is its request's state slot."""
    dev = "cuda"
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32, device=dev)
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lengths)]).to(torch.int32).to(dev)
    row = torch.cat([torch.full((n,), s) for s, n in zip(slots, lengths)]).to(torch.int32).to(dev)
    return cu, pos, row


@pytest.mark.parametrize("heads,kv_heads,dk,dv,taps", [(4, 2, 16, 8, 3), (3, 1, 10, 6, 1), (2, 2, 64, 64, 4),
                                                      (1, 1, 20, 12, 2), (6, 3, 32, 40, 3), (2, 1, 128, 32, 4),
                                                      (1, 1, 320, 16, 2), (2, 2, 36, 20, 3), (60, 30, 64, 128, 2), (2, 1, 16, 10, 2),
                                                      (3, 3, 64, 6, 3)])
def test_delta_rule_kernels(heads, kv_heads, dk, dv, taps):
    """The convolution, unit norms, decay and the recurrence over two requests in three steps (a portion each, then a
    portion beside a single token, then a single token each), on state slots that are not the requests' numbers,
    against the plain functions.  The sizes reach every number of key channels per thread the kernel picks by itself
    (few and many blocks, heads of 10 to 320 key channels, single tokens only)."""
    _delta_rule_case(heads, kv_heads, dk, dv, taps)


@pytest.mark.parametrize("channels_per_thread", [4, 8, 16, 32])
def test_delta_rule_every_thread_layout(channels_per_thread, monkeypatch):
    """The same recurrence with 4, 8, 16 and 32 key channels per thread (the kernel reads the choice at every launch)."""
    monkeypatch.setenv("GLLM_B200_DELTA_DPT", str(channels_per_thread))
    _delta_rule_case(2, 1, 64, 48, 3)


def _delta_rule_case(heads, kv_heads, dk, dv, taps):
    from gllm_b200.ops import stateful

    g = torch.Generator().manual_seed(heads * 100 + dk)
    qk_cols, channels = 2 * kv_heads * dk, 2 * kv_heads * dk + heads * dv
    total = {0: 22, 1: 10}
    x = {r: torch.randn(n, channels, generator=g) for r, n in total.items()}
    raw = {r: torch.randn(n, heads * dk, generator=g) * 2 for r, n in total.items()}
    braw = {r: torch.randn(n, heads, generator=g) * 2 for r, n in total.items()}
    conv_w = torch.randn(channels, taps, generator=g) * 0.6
    dt_bias, A_log = torch.randn(heads * dk, generator=g) * 0.5, torch.randn(heads, generator=g) * 0.5
    unit_eps, q_scale = 1e-6, dk ** -0.5

    def plain_request(r):
        T = total[r]
        xc, _ = plain.short_conv(x[r].to(F), conv_w.to(F), torch.zeros(taps - 1, channels, dtype=F))
        q = plain.unit(xc[:, :kv_heads * dk].view(T, kv_heads, dk)) * q_scale
        k = plain.unit(xc[:, kv_heads * dk:qk_cols].view(T, kv_heads, dk))
        rep = heads // kv_heads
        v = xc[:, qk_cols:].view(T, heads, dv)
        sp = torch.nn.functional.softplus(raw[r].to(F) + dt_bias.to(F)).view(T, heads, dk)
        dec = torch.exp(-torch.exp(A_log.to(F))[None, :, None] * sp)
        S = torch.zeros(heads, dk, dv, dtype=F)
        o = plain.delta_rule(q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1), v, dec,
                             torch.sigmoid(braw[r].to(F)), S)
        return o.reshape(T, heads * dv), S

    want = {r: plain_request(r) for r in total}
    slots = 5
    state = torch.full((slots, heads, dv, dk), 7.0, device="cuda")
    conv_state = torch.full((slots, max(taps - 1, 0), channels), 7.0, device="cuda")
    slot_of = {0: 3, 1: 1}
    for s in slot_of.values():                           # a request's slot starts at zero
        state[s] = 0
        conv_state[s] = 0
    got = {r: [] for r in total}
    done = {0: 0, 1: 0}
    for plan in ([(0, 13), (1, 8)], [(1, 1), (0, 8)], [(0, 1), (1, 1)]):
        lengths = [n for _, n in plan]
        cu, pos, row = _batch(lengths, [done[r] for r, _ in plan], [slot_of[r] for r, _ in plan])
        cat = lambda d: torch.cat([d[r][done[r]:done[r] + n] for r, n in plan]).cuda().contiguous()
        ss = torch.tensor([slot_of[r] for r, _ in plan], dtype=torch.int32, device="cuda")
        qk, v, dec, beta = stateful.delta_prep(cat(x), conv_w.cuda(), conv_state, pos, row, cu, ss, len(plan), cat(raw),
                                               dt_bias.cuda(), A_log.cuda(), cat(braw), heads, kv_heads, dk, dv,
                                               unit_eps, q_scale, max_q_len=max(lengths))
        o = stateful.delta_rule(qk, v, dec, beta, state, cu, ss, len(plan), heads, kv_heads, dk, dv,
                                max_q_len=max(lengths))
        at = 0
        for r, n in plan:
            got[r].append(o[at:at + n].double().cpu())
            at += n
            done[r] += n
    for r in total:
        o, S = want[r]
        assert torch.allclose(torch.cat(got[r]), o, rtol=2e-4, atol=2e-5), r
        assert torch.allclose(state[slot_of[r]].double().cpu().transpose(1, 2), S, rtol=2e-4, atol=2e-5), r
    assert float(state[0].min()) == 7.0 and (taps == 1 or float(conv_state[4].min()) == 7.0)   # others: untouched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,inter", [(5, 24), (3, 20), (70, 64)])
def test_activation_with_the_gate_and_up_biases(dtype, rows, inter):
    """``silu(gate + b_g) * (up + b_u)`` in one kernel gives what the bias kernel followed by the activation gives, bit
    for bit, and what the plain formula gives."""
    from gllm_b200 import ops

    g = torch.Generator().manual_seed(rows * inter)
    x = torch.randn(rows, 2 * inter, generator=g).to(dtype).cuda()
    bias = torch.randn(2 * inter, generator=g).cuda()
    fused = ops.silu_mul(x, bias=bias)
    two_steps = ops.silu_mul(ops.add_bias(x.clone(), bias))
    assert torch.equal(fused, two_steps)
    y = (x.double() + bias.double()).cpu()
    want = torch.nn.functional.silu(y[:, :inter]) * y[:, inter:]
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(fused.double().cpu(), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("experts,top,groups,keep", [(16, 6, 4, 2), (8, 2, 4, 2), (6, 3, 1, 1), (4, 1, 4, 2),
                                                      (12, 5, 3, 2), (64, 8, 8, 4), (5, 5, 1, 1)])
def test_router_kernel(experts, top, groups, keep):
    from gllm_b200.ops import moe

    g = torch.Generator().manual_seed(experts + top)
    # the plain routing reports its closest call: the comparison must not rest on fp32 rounding
    z = torch.randn(50, experts, generator=g) * 2
    corr = torch.randn(experts, generator=g) * 0.5 - 0.3                            # choice scores can be negative
    router = {"experts": experts, "top": top}
    if groups > 1:
        router["groups"] = {"count": groups, "keep": keep}
    w = {"m.router": torch.eye(experts, dtype=F), "m.correction": corr.to(F)}
    margins: list = []
    chosen, weights = plain.route(z.to(F), w, "m", router, margins)
    ids, wts = moe.route(z.cuda(), corr.cuda(), top, groups, keep if groups > 1 else 1)
    close = min(margins) < 1e-5 if margins else False
    assert not close, "the test's scores came too close; change the seed"
    for t in range(z.shape[0]):
        a = dict(zip(chosen[t].tolist(), weights[t].tolist()))
        b = dict(zip(ids[t].tolist(), wts[t].tolist()))
        assert set(a) == set(b), (t, a, b)
        assert all(abs(a[e] - b[e]) < 1e-6 for e in a)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,ff,experts,top", [(37, 64, 32, 8, 2), (1, 44, 20, 4, 1), (130, 128, 64, 16, 4),
                                                     (5, 40, 24, 6, 6)])
def test_expert_products(dtype, n, width, ff, experts, top):
    """Sorting the pairs by expert, the two products over tiles of one expert and the weighted sum, against a loop."""
    from gllm_b200.ops import moe

    g = torch.Generator().manual_seed(n)
    rnd = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).float()
    x, wgu, wd = rnd(n, width), rnd(experts, 2 * ff, width) / math.sqrt(width), rnd(experts, width, ff) / math.sqrt(ff)
    shared = rnd(n, width)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    wts = torch.rand(n, top, generator=g)
    want = shared.to(F).clone()
    for t in range(n):
        for e, a in zip(ids[t].tolist(), wts[t].to(F)):
            gu = wgu[e].to(F) @ x[t].to(F)
            h = torch.nn.functional.silu(gu[:ff]) * gu[ff:]
            if dtype == torch.bfloat16:
                h = h.to(torch.bfloat16).to(F)
            want[t] += a * (wd[e].to(F) @ h)
    plan = moe.align(ids.cuda(), experts)
    hidden = moe.expert_product(x.to(dtype).cuda(), top, wgu.to(dtype).cuda(), plan, n * top, gated=True)
    y = moe.expert_product(hidden, 1, wd.to(dtype).cuda(), plan, n * top, gated=False)
    out = moe.combine(y, wts.cuda(), shared.to(dtype).cuda(), dtype).double().cpu()
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    assert float((out - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("n,width,ff,experts,top", [(37, 64, 64, 8, 2), (1, 48, 64, 4, 1), (700, 128, 192, 16, 4),
                                                     (3000, 256, 128, 4, 2), (5, 40, 128, 6, 6)])
def test_expert_products_on_the_tensor_cores(n, width, ff, experts, top):
    """The same through the grouped tcgen05 products: rows copied into the order of the sorted pairs (tiles of 128
    rows of one expert, the last one of an expert partly empty), results looked up per pair; some experts unused."""
    from gllm_b200 import ops
    from gllm_b200.ops import moe

    assert moe.tensor_cores_take(torch.bfloat16, width, ff)
    g = torch.Generator().manual_seed(n)
    rnd = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).float()
    x, wg, wu = rnd(n, width), rnd(experts, ff, width) / math.sqrt(width), rnd(experts, ff, width) / math.sqrt(width)
    wd, shared = rnd(experts, width, ff) / math.sqrt(ff), rnd(n, width)
    usable = max(top, experts - 1)                                # the last expert stays unused where there is room
    ids = torch.stack([torch.randperm(usable, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    wts = torch.rand(n, top, generator=g)
    gate, up = torch.einsum("tw,efw->tef", x.to(F), wg.to(F)), torch.einsum("tw,efw->tef", x.to(F), wu.to(F))
    hidden = (torch.nn.functional.silu(gate) * up).to(torch.bfloat16).to(F)
    each = torch.einsum("tef,ewf->tew", hidden, wd.to(F))
    want = shared.to(F) + (each.gather(1, ids.long()[:, :, None].expand(n, top, width)) * wts.to(F)[:, :, None]).sum(1)
    stacked = torch.stack([ops.interleave_gate_up(wg[e], wu[e]) for e in range(experts)]).to(torch.bfloat16).cuda()
    out = moe.apply_experts(x.to(torch.bfloat16).cuda(), ids.cuda(), wts.cuda(), stacked, wd.to(torch.bfloat16).cuda(),
                            shared.to(torch.bfloat16).cuda(), True).double().cpu()
    assert float((out - want).abs().max()) <= 2e-2 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,stored,dims,scaled", [(4, 2, 32, 32, 32, True), (2, 1, 24, 32, 16, False),
                                                                   (3, 3, 12, 32, 0, False), (1, 1, 36, 64, 36, True),
                                                                   (2, 2, 128, 128, 64, True)])
def test_rotation_then_unit_norm_and_store(dtype, heads, kv_heads, dim, stored, dims, scaled):
    """Neighbouring pairs turn, sine and cosine carry the multiplier, the head is divided by its root mean square over
    ``dim`` (heads are stored ``stored`` wide, zeros behind), keys and values land in their pages."""
    from gllm_b200 import ops

    rot = {"base": 500.0, "dims": dims}
    if scaled:
        rot["scaling"] = {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}
    g = torch.Generator().manual_seed(dim)
    n, eps, block = 19, 1e-5, 4
    total = heads + 2 * kv_heads
    x = torch.zeros(n, total, stored)
    x[:, :, :dim] = torch.randn(n, total, dim, generator=g)
    x = x.to(dtype).float()
    pos = torch.cat([torch.randint(0, 100, (n - 6,), generator=g), torch.randint(100, 3000, (6,), generator=g)])
    f, mult = plain.yarn_frequencies(rot) if dims else (None, 1.0)
    qk = plain.rms(plain.rotate_pairs(x[:, :heads + kv_heads, :dim].to(F), pos, rot), eps)
    pages = torch.zeros(8, 2, kv_heads, block, stored, dtype=dtype, device="cuda")
    slots = torch.randperm(8 * block, generator=g)[:n].to(torch.int32)
    out = ops.rope_norm_store(x.view(n, -1).to(dtype).cuda(), pos.to(torch.int32).cuda(),
                              f.float().cuda() if dims else None, mult, slots.cuda(), pages, heads, kv_heads, stored,
                              dims, True, dim, eps).view(n, total, stored).double().cpu()
    # an fp32 angle p * f is rounded by up to p * 2^-24: far positions get that much more room
    tol = (2e-5 + pos.double() * 2.0 ** -23 if dtype == torch.float32 else torch.full((n,), 2e-2, dtype=F))
    err = (out[:, :heads + kv_heads, :dim] - qk).abs().amax((1, 2))
    assert bool((err <= tol * float(qk.abs().max())).all()), (err / tol).max()
    assert float(out[:, :, dim:].abs().max()) == 0.0 if stored > dim else True
    assert torch.equal(out[:, heads + kv_heads:], x[:, heads + kv_heads:].double())          # values pass unchanged
    stored_pages = pages.double().cpu()
    for t in range(n):
        p, o = divmod(int(slots[t]), block)
        assert torch.equal(stored_pages[p, 0, :, o], out[t, heads:heads + kv_heads])
        assert torch.equal(stored_pages[p, 1, :, o], out[t, heads + kv_heads:])


# ------------------------------------------------------------------ the model through the step function
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["left", "right", "both", "dense", "routed", "routed_plain", "repeated"])
def test_each_mechanism_alone(kind, dtype, tmp_path):
    """One layer with one half of the mixer switched off by its scale, with each feed-forward, and one layer run
    three times: a portion, then single tokens; then the whole prompt at once."""
    if kind == "left":
        cfg = one_layer(_left(4, 2, 24, 40, 0.3, 16, base=300.0, scaling=(4.0, 32, 8.0, 1.0)), left_scale=1.3,
                        right_scale=0.0)
    elif kind == "right":
        cfg = one_layer(right=_right(4, 2, 16, 24, 3), left_scale=0.0, right_scale=0.7)
    elif kind == "dense":
        cfg = one_layer(mlp={"kind": "dense", "ff": 72})
    elif kind == "routed":
        cfg = one_layer(mlp=_moe(24, 12, 3, (4, 2), 40))
    elif kind == "routed_plain":
        cfg = one_layer(mlp=_moe(40, 5, 2))
    else:
        cfg = one_layer(left_scale=0.6, right_scale=0.9)
        if kind == "repeated":
            cfg["loop"] = {"start": 0, "stop": 1, "times": 3}
    weights, _, runner = make(cfg, tmp_path, dtype)
    toks = tokens_of(cfg, 75, 2)
    want = {"r": plain.forward(cfg, weights, toks)}
    steps, index = steps_of(toks, [40] + [1] * 35)
    compare(run_steps(runner, steps), index, want, *tolerance(dtype))
    steps, index = steps_of(toks, [75])
    compare(run_steps(runner, steps), index, want, *tolerance(dtype))


def test_residual_after_every_layer_run(tmp_path):
    """The fp32 residual stream after every run of a layer (a repeated layer counts each time) against the plain
    one: the add of the embedding output before a further pass and both post-norms are in it."""
    from gllm_b200 import ops

    cfg = MIFIDRA["A"]
    weights, _, runner = make(cfg, tmp_path, "float32")
    seen = []
    for block in runner.model.layers:
        inner = block.forward

        def wrapped(branch, resid, ctx, cache, inner=inner):
            out, resid = inner(branch, resid, ctx, cache)
            x = resid.double().cpu()
            if isinstance(out, ops.Pending) and out.value is not None:
                v = ops.as_tensor(out.value).double().cpu()
                x = x + plain.rms_norm(v, out.post_weight.double().cpu(), out.post_eps)
            seen.append(x)
            return out, resid

        block.forward = wrapped
    toks = tokens_of(cfg, 11, 3)
    want: list = []
    plain.forward(cfg, weights, toks, layers_out=want)
    runner.run(steps_entries(toks))
    assert len(seen) == len(want) == 8
    for i, (a, b) in enumerate(zip(seen, want)):
        assert float((a - b).abs().max()) <= 1e-4 * max(1.0, float(b.abs().max())), i


def steps_entries(toks, rid="r"):
    from gllm_b200.engine.step import StepEntry

    return [StepEntry(rid, list(toks), [len(toks) - 1])]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_all_cuts_and_mixed_batches(name, dtype, tmp_path):
    from gllm_b200.engine.replay import build_runner

    cfg = MIFIDRA[name]
    weights, folder, runner = make(cfg, tmp_path, dtype, max_tokens=rounded(max(LENGTHS.values())),
                                   block_size=PAGE[name])
    seqs = sequences(cfg["vocab"], seed=5)
    want = {k: plain.forward(cfg, weights, v) for k, v in seqs.items()}
    check = lambda results, index: compare(results, index, want, *tolerance(dtype))
    if name == "B" and dtype == "bfloat16":
        # narrow heads and few columns: at some early positions rounding alone moves the logits by a tenth
        moved = {k: plain.forward(cfg, weights, v, stored=torch.bfloat16) for k, v in seqs.items()}
        check = lambda results, index: compare_beside_rounding(results, index, want, moved, BF16_TOL_MAX)
    steps, index = single_request_steps(seqs)
    check(run_steps(runner, steps), index)
    runner.cache.check_invariants()
    # four live requests at most over 448 tokens of pages: pages and slots are used again
    _, small = build_runner(folder, dtype, 448, block_size=PAGE[name])
    steps, index = mixed_steps(seqs, max_tokens=448, seed=9)
    check(run_steps(small, steps), index)
    small.cache.check_invariants()
    assert all(g.allocator.total_reused > 0 for g in small.cache.groups)


def test_replay_through_the_command(tmp_path):
    cfg = MIFIDRA["A"]
    weights = decisive_routing(cfg, draw_weights(cfg, seed=7, sharp=1.5))
    folder = write_model(cfg, weights, str(tmp_path / "model"))
    seqs = sequences(cfg["vocab"], seed=6)
    want = {k: plain.forward(cfg, weights, v) for k, v in seqs.items()}
    steps, index = mixed_steps(seqs, max_tokens=448, seed=3)
    results = replay(folder, "float32", steps, str(tmp_path / "out"), max_tokens=448, vocab=cfg["vocab"])
    compare(results, index, want, FP32_TOL)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_at_every_edge(dtype, tmp_path):
    """Portions that end just before, at and just after the edges the kernels have: pages of 16, the attention's
    blocks of keys, the convolution's taps, the tiles of the expert products."""
    cfg = MIFIDRA["C"]
    weights, _, runner = make(cfg, tmp_path, dtype, max_tokens=256)
    toks = tokens_of(cfg, 200, 8)
    want = {"r": plain.forward(cfg, weights, toks)}
    for cuts in ([7, 1, 1, 7, 15, 2, 31, 1, 33, 16, 17, 9, 8, 2, 2, 3, 45],
                 [2, 2, 2, 2, 8, 16, 32, 64, 63, 9],
                 [1, 1, 1, 1, 1, 3, 24, 31, 33, 104]):
        steps, index = steps_of(toks, cuts)
        compare(run_steps(runner, steps), index, want, *tolerance(dtype))


def far_key_model(dim=32, vdim=32, stored_heads=(2, 1)):
    """The attention half alone, built so that one far key decides the last token's logits: token 1's key and
    token 2's query point the same way (every other query and key is orthogonal to that direction), the scale is
    large, so the last token's softmax puts nearly all its weight on that one key among hundreds."""
    heads, kv_heads = stored_heads
    cfg = one_layer(_left(heads, kv_heads, dim, vdim, 0.5, 0), width=48, left_scale=1.0, right_scale=0.0)
    w = draw_weights(cfg, seed=11)
    W = cfg["width"]
    ca, cb = W - 1, W - 2                      # marker columns: only tokens 1 and 2 have something there
    w["embed"][:, [ca, cb]] = 0.0
    w["embed"][1, ca] = 4.0
    w["embed"][2, cb] = 4.0
    for name in ("l0.mix.left.q", "l0.mix.left.k"):
        w[name][:, [ca, cb]] = 0.0
    # after the unit norm a head has root mean square 1: the marker's direction dominates its own head entirely
    w["l0.mix.left.k"][:dim, ca] = 4.0
    w["l0.mix.left.q"][:dim, cb] = 4.0
    w["l0.mix.left.q"][dim:2 * dim, cb] = 4.0 if heads > 1 else 0.0
    w["l0.mix.left.v"] *= 3.0
    w["final.norm"][[ca, cb]] = 0.0
    return cfg, {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim,vdim", [(32, 32), (24, 40)])
def test_a_far_key_at_page_and_block_edges(dim, vdim, dtype, tmp_path):
    from gllm_b200.engine.replay import build_runner

    cfg, weights = far_key_model(dim, vdim)
    folder = write_model(cfg, weights, str(tmp_path / "model"))
    _, runner = build_runner(folder, dtype, 1024, block_size=16)
    g = torch.Generator().manual_seed(5)
    n = 600
    tol_max, _ = tolerance(dtype)
    for far in (0, 15, 16, 17, 31, 32, 33, 63, 64, 127, 128, 255, 256, 511):
        toks = torch.randint(3, cfg["vocab"], (n,), generator=g).tolist()
        toks[far], toks[-1] = 1, 2
        want = plain.forward(cfg, weights, toks)
        without = list(toks)
        without[far] = 3
        blind = plain.forward(cfg, weights, without)
        scale = max(1.0, float(want.abs().max()))
        # the test is sharp: losing that one key moves the last logits by far more than the tolerance
        assert float((want[-1] - blind[-1]).abs().max()) > (20 if dtype == "float32" else 4) * tol_max * scale
        for cuts in ([n], [n - 1, 1], [far + 1, n - far - 3, 2] if far + 3 < n else [n]):
            steps, index = steps_of(toks, cuts)
            compare(run_steps(runner, steps), [i for i in index if i[3] >= n - 2], {"r": want}, tol_max, None)


def far_write_model():
    """The delta rule half alone, built so that what ONE far token wrote decides the last token's logits: key
    channel 0 is written only by token 1 (and, through the convolution's older tap, by its successor) and read
    only by token 2; the decays are near one.  The head's read-out at the last token is then that far value,
    decayed, and dividing it by its root mean square makes its direction what counts."""
    cfg = one_layer(right=_right(2, 1, 16, 16, 2), width=48, left_scale=0.0, right_scale=1.0)
    w = draw_weights(cfg, seed=17)
    W = cfg["width"]
    ca, cb = W - 1, W - 2                      # marker columns: only tokens 1 and 2 have something there
    w["embed"][:, [ca, cb]] = 0.0
    w["embed"][1, ca] = 4.0
    w["embed"][2, cb] = 4.0
    for name in ("l0.mix.right.q", "l0.mix.right.k"):
        w[name][:, [ca, cb]] = 0.0
        w[name][0, :] = 0.0                    # channel 0 reads the markers only
    w["l0.mix.right.k"][0, ca] = 6.0
    w["l0.mix.right.q"][0, cb] = 6.0
    w["l0.mix.right.q.conv"][0] = torch.tensor([0.0, 1.0])
    w["l0.mix.right.k.conv"][0] = torch.tensor([0.5, 1.0])
    w["l0.mix.right.A_log"][:] = -6.0          # exp(-exp(-6) softplus(..)): about 0.998 a token
    w["l0.mix.right.b"][:, ca] = 2.0           # token 1 writes with beta near one
    w["final.norm"][[ca, cb]] = 0.0
    return cfg, {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_write_far_back_is_still_read(dtype, tmp_path):
    """What a token wrote into the state hundreds of tokens ago decides the last logits: in a whole prompt, across
    portions whose edges fall right behind the write, and with the last tokens decoded alone."""
    cfg, w = far_write_model()
    _, _, runner = make(cfg, tmp_path, dtype, weights=w, max_tokens=512)
    g = torch.Generator().manual_seed(21)
    n = 400
    tol_max, _ = tolerance(dtype)
    for far in (0, 1, 15, 16, 17, 200, 383):
        toks = torch.randint(3, cfg["vocab"], (n,), generator=g).tolist()
        toks[far], toks[-1] = 1, 2
        want = plain.forward(cfg, w, toks)
        without = list(toks)
        without[far] = 3
        scale = max(1.0, float(want.abs().max()))
        assert float((want[-1] - plain.forward(cfg, w, without)[-1]).abs().max()) > (
            20 if dtype == "float32" else 3) * tol_max * scale
        for cuts in ([n], [far + 1, n - far - 3, 2], [n - 17] + [1] * 17):
            steps, index = steps_of(toks, cuts)
            compare(run_steps(runner, steps), [i for i in index if i[3] >= n - 2], {"r": want}, tol_max, None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(dtype, tmp_path):
    """Prompts of one, two and three tokens, then hundreds of tokens decoded one by one (replays of the decode
    graph): state that is lost, doubled or started wrong shows at once or adds up."""
    cfg = MIFIDRA["C"]
    weights, _, runner = make(cfg, tmp_path, dtype, max_tokens=512)
    g = torch.Generator().manual_seed(12)
    for first in (1, 2, 3):
        n = first + (330 if first == 2 else 20)
        toks = torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
        want = {"r": plain.forward(cfg, weights, toks)}
        steps, index = steps_of(toks, [first] + [1] * (n - first))
        compare(run_steps(runner, steps), index, want, *tolerance(dtype))
    assert runner.graph_replays > 300


def test_a_slot_and_its_pages_used_again_start_clean(tmp_path):
    """One state slot and a pool of four pages: the second request gets the first one's slot and pages."""
    cfg = MIFIDRA["A"]
    weights, _, runner = make(cfg, tmp_path, "float32", max_tokens=64, max_live=1)
    g = torch.Generator().manual_seed(13)
    a = torch.randint(0, cfg["vocab"], (60,), generator=g).tolist()
    b = torch.randint(0, cfg["vocab"], (50,), generator=g).tolist()
    for rid, toks, cuts in (("a", a, [33, 20, 7]), ("b", b, [3, 40] + [1] * 7), ("c", a, [60])):
        steps, index = steps_of(toks, cuts, rid=rid)
        compare(run_steps(runner, steps), index, {rid: plain.forward(cfg, weights, toks)}, FP32_TOL)
    assert runner.cache.groups[0].allocator.total_reused > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_greedy_generation_through_the_entry_point(name, dtype, tmp_path):
    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine

    cfg = MIFIDRA[name]
    weights = decisive_routing(cfg, draw_weights(cfg, seed=21))
    folder = write_model(cfg, weights, str(tmp_path / "m"))
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (1, 7, 16, 23, 40)]
    # few pages, small portions: chunked prefill, continuous batching and preemption happen
    params = GeneratorParams(block_size=8, max_batch_size=3, max_seq_len=64, num_blocks=10, model_dtype=dtype,
                             max_num_batched_tokens=24, prefill_chunk=8)
    engine = LLMEngine(folder, params, device="cuda:0")
    reqs = [GenerationRequest(prompt_token_ids=p, max_new_tokens=12, temperature=0.0, ignore_eos=True) for p in prompts]
    results = engine.generate(reqs)
    slack = 1e-5 if dtype == "float32" else 0.05
    for p, r in zip(prompts, results):
        assert len(r.token_ids) == 12 and r.finish_reason == "length"
        tokens = list(p)
        for t in r.token_ids:
            logits = plain.forward(cfg, weights, tokens)[-1]
            best = int(logits.argmax())
            if t != best:
                assert float(logits[best] - logits[t]) <= slack * float(logits.abs().max()), (len(tokens), t, best)
            tokens.append(t)
    engine.cache.check_invariants()
    assert not engine.scheduler.has_work
    if name == "A":
        assert engine.counters["preemptions"] >= 1
    if dtype == "float32":
        for req, r in zip(reqs, results):
            assert engine.generate([req])[0].token_ids == r.token_ids


def test_random_weights_mode_writes_a_model_that_runs(tmp_path):
    from gllm_b200.config import load_config
    from gllm_b200.engine.replay import build_runner
    from gllm_b200.weights import write_random_model

    cfg = copy.deepcopy(MIFIDRA["C"])
    for layer in cfg["layers"]:              # sizes that only a checkpoint's tensors give are named for this mode
        layer["mixer"]["right"].update(decay_rank=6, gate_rank=12)
    folder = write_random_model(str(tmp_path / "m"), load_config(cfg), seed=3)
    assert os.path.isfile(os.path.join(folder, "model.safetensors"))
    _, runner = build_runner(folder, "bfloat16", 128)
    steps, _ = steps_of(list(range(40)), [30, 1, 9])
    out = run_steps(runner, steps)
    assert all(np.isfinite(v).all() for v in out.values())
