"""Sazisun on the GPU against the plain implementation: each kernel of its mechanisms alone, each mechanism alone in
a model of one layer, whole prompts against token by token decoding and portions of every size, mixed batches over a
pool so small that pages and state slots are used again, a key far away and at the edges of pages and key blocks,
the first tokens, long decoding through the decode graphs, sizes of every kind, layers that read another layer's
keys, and greedy generation through the engine."""

import copy

import numpy as np
import pytest
import torch

import plain_sazisun as plain
from replay_helpers import (BF16_TOL_MAX, BF16_TOL_MEAN, FP32_TOL, LENGTHS, compare, mixed_steps, replay, rounded,
                            run_steps, sequences, single_request_steps)
from tiny_sazisun import SAZISUN, _att, _dense, _moe, _ssd, decisive_routing, draw_weights, one_layer, write_model

pytestmark = pytest.mark.gpu

PAGE = {"A": 4, "B": 8, "C": 16}
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


def _batch(lengths, starts, slots):
    """The flat batch's index tensors for requests bringing ``lengths`` tokens from positions ``starts``; a token's
    row is its request's state slot."""
    dev = "cuda"
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32, device=dev)
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lengths)]).to(torch.int32).to(dev)
    row = torch.cat([torch.full((n,), s) for s, n in zip(slots, lengths)]).to(torch.int32).to(dev)
    return cu, pos, row


# ------------------------------------------------------------------ the kernels of each mechanism alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width", [(5, 64), (3, 50), (70, 1024), (1, 7)])
def test_the_norm_without_a_statistic(dtype, rows, width):
    """``tanh(alpha x) w + b`` with the residual add: a branch given as a tensor, as unsummed splits, and none; only
    some rows (the residual then stays as it is)."""
    from gllm_b200 import ops

    g = torch.Generator().manual_seed(rows * width)
    resid = torch.randn(rows, width, generator=g) * 3
    branch = torch.randn(rows, width, generator=g).to(dtype)
    w, b = torch.randn(width, generator=g), torch.randn(width, generator=g) * 0.2
    alpha = torch.tensor([0.7])
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    want = torch.tanh(0.7 * (resid.double() + branch.double())) * w.double() + b.double()
    r = resid.cuda()
    got = ops.add_dyt(branch.cuda(), r, alpha.cuda(), w.cuda(), b.cuda(), dtype)
    assert torch.allclose(got.double().cpu(), want, atol=tol * 3, rtol=tol)
    assert torch.allclose(r.cpu(), resid + branch.float(), atol=1e-6)
    # unsummed splits of a product: added in ascending order, rounded as the product would have rounded them
    parts = torch.randn(3, rows, width, generator=g)
    summed = (parts[0] + parts[1] + parts[2]).to(dtype).float()
    r = resid.cuda()
    got = ops.add_dyt(ops.SplitSum(parts.cuda(), dtype), r, alpha.cuda(), w.cuda(), b.cuda(), dtype)
    want = torch.tanh(0.7 * (resid.double() + summed.double())) * w.double() + b.double()
    assert torch.allclose(got.double().cpu(), want, atol=tol * 3, rtol=tol)
    # no branch, chosen rows: the residual is not written
    pick = torch.tensor([rows - 1, 0], dtype=torch.int32)
    r = resid.cuda()
    got = ops.add_dyt(None, r, alpha.cuda(), w.cuda(), None, dtype, rows=pick.cuda())
    want = (torch.tanh(0.7 * resid.double()) * w.double())[pick.long()]
    assert torch.allclose(got.double().cpu(), want, atol=tol * 3, rtol=tol) and torch.equal(r.cpu(), resid)


@pytest.mark.parametrize("heads,vdim,state,groups,taps,norm_groups", [
    (4, 16, 16, 2, 4, 2), (3, 10, 12, 1, 2, 1), (2, 24, 8, 2, 1, 4), (8, 64, 128, 1, 4, 8), (2, 6, 160, 2, 3, 3),
    (6, 32, 64, 6, 2, 1), (1, 40, 20, 1, 4, 5), (2, 8, 6, 1, 2, 2), (5, 12, 33, 5, 3, 1), (2, 16, 300, 2, 2, 1)])
def test_step_sized_recurrence_kernels(heads, vdim, state, groups, taps, norm_groups):
    """The convolution with its state, the recurrence with one step size per head and token (heads sharing their
    input and read-out projections in groups) and the gated norm over groups of columns, for two requests in three
    steps (a portion each, then a portion beside a single token, then a single token each), on state slots that are
    not the requests' numbers, against the plain functions."""
    from gllm_b200.ops import stateful

    g = torch.Generator().manual_seed(heads * 100 + state)
    inner, gn = heads * vdim, groups * state
    channels = inner + 2 * gn
    total = {0: 22, 1: 10}
    z = {r: torch.randn(n, inner, generator=g) for r, n in total.items()}
    raw = {r: torch.randn(n, channels, generator=g) for r, n in total.items()}
    dt_raw = {r: torch.randn(n, heads, generator=g) * 2 for r, n in total.items()}
    conv_w, conv_b = torch.randn(channels, taps, generator=g) * 0.6, torch.randn(channels, generator=g) * 0.3
    dt_bias, A_log = torch.randn(heads, generator=g) * 0.5, torch.randn(heads, generator=g) * 0.5
    D, norm_w, eps = torch.randn(heads, generator=g), 1 + torch.randn(inner, generator=g) * 0.2, 1e-5

    def plain_request(r):
        T = total[r]
        xbc = plain.silu(plain.causal_conv(raw[r].to(F), conv_w.to(F), conv_b.to(F)))
        x = xbc[:, :inner].view(T, heads, vdim)
        B, C = xbc[:, inner:inner + gn].view(T, groups, state), xbc[:, inner + gn:].view(T, groups, state)
        dt = plain.softplus(dt_raw[r].to(F) + dt_bias.to(F))
        y = plain.ssd_scan(x, B, C, dt, A_log.to(F), D.to(F), heads // groups).reshape(T, inner)
        y = (y * plain.silu(z[r].to(F))).view(T, norm_groups, -1)
        y = y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)
        return y.reshape(T, inner) * norm_w.to(F)

    want = {r: plain_request(r) for r in total}
    slots = 5
    state_t = torch.full((slots, heads, vdim, state), 7.0, device="cuda")
    conv_state = torch.full((slots, max(taps - 1, 0), channels), 7.0, device="cuda")
    slot_of = {0: 3, 1: 1}
    for s in slot_of.values():                           # a request's slot starts at zero
        state_t[s] = 0
        conv_state[s] = 0
    A = (-torch.exp(A_log)).cuda()
    done = {0: 0, 1: 0}
    got = {r: [] for r in total}
    for plan in ([(0, 13), (1, 8)], [(1, 1), (0, 8)], [(0, 1), (1, 1)]):
        lengths = [n for _, n in plan]
        cu, pos, row = _batch(lengths, [done[r] for r, _ in plan], [slot_of[r] for r, _ in plan])
        slots_t = torch.tensor([slot_of[r] for r, _ in plan], dtype=torch.int32, device="cuda")
        cat = lambda d: torch.cat([d[r][done[r]:done[r] + n] for r, n in plan]).cuda()
        # the convolution's inputs as a slice of wider rows, as the mixer hands them over
        wide = torch.cat([cat(z), cat(raw)], 1).contiguous()
        rawc = wide[:, inner:]
        xbc = stateful.conv_silu(rawc, conv_w.cuda(), conv_b.cuda(), conv_state, pos, row)
        stateful.conv_state_advance(rawc, conv_state, cu, slots_t, len(plan))
        y = stateful.matrix_recurrence(stateful.STEP_SIZED, xbc[:, inner + gn:], xbc[:, inner:inner + gn], xbc[:, :inner],
                                       cat(dt_raw), dt_bias.cuda(), A, 0.0, 1.0, state_t, None, cu, slots_t, len(plan),
                                       heads, state, vdim, max_q_len=max(lengths), heads_per_group=heads // groups)
        out = stateful.gated_group_norm(y, wide[:, :inner], norm_w.cuda(), norm_groups, eps, skip=D.cuda(),
                                        x=xbc[:, :inner], head_width=vdim)
        at = 0
        for r, n in plan:
            got[r].append(out[at:at + n].double().cpu())
            at += n
            done[r] += n
    for r in total:
        g_all = torch.cat(got[r])
        assert g_all.shape[0] == total[r]
        assert torch.allclose(g_all, want[r], atol=2e-4, rtol=2e-4), (r, float((g_all - want[r]).abs().max()))
    assert float(state_t[0].min()) == 7.0 and float(conv_state[4].min() if taps > 1 else 7.0) == 7.0   # others' slots


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,dims,page", [(4, 2, 16, 24, 8, 4), (3, 1, 10, 6, 10, 8),
                                                              (2, 2, 64, 64, 32, 16), (1, 1, 12, 20, 0, 16),
                                                              (6, 3, 40, 72, 20, 16), (2, 1, 256, 256, 64, 32)])
def test_differential_attention_kernels(heads, kv_heads, dim, vdim, dims, page):
    """Rotation, the store into shuffled pages and the attention of two requests fed in portions and single tokens,
    against the plain functions.  One early key is made to stand out in the first map only (its score is far above
    the cap's linear range for every later query), others sit right at page borders; the scores spread beyond the
    cap."""
    from gllm_b200.ops import differential

    g = torch.Generator().manual_seed(heads * 1000 + dim)
    m = _att(heads, kv_heads, dim, vdim, 0.3, dims, softcap=6.0, diff=0.35, base=300.0,
             scaling=(4.0, 1.0, 4.0, 32) if dims else None)
    lam, eps = 0.55, 1e-5
    total = {0: 150, 1: 41}
    qw, kw, gw = heads * 2 * dim, kv_heads * 2 * dim, heads * vdim
    proj = {r: torch.randn(n, qw + kw + kv_heads * vdim + gw, generator=g) for r, n in total.items()}
    far = 3                                               # the key that stands out in map 1 of every key head
    for kv in range(kv_heads):
        proj[0][far, qw + kv * 2 * dim + dims: qw + kv * 2 * dim + dim] *= 6.0
    pages_per = {r: -(-n // page) for r, n in total.items()}
    n_pages = sum(pages_per.values()) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((4, max(pages_per.values())), -1, dtype=torch.int32)
    slot_of = {0: 2, 1: 0}
    for r in total:
        for i in range(pages_per[r]):
            table[slot_of[r], i] = order.pop()
    inv_freq = plain.scaled_frequencies(m["rot"]).to(torch.float32).cuda() if dims else None

    def plain_rows(rows):
        T = rows.shape[0]
        x, p = rows.to(F), torch.arange(T)
        q = plain.rotate_pairs(x[:, :qw].reshape(T, heads * 2, dim), p, m["rot"]).view(T, heads, 2, dim)
        k = plain.rotate_pairs(x[:, qw:qw + kw].reshape(T, kv_heads * 2, dim), p, m["rot"]).view(T, kv_heads, 2, dim)
        v = x[:, qw + kw: qw + kw + kv_heads * vdim].view(T, kv_heads, vdim)
        return plain.attend(q, k, v, p, p, m, lam, eps, gate=x[:, -gw:])

    want = {r: plain_rows(proj[r]) for r in total}
    cache = torch.zeros(n_pages, page * kv_heads * (2 * dim + vdim), device="cuda")
    done = {0: 0, 1: 0}
    got = {r: [] for r in total}
    plans = [[(0, 37), (1, 9)], [(1, 1), (0, 2)], [(0, 1), (1, 1)], [(0, 64), (1, 30)], [(0, 46)]]
    for plan in plans:
        lengths = [n for _, n in plan]
        _, pos, row = _batch(lengths, [done[r] for r, _ in plan], [slot_of[r] for r, _ in plan])
        x = torch.cat([proj[r][done[r]:done[r] + n] for r, n in plan]).cuda()
        slot_map = torch.cat([torch.tensor([int(table[slot_of[r], t // page]) * page + t % page
                                            for t in range(done[r], done[r] + n)]) for r, n in plan])
        differential.diff_rope_store(x, pos, inv_freq, dims, True, slot_map.to(torch.int32).cuda(), cache, heads,
                                     kv_heads, dim, vdim, True, page)
        out = differential.differential_attention(x, x[:, -gw:], cache, table.cuda(), pos, row, heads, kv_heads, dim,
                                                  vdim, page, m["scale"], m["softcap"], lam, eps, 1.0 - m["diff"])
        at = 0
        for r, n in plan:
            got[r].append(out[at:at + n].double().cpu())
            at += n
            done[r] += n
    for r in total:
        g_all = torch.cat(got[r])
        assert done[r] == total[r]
        assert torch.allclose(g_all, want[r], atol=3e-4, rtol=3e-4), (r, float((g_all - want[r]).abs().max()))
    if dims < dim:
        # the key that stands out does carry weight far away: without it the last rows come out differently
        muted = proj[0].clone()
        muted[far, qw:qw + kw] = 0
        assert float((want[0][-20:] - plain_rows(muted)[-20:]).abs().max()) > 0.05


class _Step:
    """What the tensor-core attention reads of a step: per-request lengths and slots, and the step's scratch."""

    def __init__(self, lengths, starts, slots):
        from gllm_b200.engine.step import Workspace

        dev = "cuda"
        self.cu_q = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32, device=dev)
        self.context_lens = torch.tensor(starts, dtype=torch.int32, device=dev)
        self.state_slots = torch.tensor(slots, dtype=torch.int32, device=dev)
        self.num_requests, self.max_q_len = len(lengths), max(lengths)
        self.max_seq_len = max(s + n for s, n in zip(starts, lengths))
        self.workspace = Workspace(dev)


@pytest.mark.parametrize("heads,kv_heads,dim,vdim,dims,page", [(4, 2, 64, 64, 32, 16), (3, 1, 32, 96, 32, 8),
                                                              (2, 2, 128, 128, 64, 16), (8, 2, 64, 128, 16, 32),
                                                              (5, 5, 32, 32, 0, 16)])
def test_differential_attention_on_the_tensor_cores(heads, kv_heads, dim, vdim, dims, page):
    """The bf16 kernel pair (tiles of 64 keys, two maps as two sets of CTAs, the combining kernel) against the plain
    functions on the same bf16 inputs: two requests in portions and single tokens over shuffled pages, then single
    tokens over a context long enough that every request's keys are cut into ranges that are merged afterwards."""
    from gllm_b200.ops import differential

    g = torch.Generator().manual_seed(heads * 1000 + dim)
    m = _att(heads, kv_heads, dim, vdim, 0.5 * dim ** -0.5, dims, softcap=5.0, diff=0.35, base=300.0,
             scaling=(4.0, 1.0, 4.0, 32) if dims else None)
    lam, eps = 0.55, 1e-5
    total = {0: 700, 1: 150}
    qw, kw, gw = heads * 2 * dim, kv_heads * 2 * dim, heads * vdim
    proj = {r: (torch.randn(n, qw + kw + kv_heads * vdim + gw, generator=g) * 1.5).to(torch.bfloat16)
            for r, n in total.items()}
    pages_per = {r: -(-n // page) for r, n in total.items()}
    n_pages = sum(pages_per.values()) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.full((4, max(pages_per.values())), -1, dtype=torch.int32)
    slot_of = {0: 2, 1: 0}
    for r in total:
        for i in range(pages_per[r]):
            table[slot_of[r], i] = order.pop()
    inv_freq = plain.scaled_frequencies(m["rot"]).to(torch.float32).cuda() if dims else None

    def plain_rows(rows):
        T = rows.shape[0]
        x, p = rows.to(F), torch.arange(T)
        bf = lambda t: t.to(torch.bfloat16).to(F)                       # what the kernel reads back is bf16
        q = bf(plain.rotate_pairs(x[:, :qw].reshape(T, heads * 2, dim), p, m["rot"])).view(T, heads, 2, dim)
        k = bf(plain.rotate_pairs(x[:, qw:qw + kw].reshape(T, kv_heads * 2, dim), p, m["rot"])).view(T, kv_heads, 2, dim)
        v = x[:, qw + kw: qw + kw + kv_heads * vdim].view(T, kv_heads, vdim)
        return plain.attend(q, k, v, p, p, m, lam, eps, gate=x[:, -gw:])

    want = {r: plain_rows(proj[r]) for r in total}
    cache = torch.zeros(n_pages, page * kv_heads * (2 * dim + vdim), device="cuda", dtype=torch.bfloat16)
    done = {0: 0, 1: 0}
    got = {r: [] for r in total}
    plans = [[(0, 200), (1, 70)], [(1, 1), (0, 2)], [(0, 1), (1, 1)], [(0, 129), (1, 63)], [(0, 360)]]
    plans += [[(0, 1), (1, 1)]] * 6 + [[(0, 1)]] + [[(1, 9), (0, 1)]]
    split_steps = 0
    for plan in plans:
        lengths, starts = [n for _, n in plan], [done[r] for r, _ in plan]
        _, pos, row = _batch(lengths, starts, [slot_of[r] for r, _ in plan])
        step = _Step(lengths, starts, [slot_of[r] for r, _ in plan])
        x = torch.cat([proj[r][done[r]:done[r] + n] for r, n in plan]).cuda()
        slot_map = torch.cat([torch.tensor([int(table[slot_of[r], t // page]) * page + t % page
                                            for t in range(done[r], done[r] + n)]) for r, n in plan])
        differential.diff_rope_store(x, pos, inv_freq, dims, True, slot_map.to(torch.int32).cuda(), cache, heads,
                                     kv_heads, dim, vdim, True, page)
        out = differential.differential_attention(x, x[:, -gw:], cache, table.cuda(), pos, row, heads, kv_heads, dim,
                                                  vdim, page, m["scale"], m["softcap"], lam, eps, 1.0 - m["diff"],
                                                  batch=step)
        split_steps += step.max_q_len == 1 and step.max_seq_len > 2 * differential.SPLIT_KEYS
        at = 0
        for r, n in plan:
            got[r].append(out[at:at + n].double().cpu())
            at += n
            done[r] += n
    assert split_steps >= 5
    for r in total:
        g_all = torch.cat(got[r])
        assert g_all.shape[0] == done[r] <= total[r]
        err = (g_all - want[r][:done[r]]).abs()
        assert float(err.max()) < 0.06 and float(err.mean()) < 0.006, (r, float(err.max()), float(err.mean()))


@pytest.mark.parametrize("experts,top,groups,keep,scale", [(16, 5, 4, 3, 1.75), (8, 2, 4, 2, 1.5), (6, 1, 1, 1, 1.0),
                                                           (4, 4, 2, 2, 0.5), (8, 3, 2, 1, 2.5), (40, 8, 8, 4, 1.0)])
def test_router_with_softmax_scores_and_group_maxima(experts, top, groups, keep, scale):
    from gllm_b200.ops import moe

    g = torch.Generator().manual_seed(experts * 10 + top)
    logits = torch.randn(300, experts, generator=g) * 3
    mlp = _moe(8, experts, top, scale, (groups, keep) if groups > 1 else None)
    chosen, weights = plain.route(logits.to(F), mlp, {"r.router": torch.eye(experts, dtype=F)}, "r")
    wide = torch.cat([logits, torch.zeros(300, 1)], 1).cuda()            # the logits as a slice of wider rows
    ids, w = moe.route(wide[:, :experts], None, top, groups, keep, True, score="softmax", group_score="max",
                       renormalize_eps=1e-20, scale=scale)
    for t in range(300):
        a = dict(zip(chosen[t].tolist(), weights[t].tolist()))
        b = dict(zip(ids[t].tolist(), w[t].tolist()))
        assert set(a) == set(b), t
        assert all(abs(a[e] - b[e]) < 1e-5 for e in a), t


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,ff,experts,top", [(37, 64, 32, 8, 2), (1, 44, 20, 4, 1), (300, 128, 64, 16, 4),
                                                   (9, 48, 24, 6, 6)])
def test_experts_without_a_gate_and_a_gated_shared_expert(dtype, n, width, ff, experts, top):
    """``down(relu(up x)^2)`` for the chosen experts, weighted, plus ``sigmoid(gate) * shared``; bf16 sizes that the
    tensor-core kernel takes run there, the others (and float32) on the CUDA cores."""
    from gllm_b200.ops import moe

    g = torch.Generator().manual_seed(n + width)
    rnd = lambda *s: torch.randn(*s, generator=g).to(dtype)
    x, up, down = rnd(n, width), rnd(experts, ff, width) / width ** 0.5, rnd(experts, width, ff) / ff ** 0.5
    shared, gate = rnd(n, width), torch.randn(n, 3, generator=g)
    ids = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    weights = torch.rand(n, top, generator=g) + 0.1
    want = torch.zeros(n, width, dtype=F)
    for t in range(n):
        for s in range(top):
            e = int(ids[t, s])
            hidden = torch.relu(up[e].to(F) @ x[t].to(F)) ** 2
            if dtype == torch.bfloat16:
                hidden = hidden.to(dtype).to(F)
            want[t] += float(weights[t, s]) * (down[e].to(F) @ hidden)
    want += plain.sigmoid(gate[:, 1:2].to(F)) * shared.to(F)
    cores = moe.tensor_cores_take(dtype, width, ff, gated=False)
    assert cores == (dtype == torch.bfloat16 and width % 8 == 0 and ff % 8 == 0)
    got = moe.apply_experts(x.cuda(), ids.cuda(), weights.cuda(), up.cuda().contiguous(), down.cuda().contiguous(),
                            shared.cuda(), cores, gated=False, shared_gate=gate.cuda()[:, 1])
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    assert torch.allclose(got.double().cpu(), want, atol=tol * float(want.abs().max()), rtol=tol)


# ------------------------------------------------------------------ each mechanism alone in a model of one layer
ALONE = {
    "attention": one_layer(_att(4, 2, 16, 24, 0.2, 8, softcap=10.0, diff=0.3, scaling=(4.0, 1.0, 4.0, 64))),
    "attention_one_head": one_layer(_att(1, 1, 40, 8, 0.15, 40, softcap=60.0, diff=0.9), width=40),
    "recurrence": one_layer(_ssd(4, 16, 16, 2, 4, 2)),
    "recurrence_head_groups": one_layer(_ssd(6, 8, 20, 6, 3, 1), width=56),
    "dense": one_layer(_ssd(2, 8, 8, 1, 2, 1), _dense(72)),
    "experts": one_layer(_ssd(2, 8, 8, 1, 2, 1), _moe(24, 8, 2, 1.7, (4, 2), 40)),
    "experts_plain": one_layer(_ssd(2, 8, 8, 1, 2, 1), _moe(16, 5, 5, 0.8)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", sorted(ALONE))
def test_each_mechanism_alone(kind, dtype, tmp_path):
    cfg = ALONE[kind]
    weights, _, runner = make(cfg, tmp_path, dtype, max_tokens=256, block_size=8)
    toks = torch.randint(0, cfg["vocab"], (90,), generator=torch.Generator().manual_seed(3)).tolist()
    want = {"r": plain.forward(cfg, weights, toks)}
    for rid, cuts in (("r", [90]), ("r", [40, 2, 17] + [1] * 31)):
        steps, index = steps_of(toks, cuts, rid=rid)
        compare(run_steps(runner, steps), index, want, *tolerance(dtype))


def test_residual_after_every_layer(tmp_path):
    """The fp32 residual stream after each layer (the branch that is still pending added) against the plain one."""
    from gllm_b200 import ops

    cfg = SAZISUN["A"]
    weights, _, runner = make(cfg, tmp_path, "float32")
    toks = torch.randint(0, cfg["vocab"], (23,), generator=torch.Generator().manual_seed(8)).tolist()
    _, layers = plain.forward(cfg, weights, toks, return_layers=True)
    seen = []
    for layer in runner.model.layers:
        def wrapped(branch, resid, ctx, cache, inner=layer.forward):
            out, resid = inner(branch, resid, ctx, cache)
            total = resid.clone()
            if out is not None and out is not ops.ADDED:
                total += ops.as_tensor(out).float()
            seen.append(total)
            return out, resid
        layer.forward = wrapped
    run_steps(runner, steps_of(toks, [23])[0])
    assert len(seen) == len(cfg["layers"])
    for i, got in enumerate(seen):
        assert torch.allclose(got.double().cpu(), layers[i], atol=2e-4, rtol=2e-4), i


# ------------------------------------------------------------------ whole models: cuts, batches, pages used again
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SAZISUN))
def test_all_cuts_and_mixed_batches(name, dtype, tmp_path):
    from gllm_b200.engine.replay import build_runner

    cfg = SAZISUN[name]
    weights, folder, runner = make(cfg, tmp_path, dtype, max_tokens=rounded(max(LENGTHS.values())),
                                   block_size=PAGE[name])
    seqs = sequences(cfg["vocab"], seed=5)
    want = {k: plain.forward(cfg, weights, v) for k, v in seqs.items()}
    steps, index = single_request_steps(seqs)
    compare(run_steps(runner, steps), index, want, *tolerance(dtype))
    runner.cache.check_invariants()
    # four live requests at most over 448 tokens of pages: pages and slots are used again
    _, small = build_runner(folder, dtype, 448, block_size=PAGE[name])
    steps, index = mixed_steps(seqs, max_tokens=448, seed=9)
    compare(run_steps(small, steps), index, want, *tolerance(dtype))
    small.cache.check_invariants()
    assert all(g.allocator.total_reused > 0 for g in small.cache.groups)


def test_replay_through_the_command(tmp_path):
    cfg = SAZISUN["A"]
    weights = decisive_routing(cfg, draw_weights(cfg, seed=7, sharp=1.5))
    folder = write_model(cfg, weights, str(tmp_path / "model"))
    seqs = sequences(cfg["vocab"], seed=6)
    want = {k: plain.forward(cfg, weights, v) for k, v in seqs.items()}
    steps, index = mixed_steps(seqs, max_tokens=448, seed=3)
    results = replay(folder, "float32", steps, str(tmp_path / "out"), max_tokens=448, vocab=cfg["vocab"])
    compare(results, index, want, FP32_TOL)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_at_every_edge(dtype, tmp_path):
    """Portions that end one token before, at and after every page border and key-block border (pages of 16, key
    blocks of 32), down to two tokens, through a layer that owns its keys and one that reads them."""
    cfg = SAZISUN["C"]
    weights, _, runner = make(cfg, tmp_path, dtype, max_tokens=256, block_size=16)
    toks = torch.randint(0, cfg["vocab"], (100,), generator=torch.Generator().manual_seed(10)).tolist()
    want = {"r": plain.forward(cfg, weights, toks)}
    for cuts in ([15, 2, 15, 1, 31, 2, 30, 4], [16, 16, 1, 31, 33, 3], [17, 14, 2, 2, 29, 36], [2] * 50):
        steps, index = steps_of(toks, cuts)
        compare(run_steps(runner, steps), index, want, *tolerance(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_in_a_model(dtype, tmp_path):
    """One layer of attention whose first map looks for one token: the keys of token ``MARK`` and the queries of
    token ``ASK`` are scaled up along one unrotated column, so that a query at position 400 gives most of its first
    map's weight to a key at position 5, 21 pages and 12 key blocks back; read in a prompt, in portions and decoded
    alone.  Without the far key the asked positions' logits differ by far more than the tolerance."""
    cfg = one_layer(_att(2, 1, 16, 16, 0.25, 8, softcap=40.0, diff=0.2), width=32, vocab=60)
    weights = draw_weights(cfg, seed=15)
    MARK, ASK, col = 7, 11, 12                                   # column 12 of a map is not rotated
    weights["embed"][:, :2] = 0                                  # the two columns that carry the marks
    weights["embed"][MARK] = 0
    weights["embed"][MARK, 0] = 4.0
    weights["embed"][ASK] = 0
    weights["embed"][ASK, 1] = 4.0
    for name, column in (("l0.mix.k", 0), ("l0.mix.q", 1)):
        w = weights[name].clone()
        w[:, column] = 0
        for unit in range(0, w.shape[0] // 16, 2):               # map 1 of every head
            w[unit * 16 + col, column] = 6.0
        weights[name] = w
    weights["l0.norm1"][:2], weights["l0.norm1.b"][:2] = 1.0, 0.0
    g = torch.Generator().manual_seed(16)
    toks = [int(t) for t in torch.randint(12, 60, (420,), generator=g)]
    toks[5] = MARK
    for p in (100, 257, 400, 415):
        toks[p] = ASK
    _, _, runner = make(cfg, tmp_path, dtype, max_tokens=448, block_size=16, weights=weights)
    want = {"r": plain.forward(cfg, weights, toks)}
    without = list(toks)
    without[5] = 13
    moved = (plain.forward(cfg, weights, without)[400] - want["r"][400]).abs().max()
    assert float(moved) > 0.1 * float(want["r"].abs().max())
    for cuts in ([420], [399, 1, 1] + [19], [64] * 6 + [16, 2, 2] + [1] * 16):
        steps, index = steps_of(toks, cuts)
        compare(run_steps(runner, steps), index, want, *tolerance(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(dtype, tmp_path):
    """Prompts of one, two and three tokens, then hundreds of tokens decoded one by one (replays of the decode
    graph): state that is lost, doubled or started wrong shows at once or adds up."""
    cfg = SAZISUN["A"]
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
    cfg = SAZISUN["B"]
    weights, _, runner = make(cfg, tmp_path, "float32", max_tokens=64, max_live=1)
    g = torch.Generator().manual_seed(13)
    a = torch.randint(0, cfg["vocab"], (60,), generator=g).tolist()
    b = torch.randint(0, cfg["vocab"], (50,), generator=g).tolist()
    for rid, toks, cuts in (("a", a, [33, 20, 7]), ("b", b, [3, 40] + [1] * 7), ("c", a, [60])):
        steps, index = steps_of(toks, cuts, rid=rid)
        compare(run_steps(runner, steps), index, {rid: plain.forward(cfg, weights, toks)}, FP32_TOL)
    assert runner.cache.groups[0].allocator.total_reused > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(name, dtype, tmp_path):
    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine

    cfg = SAZISUN[name]
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
    if dtype == "float32":
        for req, r in zip(reqs, results):
            assert engine.generate([req])[0].token_ids == r.token_ids


def test_random_weights_mode_writes_a_model_that_runs(tmp_path):
    from gllm_b200.config import load_config
    from gllm_b200.engine.replay import build_runner
    from gllm_b200.weights import write_random_model

    folder = write_random_model(str(tmp_path / "m"), load_config(copy.deepcopy(SAZISUN["C"])), seed=3, std=0.05)
    _, runner = build_runner(folder, "bfloat16", 256)
    toks = list(range(1, 70))
    whole = run_steps(runner, steps_of(toks, [69], rid="a")[0])[0]
    cut = run_steps(runner, steps_of(toks, [30, 38, 1], rid="b")[0])
    assert np.isfinite(whole).all()
    assert np.abs(whole[-1] - cut[2][0]).max() <= 0.05 * max(1.0, np.abs(whole).max())
