"""Fakilorn on the GPU against the plain implementation: each new mechanism alone, then the step
function under every way of cutting requests into steps, then generation through the entry point."""

from __future__ import annotations

import io
import itertools
import json
import math

import numpy as np
import pytest
import torch

import plain_fakilorn as plain
from fakilorn_cases import (PAGE_TOKENS, assert_rows_close, config, plain_greedy, plain_logits,
                            random_weights, relative_error, tokens_for)

from mini_gpt_inference_b200 import EngineConfig, FakilornConfig, LLMEngine, SamplingParams
from mini_gpt_inference_b200.cache.storage import PagedKVView
from mini_gpt_inference_b200.engine.build import load_model, make_runner
from mini_gpt_inference_b200.engine.runner import StepEntry

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# Largest |engine - plain| on a row of logits, over the row's own spread.  32-bit: rounding of sums.
# bfloat16: both sides use the same bfloat16 weights; activations are rounded to 8 bits between
# kernels.  A lost key, gate, expert or blend shows as 0.3 and more.
TOL = {"float32": 3e-4, "bfloat16": 6e-2}


@pytest.fixture(scope="module")
def ops():
    from mini_gpt_inference_b200.kernels.ops import default_ops

    return default_ops("cuda:0")


def dev(t, dtype=None):
    return t.to(device="cuda:0", dtype=dtype or t.dtype).contiguous()


class Ctx:
    """The few fields of a step's context that the attention kernels read."""

    def __init__(self, tables, token_request, positions, q_len, decode_only=False):
        self.block_tables = [dev(torch.tensor(tables, dtype=torch.int32))]
        self.token_request = dev(torch.tensor(token_request, dtype=torch.int32))
        self.positions = dev(torch.tensor(positions, dtype=torch.int32))
        starts = [sum(q_len[:i]) for i in range(len(q_len))]
        self.req_q_start = dev(torch.tensor(starts, dtype=torch.int32))
        self.req_q_len = dev(torch.tensor(q_len, dtype=torch.int32))
        self.host_q_len = list(q_len)
        self.decode_only = decode_only
        self.max_ctx_after = max(positions) + 1


# ---- mechanisms alone ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,groups,d,dv", [(4, 2, 24, 16), (3, 3, 40, 40), (5, 1, 10, 70)])
def test_unit_norm_blend_and_page_write(ops, dtype, heads, groups, d, dv):
    t, n, pt, pages, eps = DTYPES[dtype], 7, 4, 6, 1e-3
    gen = torch.Generator().manual_seed(d)
    ld = heads * d + groups * d + groups * dv + 5
    proj = (3 * torch.randn(n, ld, generator=gen)).to(t)
    other = torch.randn(n, groups * dv + 3, generator=gen).to(t)
    lam = torch.tensor([0.3])
    slots = torch.tensor([9, 3, -1, 20, 21, 0, 14], dtype=torch.int32)
    positions = torch.tensor([4, 1, -1, 0, 1, 2, 9], dtype=torch.int32)
    k_off, v_off = heads * d, heads * d + groups * d
    for blend in (False, True):
        k_pages = torch.full((pages, groups, pt, d), float("nan"), dtype=t, device="cuda:0")
        v_pages = torch.full((pages, groups, pt, dv), float("nan"), dtype=t, device="cuda:0")
        cache = PagedKVView(k_pages, v_pages, 0, pt, None, True)
        work = dev(proj)
        ops.head_prepare(work, heads, groups, d, dv, 0, k_off, v_off, True, eps, cache, dev(slots), dev(positions),
                         v_other=dev(other)[:, : groups * dv] if blend else None, blend=dev(lam) if blend else None)
        x = proj.double()
        q = plain.unit_rms(x[:, :k_off].view(n, heads, d), eps).view(n, -1)
        k = plain.unit_rms(x[:, k_off:v_off].view(n, groups, d), eps)
        v = x[:, v_off: v_off + groups * dv]
        if blend:
            v = plain.blend_values(v, other.double()[:, : groups * dv], 0.3)
        v = v.view(n, groups, dv)
        tol = 1e-5 if dtype == "float32" else 2e-2
        live = positions >= 0
        got = work.double().cpu()
        assert torch.allclose(got[live, :k_off], q[live], atol=tol, rtol=tol)
        assert torch.equal(got[~live], x[~live]) and torch.equal(got[:, k_off:], x[:, k_off:])
        kp, vp = k_pages.double().cpu(), v_pages.double().cpu()
        written = torch.zeros(pages * pt, dtype=torch.bool)
        for i in range(n):
            s = int(slots[i])
            if s < 0:
                continue
            written[s] = True
            assert torch.allclose(kp[s // pt, :, s % pt], k[i], atol=tol, rtol=tol)
            assert torch.allclose(vp[s // pt, :, s % pt], v[i], atol=tol, rtol=tol)
        rows = kp.permute(0, 2, 1, 3).reshape(pages * pt, -1)
        assert torch.isnan(rows[~written]).all() and not torch.isnan(rows[written]).any()


@pytest.mark.parametrize("dtype,path", [("float32", "general"), ("bfloat16", "general"), ("bfloat16", "tiles"),
                                        ("bfloat16", "ranges")])
@pytest.mark.parametrize("heads,groups,d,dv,pt", [(4, 2, 24, 16, 8), (3, 3, 32, 32, 16), (6, 1, 10, 70, 4),
                                                  (8, 2, 96, 32, 16), (16, 1, 128, 128, 32), (5, 5, 72, 104, 8)])
def test_attention_far_key_gate_and_sizes(ops, dtype, path, heads, groups, d, dv, pt):
    """Two requests on scattered pages.  Every query is made to point at one key far back (or, for the
    second request, at the key of a page's last row): with a large scale nearly all weight lies
    there, so an attention that misses that key, a head's group or the gate is off by far."""
    t = DTYPES[dtype]
    lengths = [300, 45]
    gen = torch.Generator().manual_seed(pt)
    per_req = [-(-n // pt) for n in lengths]
    order = torch.randperm(sum(per_req) + 3, generator=gen).tolist()
    tables = [order[: per_req[0]], order[per_req[0]: per_req[0] + per_req[1]] + [-1] * (per_req[0] - per_req[1])]
    k_all = [torch.randn(n, groups, d, generator=gen) for n in lengths]
    v_all = [torch.randn(n, groups, dv, generator=gen) for n in lengths]
    # queries: the last 5 positions of request 0 and positions 20..44 of request 1
    rows = [(0, p) for p in range(295, 300)] + [(1, p) for p in range(20, 45)]
    targets = [3, 77, 150, 294, 299] + [pt * (p // pt) - 1 if p >= pt else 0 for p in range(20, 45)]
    for r, j in sorted({(r, j) for (r, _), j in zip(rows, targets)}):
        k_all[r][j] *= 3.0                                    # the chosen keys are long: they win against hundreds
    k_pages = torch.full((len(order), groups, pt, d), float("nan"))
    v_pages = torch.full((len(order), groups, pt, dv), float("nan"))
    for r, n in enumerate(lengths):
        for j in range(n):
            k_pages[tables[r][j // pt], :, j % pt] = k_all[r][j]
            v_pages[tables[r][j // pt], :, j % pt] = v_all[r][j]
    n = len(rows)
    q = 0.3 * torch.randn(n, heads, d, generator=gen)
    for i, ((r, p), j) in enumerate(zip(rows, targets)):
        for h in range(heads):
            q[i, h] += 0.7 * k_all[r][j, h // (heads // groups)]
    gate = torch.randn(n, heads * dv, generator=gen)
    scale = 6.0 / math.sqrt(d)
    q_rows = torch.cat([q.reshape(n, -1), torch.randn(n, 8, generator=gen)], dim=1).to(t)     # wider rows
    gate_rows = torch.cat([torch.randn(n, 4, generator=gen), gate], dim=1).to(t)
    cache = PagedKVView(dev(k_pages, t), dev(v_pages, t), 0, pt, None, False)
    ctx = Ctx(tables, [r for r, _ in rows], [p for _, p in rows], [5, 25], decode_only=path == "ranges")
    g_dev = dev(gate_rows)
    launches = ops.launches
    ops.use_mma_attention = path != "general"
    try:
        got = ops.paged_attention_general(dev(q_rows), heads, groups, d, dv, scale, cache, ctx, gate=g_dev[:, 4:])
        got_plain = ops.paged_attention_general(dev(q_rows), heads, groups, d, dv, scale, cache, ctx)
    finally:
        ops.use_mma_attention = True
    if d % 8 == 0 and dv % 8 == 0:
        # sizes that the tensor-core kernels take: they ran (ranges: two launches a call), or they were off
        assert ops.launches - launches == {"general": 2, "tiles": 2, "ranges": 4}[path]
    if path == "ranges":
        # the ranges merged by the last CTA of a token instead of by a second kernel: the same numbers
        ops.merge_ranges_in_last_cta = True
        try:
            again = ops.paged_attention_general(dev(q_rows), heads, groups, d, dv, scale, cache, ctx, gate=g_dev[:, 4:])
        finally:
            ops.merge_ranges_in_last_cta = False
        assert torch.allclose(again.float(), got.float(), atol=1e-2, rtol=1e-2)
    want = torch.empty(n, heads, dv, dtype=torch.float64)
    peak = []
    for i, (r, p) in enumerate(rows):
        for h in range(heads):
            g = h // (heads // groups)
            s = (k_all[r][: p + 1, g].to(t).double() @ q_rows[i, h * d: (h + 1) * d].double()) * scale
            w = torch.softmax(s, 0)
            peak.append(float(w[targets[i]]))
            want[i, h] = w @ v_all[r][: p + 1, g].to(t).double()
    assert min(peak) > 0.5                                   # the chosen key does carry the weight
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert torch.allclose(got_plain.double().cpu(), want.view(n, -1), atol=tol, rtol=tol)
    gated = want.view(n, -1) * torch.sigmoid(gate_rows[:, 4:].double())
    assert torch.allclose(got.double().cpu(), gated, atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype,path", [("float32", "general"), ("bfloat16", "general"), ("bfloat16", "tiles"),
                                        ("bfloat16", "ranges")])
@pytest.mark.parametrize("window,pt", [(40, 8), (64, 16), (129, 4)])
def test_attention_window_edges(ops, dtype, path, window, pt):
    """A window of the last `window` keys (a parameter of the mixer that this design leaves unused):
    the key just outside the window is made the most attractive of all, the first key inside it the
    second most; a kernel that is one key off at either edge gives another row."""
    t = DTYPES[dtype]
    heads, groups, d, dv, length = 4, 2, 32, 48, 300
    gen = torch.Generator().manual_seed(window)
    n_pages = -(-length // pt)
    order = torch.randperm(n_pages + 2, generator=gen).tolist()
    tables = [order[:n_pages]]
    k_all = torch.randn(length, groups, d, generator=gen)
    v_all = torch.randn(length, groups, dv, generator=gen)
    positions = list(range(length - 24, length))
    direction = torch.randn(groups, d, generator=gen)
    for p in positions:                                         # (edges of neighbouring queries overlap: the
        k_all[p - window] = 4.0 * direction                     #  later assignment wins, the oracle sees the same)
        k_all[p - window + 1] = 3.0 * direction
    k_pages = torch.full((len(order), groups, pt, d), float("nan"))
    v_pages = torch.full((len(order), groups, pt, dv), float("nan"))
    for j in range(length):
        k_pages[tables[0][j // pt], :, j % pt] = k_all[j]
        v_pages[tables[0][j // pt], :, j % pt] = v_all[j]
    n = len(positions)
    q = (0.2 * torch.randn(n, heads, d, generator=gen)
         + direction.repeat_interleave(heads // groups, 0)[None]).reshape(n, -1).to(t)
    cache = PagedKVView(dev(k_pages, t), dev(v_pages, t), 0, pt, window, False)
    ctx = Ctx(tables, [0] * n, positions, [n], decode_only=path == "ranges")
    ops.use_mma_attention = path != "general"
    try:
        got = ops.paged_attention_general(dev(q), heads, groups, d, dv, 1.0 / math.sqrt(d), cache, ctx)
    finally:
        ops.use_mma_attention = True
    want = torch.empty(n, heads, dv, dtype=torch.float64)
    inside = []
    for i, p in enumerate(positions):
        lo = p - window + 1
        for h in range(heads):
            g = h // (heads // groups)
            s = (k_all[lo: p + 1, g].to(t).double() @ q[i, h * d: (h + 1) * d].double()) / math.sqrt(d)
            w = torch.softmax(s, 0)
            inside.append(float(w[0]))
            want[i, h] = w @ v_all[lo: p + 1, g].to(t).double()
    assert max(inside) > 0.3                                    # the first key inside the window matters
    tol = 2e-5 if dtype == "float32" else 3e-2
    assert torch.allclose(got.double().cpu(), want.view(n, -1), atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("m,n,k", [(1, 96, 64), (9, 37, 50), (40, 200, 96), (150, 256, 64), (300, 96, 256)])
def test_squared_relu_projection(ops, dtype, m, n, k):
    t = DTYPES[dtype]
    gen = torch.Generator().manual_seed(m)
    x, w = torch.randn(m, k, generator=gen).to(t), (torch.randn(n, k, generator=gen) / math.sqrt(k)).to(t)
    got = ops.linear(dev(x), dev(w), None, "relu_sq", t)
    want = torch.relu(x.double() @ w.double().T) ** 2
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert torch.allclose(got.double().cpu(), want, atol=tol, rtol=tol)
    assert (want == 0).any() and (got.double().cpu()[want == 0] == 0).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,width,inner,shared", [(5, 2, 64, 40, 24), (4, 1, 96, 48, None),
                                                            (6, 6, 50, 11, 9), (1, 1, 32, 16, 8), (40, 3, 64, 8, None)])
def test_router_and_experts(ops, dtype, experts, top, width, inner, shared):
    t = DTYPES[dtype]
    gen = torch.Generator().manual_seed(experts * 10 + top)
    n = 70
    y = torch.randn(n, width, generator=gen).to(t)
    w = {"router": torch.randn(experts, width, generator=gen).to(torch.bfloat16)}
    for e in range(experts):
        w[f"e{e}.gate"] = (torch.randn(inner, width, generator=gen) / math.sqrt(width)).to(t)
        w[f"e{e}.up"] = (torch.randn(inner, width, generator=gen) / math.sqrt(width)).to(t)
        w[f"e{e}.down"] = (torch.randn(width, inner, generator=gen) / math.sqrt(inner)).to(t)
    sg = torch.randn(width, generator=gen).to(torch.bfloat16)
    positions = torch.arange(n, dtype=torch.int32)
    positions[13] = -1                                        # a padding row chooses nothing
    ids, weights, gate = ops.moe_route(dev(y), dev(w["router"], torch.float32), dev(sg, torch.float32),
                                       dev(positions), top)
    want_ids, want_w = plain.route(y.double(), w["router"].double(), top)
    live = positions >= 0
    assert torch.equal(ids.cpu()[live].long(), want_ids[live]) and (ids.cpu()[13] == -1).all()
    assert torch.allclose(weights.double().cpu()[live], want_w[live], atol=1e-5)
    assert torch.allclose(gate.double().cpu()[live], torch.sigmoid(y.double() @ sg.double())[live], atol=1e-5)
    w_in = torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(experts)])
    w_out = torch.stack([w[f"e{e}.down"] for e in range(experts)])
    residual = torch.randn(n, width, generator=gen)
    res_dev = dev(residual)
    ops.moe_experts_residual(dev(y), ids, weights, dev(w_in), dev(w_out), res_dev)
    mlp = {"router": {"experts": experts, "top": top}}
    want = residual.double() + plain.routed_ff(y.double(), {k: v.double() for k, v in w.items()}, "", mlp)
    tol = 2e-5 if dtype == "float32" else 3e-2
    got = res_dev.double().cpu()
    assert torch.allclose(got[live], want[live], atol=tol, rtol=tol)
    assert torch.equal(got[13], residual.double()[13])
    if shared is not None:
        gu = torch.randn(n, 2 * shared, generator=gen).to(t)
        got = ops.glu(dev(gu), gate)
        a, u = gu.double()[:, :shared], gu.double()[:, shared:]
        want = a * torch.sigmoid(a) * u * gate.double().cpu()[:, None]
        assert torch.allclose(got.double().cpu(), want, atol=tol, rtol=tol)


def test_scaled_embedding_and_head(ops):
    gen = torch.Generator().manual_seed(0)
    table = torch.randn(31, 24, generator=gen).to(torch.bfloat16)
    ids = torch.tensor([3, 30, 0, 7], dtype=torch.int32)
    pos = torch.tensor([0, 1, -1, 5], dtype=torch.int32)
    got = ops.embed(dev(ids), dev(pos), dev(table), None, scale=1.7)
    want = plain.embed(ids.tolist(), table.float(), 1.7)
    want[2] = 0
    assert torch.allclose(got.cpu(), want, atol=1e-6)
    y = torch.randn(4, 24, generator=gen)
    got = ops.logits(dev(y), dev(table.float()), scale=0.37)
    assert torch.allclose(got.cpu().double(), (y.double() @ table.double().T) * 0.37, atol=1e-5)


# ---- the step function --------------------------------------------------------------------------
CASES = [(w, d, s) for w in "ABCD" for d in ("float32", "bfloat16") for s in (1.0, 4.0)]
IDS = [f"{w}-{d}-{'sharp' if s > 1 else 'soft'}" for w, d, s in CASES]


def setup(which, dtype, sharp, num_pages=64, seed=3, max_requests=4):
    from mini_gpt_inference_b200.kernels.ops import default_ops

    raw = config(which, sharp, every_expert=dtype == "bfloat16")
    tensors = random_weights(raw, seed)
    loaded = load_model(config=FakilornConfig.from_dict(raw), tensors=tensors, dtype=dtype, device="cuda:0")
    runner = make_runner(loaded, default_ops("cuda:0"), PAGE_TOKENS[which], num_pages, max_requests)
    return raw, tensors, runner, TOL[dtype] * (2 if sharp > 1 and dtype == "bfloat16" else 1)


@pytest.mark.parametrize("which,dtype,sharp", CASES, ids=IDS)
def test_whole_prompts(which, dtype, sharp):
    raw, tensors, runner, tol = setup(which, dtype, sharp, num_pages=400)
    pt = PAGE_TOKENS[which]
    for length, seed in [(150, 1), (37, 2), (1, 3), (2, 4), (pt + 1, 5), (pt, 6), (1300, 7)]:
        tokens = tokens_for(raw, length, seed)
        got = runner.step([StepEntry("r", tokens, list(range(length)))])
        runner.finish("r")
        assert got.shape == (length, raw["vocab"]) and got.dtype == torch.float32
        assert_rows_close(got, plain_logits(raw, tensors, tokens), tol, f"whole prompt of {length}")
    runner.manager.check()
    assert runner.manager.stats()["allocated_blocks"] == 0


@pytest.mark.parametrize("which,dtype,sharp", CASES, ids=IDS)
def test_prefill_then_single_tokens(which, dtype, sharp):
    """A short prompt, then a long run of single tokens (replayed from a CUDA graph), and the same
    sequence token by token from the very first token."""
    raw, tensors, runner, tol = setup(which, dtype, sharp)
    tokens = tokens_for(raw, 120, 7)
    want = plain_logits(raw, tensors, tokens)
    outs = [runner.step([StepEntry("r", tokens[:9], list(range(9)))])]
    outs += [runner.step([StepEntry("r", tokens[t: t + 1], [0])]) for t in range(9, 120)]
    assert_rows_close(torch.cat(outs), want, tol, "prefill then single tokens")
    one_by_one = torch.cat([runner.step([StepEntry("s", tokens[t: t + 1], [0])]) for t in range(40)])
    assert_rows_close(one_by_one, want[:40], tol, "single tokens from the first")
    if dtype == "float32":
        # in 32-bit the cut into steps changes no bit
        assert torch.equal(one_by_one, torch.cat(outs)[:40])


@pytest.mark.parametrize("which,dtype,sharp", CASES, ids=IDS)
def test_portions_of_changing_size(which, dtype, sharp):
    raw, tensors, runner, tol = setup(which, dtype, sharp)
    tokens = tokens_for(raw, 131, 8)
    want = plain_logits(raw, tensors, tokens)
    sizes = itertools.cycle([13, 7, 2, 5, 2, 1, 3, 16, 2, 9, 33])
    outs, pos = [], 0
    while pos < len(tokens):
        n = min(next(sizes), len(tokens) - pos)
        outs.append(runner.step([StepEntry("r", tokens[pos: pos + n], list(range(n)))]))
        pos += n
    assert_rows_close(torch.cat(outs), want, tol, "portions of changing size")


@pytest.mark.parametrize("which,dtype,sharp", CASES, ids=IDS)
def test_mixed_batches_reuse_pages_and_slots(which, dtype, sharp):
    """Up to four live requests, portions of some beside single tokens of others, requests left out
    of steps; the pool holds the four longest and no more, so pages and slots are handed out
    again.  Every cache row starts as NaN and turns NaN again when its request ends."""
    pt = PAGE_TOKENS[which]
    lengths = [90, 29, 71, 3, 41, 2 * pt, 17, 55, 1]
    pool = sum(sorted(-(-n // pt) for n in lengths)[-4:])
    raw, tensors, runner, tol = setup(which, dtype, sharp, num_pages=pool)
    for pages in runner.storage.k + runner.storage.v:
        pages.fill_(float("nan"))
    reqs = {f"q{i}": tokens_for(raw, n, 20 + i) for i, n in enumerate(lengths)}
    want = {rid: plain_logits(raw, tensors, toks) for rid, toks in reqs.items()}
    got = {rid: [] for rid in reqs}
    waiting, live = list(reqs), {}
    sizes = itertools.cycle([5, 1, 2, 11, 1, 1, 7, 3, 1, 2, 1, 1, 19])
    gen = torch.Generator().manual_seed(99)
    while waiting or live:
        while waiting and len(live) < 4:
            live[waiting.pop(0)] = 0
        entries, order = [], []
        for rid in list(live):
            if len(live) > 1 and torch.rand((), generator=gen).item() < 0.25:
                continue
            pos = live[rid]
            n = min(next(sizes), len(reqs[rid]) - pos)
            entries.append(StepEntry(rid, reqs[rid][pos: pos + n], list(range(n))))
            order.append((rid, n))
            live[rid] = pos + n
        if not entries:
            continue
        logits = runner.step(entries)
        row = 0
        for rid, n in order:
            got[rid].append(logits[row: row + n].clone())
            row += n
            if live[rid] == len(reqs[rid]):
                tables = [list(t) for t in runner.manager.get(rid).tables]
                runner.finish(rid)
                del live[rid]
                for g, table in enumerate(tables):
                    for page in table:
                        if page >= 0:
                            runner.storage.k[g][:, page] = float("nan")
                            runner.storage.v[g][:, page] = float("nan")
    for rid in reqs:
        assert_rows_close(torch.cat(got[rid]), want[rid], tol, f"request {rid} in mixed batches")
    runner.manager.check()
    assert runner.manager.stats()["allocated_blocks"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_of_unequal_requests_equals_each_alone(dtype):
    raw, tensors, runner, tol = setup("A", dtype, 4.0, num_pages=64, max_requests=8)
    prompts = [tokens_for(raw, n, 70 + n) for n in (1, 2, 33, 64, 7)]
    alone = []
    for i, p in enumerate(prompts):
        alone.append(runner.step([StepEntry(f"a{i}", p, list(range(len(p))))]))
        runner.finish(f"a{i}")
    together = runner.step([StepEntry(f"b{i}", p, list(range(len(p)))) for i, p in enumerate(prompts)])
    if dtype == "float32":
        assert torch.equal(together, torch.cat(alone))
    else:
        assert float(relative_error(together, torch.cat(alone).cpu()).max()) < tol


# ---- generation through the entry point, its scheduler and sampler ---------------------------------
@pytest.mark.parametrize("which", "ABC")
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(which, dtype):
    raw = config(which, 2.0, every_expert=dtype == "bfloat16")
    tensors = random_weights(raw, 11)
    loaded = load_model(config=FakilornConfig.from_dict(raw), tensors=tensors, dtype=dtype, device="cuda:0")
    engine = LLMEngine(loaded, EngineConfig(dtype=dtype, block_size=PAGE_TOKENS[which], num_blocks=48,
                                            max_batch_size=3, max_num_batched_tokens=16, max_prefill_chunk=7))
    prompts = [tokens_for(raw, n, 40 + i) for i, n in enumerate([5, 1, 23, 12, 2, 17])]
    outs = engine.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0))
    for prompt, out in zip(prompts, outs):
        assert len(out["token_ids"]) == 12 and out["finish_reason"] == "length"
        seq = prompt + out["token_ids"]
        want = plain_logits(raw, tensors, seq[:-1])
        for i, token in enumerate(out["token_ids"]):
            row = want[len(prompt) - 1 + i]
            assert row.max() - row[token] <= 2 * TOL[dtype] * row.std(), (i, token, int(row.argmax()))
        if dtype == "float32":
            assert out["token_ids"] == plain_greedy(raw, tensors, prompt, 12)
    assert engine.stats()["allocated_blocks"] == 0
    engine.runner.manager.check()


def test_long_decoding_through_the_engine():
    raw = config("B", 2.0)
    tensors = random_weights(raw, 12)
    loaded = load_model(config=FakilornConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cuda:0")
    engine = LLMEngine(loaded, EngineConfig(dtype="float32", block_size=8, num_blocks=40, max_batch_size=2))
    prompt = tokens_for(raw, 3, 9)
    out = engine.generate([prompt], SamplingParams(max_tokens=260, temperature=0.0))[0]
    assert out["token_ids"] == plain_greedy(raw, tensors, prompt, 260)


def test_trace_replay(tmp_path):
    """The replay program on a model folder: two requests, portions beside single tokens, a slot
    and pages used again by a third request."""
    from mini_gpt_inference_b200.engine.trace import main
    from mini_gpt_inference_b200.weights.safetensors_io import save_file

    raw = config("A", 3.0)
    tensors = random_weights(raw, 13)
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(raw))
    save_file(tensors, folder / "model.safetensors")
    a, b, c = tokens_for(raw, 50, 1), tokens_for(raw, 20, 2), tokens_for(raw, 64, 3)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[:7], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[7:], "want": [12]}, {"id": "a", "tokens": a[31:], "want": [18]}], "end": ["a", "b"]},
        {"step": 3, "entries": [{"id": "c", "tokens": c[:62], "want": [61]}], "end": []},
        {"step": 4, "entries": [{"id": "c", "tokens": c[62:], "want": [0, 1]}], "end": ["c"]},
    ]
    for dtype in ("float32", "bfloat16"):
        if dtype == "bfloat16":                              # (see fakilorn_cases.config on every_expert)
            raw = config("A", 3.0, every_expert=True)
            (folder / "config.json").write_text(json.dumps(raw))
        out = tmp_path / dtype
        stdout = io.StringIO()
        code = main(["--model", str(folder), "--dtype", dtype, "--out", str(out), "--max-tokens", "128",
                     "--live-requests", "2"], stdin=io.StringIO("\n".join(json.dumps(s) for s in steps) + "\n"),
                    stdout=stdout)
        assert code == 0 and stdout.getvalue().split() == ["done", "0", "done", "1", "done", "2", "done", "3", "done", "4"]
        la, lb, lc = (plain_logits(raw, tensors, t) for t in (a, b, c))
        want = {0: la[[0, 29]], 1: la[[30]], 2: torch.stack([lb[19], la[49]]), 3: lc[[61]], 4: lc[[62, 63]]}
        for step, rows in want.items():
            got = torch.from_numpy(np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(rows), raw["vocab"]))
            assert_rows_close(got, rows, 2 * TOL[dtype], f"{dtype} step {step}")


def test_command_line_writes_and_generates(tmp_path):
    """bin/generate: a random-weights folder from a config.json, then greedy tokens from it that equal
    the plain implementation's on the folder's own tensors."""
    import subprocess
    import sys
    from pathlib import Path

    from mini_gpt_inference_b200.weights import load_file

    root = Path(__file__).resolve().parent.parent
    raw = config("B", 2.0)
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(raw))
    folder = tmp_path / "model"
    made = subprocess.run([sys.executable, str(root / "bin" / "generate"), "--random-weights", "3", "--config", str(cfg_path),
                           "--write-model", str(folder), "--weights-dtype", "bfloat16"], capture_output=True, text=True)
    assert made.returncode == 0, made.stderr[-2000:]
    prompt = tokens_for(raw, 9, 5)
    run = subprocess.run([sys.executable, str(root / "bin" / "generate"), "--model", str(folder), "--dtype", "float32",
                          "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "8", "--temperature", "0"],
                         capture_output=True, text=True)
    assert run.returncode == 0, run.stderr[-2000:]
    out = json.loads(run.stdout.strip().splitlines()[-1])
    assert out["token_ids"] == plain_greedy(raw, load_file(folder / "model.safetensors"), prompt, 8)
