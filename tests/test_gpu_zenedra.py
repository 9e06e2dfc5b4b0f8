"""Zenedra on the GPU against the plain implementation: each new mechanism alone, then the step
function under every way of cutting requests into steps, then generation through the entry point."""

from __future__ import annotations

import io
import itertools
import json
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_zenedra as plain
from zenedra_cases import (PAGE_TOKENS, assert_rows_close, config, plain_greedy, plain_logits, random_weights,
                           relative_error, tokens_for)

from mini_gpt_inference_b200 import EngineConfig, LLMEngine, SamplingParams, ZenedraConfig
from mini_gpt_inference_b200.cache.storage import PagedKVView
from mini_gpt_inference_b200.engine.build import load_model, make_runner
from mini_gpt_inference_b200.engine.runner import StepEntry

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# Largest |engine - plain| on a row of logits, over the row's own spread.  32-bit: rounding of sums.
# bfloat16: both sides use the same weights; activations are rounded to 8 bits between kernels.  A
# lost key, state, gate, expert or pass shows as 0.3 and more.
TOL = {"float32": 3e-4, "bfloat16": 1e-1}


@pytest.fixture(scope="module")
def ops():
    from mini_gpt_inference_b200.kernels.ops import default_ops

    return default_ops("cuda:0")


def dev(t, dtype=None):
    return t.to(device="cuda:0", dtype=dtype or t.dtype).contiguous()


def ints(values):
    return dev(torch.tensor(values, dtype=torch.int32))


def batch(q_len, ctx_before, slots, tables=None):
    """The fields of a step's context that the new kernels read."""
    starts = [sum(q_len[:i]) for i in range(len(q_len))]
    request = [r for r, n in enumerate(q_len) for _ in range(n)]
    positions = [c + i for n, c in zip(q_len, ctx_before) for i in range(n)]
    ctx = SimpleNamespace(req_q_start=ints(starts), req_q_len=ints(q_len), req_ctx_before=ints(ctx_before),
                          req_state_slot=ints(slots), token_request=ints(request), positions=ints(positions),
                          num_requests=len(q_len), host_q_len=list(q_len), decode_only=all(n == 1 for n in q_len),
                          max_ctx_after=max(positions) + 1, extra={})
    if tables is not None:
        ctx.block_tables = [ints(tables)]
    return ctx


def close(got, want, dtype, what, scale=1.0):
    tol = (2e-5 if dtype == "float32" else 2.5e-2) * scale
    err = (got.double().cpu() - want.double()).abs().max() / want.double().abs().max()
    assert err < tol, f"{what}: {float(err):.3e} of the largest value"


# ---- mechanisms alone ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,offset", [(64, 1.0), (72, 0.0), (1030, 1.0), (37, 1.0)])
def test_rms_norm(ops, dtype, width, offset):
    gen = torch.Generator().manual_seed(width)
    x, w = 3 * torch.randn(9, width, generator=gen), 0.3 * torch.randn(width, generator=gen)
    got = ops.rmsnorm(dev(x), dev(w), 1e-3, offset, DTYPES[dtype])
    close(got, plain.rms_norm(x.double(), w.double(), 1e-3, offset), dtype, "rms norm")


def test_pair_embedding_and_the_token_before(ops):
    """Three requests in one step (a first portion, a continued one whose token before lies in its state
    slot, a single first token), then a second step that continues all three; last a step whose tokens
    are still on the device where the step before left them."""
    gen = torch.Generator().manual_seed(5)
    vocab, width, buckets, mp, mc = 50, 24, 7, 31, 5
    tables = {"embed": torch.randn(vocab, width, generator=gen), "bigram": torch.randn(buckets + 1, width, generator=gen),
              "pos": torch.randn(64, width, generator=gen)}
    cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}}
    seqs = [torch.randint(0, vocab, (20,), generator=gen).tolist() for _ in range(3)]
    want = [plain.embedding(s, {k: v.double() for k, v in tables.items()}, cfg) for s in seqs]
    state = torch.full((6, 1), -7, dtype=torch.int32, device="cuda:0")
    state[4, 0] = seqs[1][9]                                  # request 1 has brought 10 tokens before
    t = {k: dev(v) for k, v in tables.items()}

    def step(q_len, before, source=None, previous=None):
        ctx = batch(q_len, before, [2, 4, 0])
        ids = [tok for s, n, c in zip(seqs, q_len, before) for tok in s[c: c + n]]
        ctx.token_ids = ints(ids if source is None else [0] * len(ids))
        got = ops.embed_pairs(ctx, t["embed"], t["bigram"], t["pos"], buckets, mp, mc, state, source=source, previous=previous)
        rows = torch.cat([w[c: c + n] for w, n, c in zip(want, q_len, before)])
        assert torch.allclose(got.cpu().double(), rows, atol=1e-5)

    step([5, 3, 1], [0, 10, 0])
    assert state[:, 0].tolist() == [seqs[2][0], -7, seqs[0][4], -7, seqs[1][12], -7]
    step([2, 1, 4], [5, 13, 1])
    fed = ints([seqs[1][14], 0, seqs[2][5], seqs[0][7]])      # ids that the step before "sampled", in another order
    step([1, 1, 1], [7, 14, 5], source=ints([3, 0, 2]), previous=fed)
    assert state[:, 0].tolist() == [seqs[2][5], -7, seqs[0][7], -7, seqs[1][14], -7]


def _memory_weights(gen, mode, c, heads, d, dv, rank=3):
    shapes = {"q": (heads * d, c), "k": (heads * d, c), "v": (heads * dv, c), "g": (heads * dv, c), "o": (c, heads * dv)}
    if mode == "gla":
        shapes.update({"norm": (dv,), "a1": (rank, c), "a2": (heads * d, rank), "a2.b": (heads * d,)})
    else:
        shapes.update({"norm": (heads * dv,), "i": (heads, c), "i.b": (heads,), "f": (heads, c), "f.b": (heads,)})
    w = {k: torch.randn(*s, generator=gen) / math.sqrt(s[-1] if len(s) > 1 else 1.0) for k, s in shapes.items()}
    return w


def _run_memory(ops, mode, t, w, h, m, cuts, slots, state, eps):
    """Projections in float64 on the host, the scan and the heads' norm and gate on the device, the output
    projection on the host again: the two kernels alone."""
    heads, d, dv = m["heads"], m["dim"], m["vdim"]
    wd = {k: v.double() for k, v in w.items()}
    outs = []
    for r, (hr, slot) in enumerate(zip(h, slots)):
        pos = 0
        for n in cuts[r]:
            x = hr[pos: pos + n].double()
            proj = torch.cat([x @ wd[k].T for k in ("q", "k", "v", "g")], dim=1)
            if mode == "gla":
                gates, const = (x @ wd["a1"].T) @ wd["a2"].T + wd["a2.b"], m["tau"]
            else:
                gates = torch.cat([x @ wd["i"].T + wd["i.b"], x @ wd["f"].T + wd["f.b"]], dim=1)
                const = m["gate_cap"]
            ctx = batch([n], [pos], [slot])
            p = dev(proj, t)
            o, aux = ops.matrix_memory_scan(ctx, mode, p, 0, heads * d, 2 * heads * d, heads, d, dv, dev(gates.float()),
                                            const, state)
            y = ops.head_norm_gate(o, aux, p[:, 2 * heads * d + heads * dv:], dev(w["norm"]), heads, dv, eps,
                                   mode == "mlstm", "sigmoid" if mode == "mlstm" else "silu", t, positions=ctx.positions)
            outs.append((r, y.double().cpu() @ wd["o"].T))
            pos += n
    return [torch.cat([o for rr, o in outs if rr == r]) for r in range(len(h))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode", ["gla", "mlstm"])
@pytest.mark.parametrize("heads,d,dv", [(2, 24, 40), (1, 8, 33), (3, 80, 96), (2, 128, 64), (1, 200, 16)])
def test_matrix_memory_prompt_portions_and_single_tokens(ops, dtype, mode, heads, d, dv):
    """Two sequences against the plain mixer: whole, in portions down to two tokens, token by token; the state
    slots start as NaN (a fresh request must not read them) and are used again by the next cutting."""
    t, c, eps = DTYPES[dtype], 48, 1e-4
    gen = torch.Generator().manual_seed(d + dv)
    m = {"heads": heads, "dim": d, "vdim": dv, "tau": 6.0, "gate_cap": 8.0}
    w = _memory_weights(gen, mode, c, heads, d, dv)
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    h = [torch.randn(n, c, generator=gen) for n in (75, 18)]
    mixer = plain.gla_mixer if mode == "gla" else plain.mlstm_mixer
    want = [mixer(x.double(), {k: v.double() for k, v in w.items()}, "", m, eps) for x in h]
    cols = dv + (1 if mode == "mlstm" else 0)
    state = torch.full((5, heads * cols * d + heads), float("nan"), device="cuda:0")
    for cuts in ([[75], [18]], [[40, 2, 17, 1, 15], [2, 16]], [[1] * 75, [1] * 18]):
        got = _run_memory(ops, mode, t, w, h, m, cuts, [3, 1], state, eps)
        for g, x in zip(got, want):
            close(g, x, dtype, f"{mode} cut as {cuts[0][:3]}", 4.0 if dtype == "bfloat16" else 3.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mode,strong", [("gla", False), ("gla", True), ("mlstm", False), ("mlstm", True)])
@pytest.mark.parametrize("heads,d,dv", [(2, 24, 40), (1, 8, 33), (2, 64, 128), (1, 128, 200), (1, 200, 16)])
def test_matrix_memory_chunk_by_chunk(ops, dtype, mode, strong, heads, d, dv):
    """The chunked form that serves prompt portions, against the plain mixer: three requests of unequal
    lengths in one step (chunks that are full, partial and of one token), then two more steps that go on
    from the state slots the one before left; the work list is made by the kernel set's own planner.  The
    kernels take 32-bit rows too (the engine gives them bfloat16 steps only), which is the sharp comparison.
    ``strong``: decays and gates so strong that a chunk's first token is forgotten many times over by its
    end, which must not overflow anything."""
    if strong and mode == "mlstm" and dtype == "bfloat16":
        pytest.skip("gates of e^40: one token owns the memory, and where the query is at right angles to its key the "
                    "rounding of bfloat16 inputs is all that is left of the read-out; the 32-bit rows are the test")
    t, c, eps = DTYPES[dtype], 48, 1e-4
    gen = torch.Generator().manual_seed(d + dv + heads)
    m = {"heads": heads, "dim": d, "vdim": dv, "tau": 0.5 if strong else 6.0, "gate_cap": 40.0 if strong else 8.0}
    w = _memory_weights(gen, mode, c, heads, d, dv)
    if strong and mode == "gla":
        w["a2.b"] = w["a2.b"] - 6.0
    if strong and mode == "mlstm":
        w["i"], w["f"], w["f.b"] = w["i"] * 40.0, w["f"] * 20.0, w["f.b"] - 10.0
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    wd = {k: v.double() for k, v in w.items()}
    h = [torch.randn(n, c, generator=gen) for n in (150, 70, 60)]
    mixer = plain.gla_mixer if mode == "gla" else plain.mlstm_mixer
    want = [mixer(x.double(), wd, "", m, eps) for x in h]
    cols = dv + (1 if mode == "mlstm" else 0)
    state = torch.full((5, heads * cols * d + heads), float("nan"), device="cuda:0")
    got = [[], [], []]
    # (the second and third step: a single token beside a long portion, each way round)
    for portions, before in (([100, 70, 5], [0, 0, 0]), ([49, 0, 1], [100, 70, 5]), ([1, 0, 54], [149, 70, 6])):
        live = [r for r in range(3) if portions[r]]
        x = torch.cat([h[r][before[r]: before[r] + portions[r]] for r in live]).double()
        proj = dev(torch.cat([x @ wd[k].T for k in ("q", "k", "v", "g")], dim=1), t)
        if mode == "gla":
            gates, const = (x @ wd["a1"].T) @ wd["a2"].T + wd["a2.b"], m["tau"]
        else:
            gates, const = torch.cat([x @ wd["i"].T + wd["i.b"], x @ wd["f"].T + wd["f.b"]], dim=1), m["gate_cap"]
        ctx = batch([portions[r] for r in live], [before[r] for r in live], [[3, 0, 4][r] for r in live])
        plan = SimpleNamespace(arrays={}, signature=[])
        ops.plan_memory_chunks(SimpleNamespace(q_len=[portions[r] for r in live], act_dtype=torch.bfloat16), plan, d, dv,
                               mode == "mlstm")
        assert len(plan.arrays) == 2 and plan.signature
        ctx.extra = {k: dev(torch.from_numpy(v)) for k, v in plan.arrays.items()}
        launches = ops.launches
        o, aux = ops.matrix_memory_scan(ctx, mode, proj, 0, heads * d, 2 * heads * d, heads, d, dv, dev(gates.float()),
                                        const, state)
        assert ops.launches == launches + 3                       # the three kernels of the chunked form ran
        y = ops.head_norm_gate(o, aux, proj[:, 2 * heads * d + heads * dv:], dev(w["norm"]), heads, dv, eps,
                               mode == "mlstm", "sigmoid" if mode == "mlstm" else "silu", t, positions=ctx.positions)
        y = y.double().cpu() @ wd["o"].T
        row = 0
        for r in live:
            got[r].append(y[row: row + portions[r]])
            row += portions[r]
    for r in range(3):
        close(torch.cat(got[r]), want[r], dtype, f"{mode} chunk by chunk, request {r}", 5.0)


def test_matrix_memory_keeps_a_far_token(ops):
    """Decays close to one: after 600 tokens the read-out still leans on token 3, whose key the last query
    repeats, thirty times as long as any other.  A state that is reset, cut off or decayed wrongly loses it."""
    gen = torch.Generator().manual_seed(11)
    heads, d, dv, n = 2, 32, 32, 600
    q, k = (torch.randn(n, heads * d, generator=gen) for _ in range(2))
    v = torch.randn(n, heads * dv, generator=gen)
    k[3] *= 30.0
    q[-1] = k[3]
    proj = torch.cat([q, k, v], dim=1)
    z = torch.full((n, heads * d), 9.0)                       # sigmoid(9) ** (1 / 4): a decay of 0.99997 a token
    state = torch.zeros(2, heads * dv * d, device="cuda:0")
    outs = []
    for cuts in ([n], [64] * 9 + [24], [300] + [1] * 300):
        pos, last = 0, None
        for c in cuts:
            ctx = batch([c], [pos], [1])
            last, _ = ops.matrix_memory_scan(ctx, "gla", dev(proj[pos: pos + c]), 0, heads * d, 2 * heads * d, heads, d, dv,
                                             dev(z[pos: pos + c]), 4.0, state)
            pos += c
        outs.append(last[-1].cpu())
    decay = math.exp(-math.log1p(math.exp(-9.0)) / 4.0)
    want = torch.zeros(heads, dv, dtype=torch.float64)
    qs = q[-1].double().view(heads, d) / math.sqrt(d)
    for j in range(n):
        want += (qs * k[j].double().view(heads, d)).sum(-1, keepdim=True) * decay ** (n - 1 - j) * v[j].double().view(heads, dv)
    from_far = ((qs * k[3].double().view(heads, d)).sum(-1, keepdim=True) * decay ** (n - 4) * v[3].double().view(heads, dv))
    assert from_far.abs().mean() > 3 * (want - from_far).abs().mean()      # the far token dominates the read-out
    for o in outs:
        assert torch.allclose(o.double(), want.reshape(-1), rtol=2e-4, atol=2e-2)


@pytest.mark.parametrize("dtype,path", [("float32", "general"), ("bfloat16", "general"), ("bfloat16", "tensor cores")])
@pytest.mark.parametrize("heads,groups,d,block,pt", [(6, 2, 16, 8, 8), (3, 3, 32, 16, 16), (5, 1, 24, 23, 4),
                                                     (8, 4, 64, 64, 16), (4, 2, 128, 100, 32)])
def test_attention_blocks_slopes_and_raw_values(ops, dtype, path, heads, groups, d, block, pt):
    """The attention mixer's middle (norms with gains, cache write, scores with the distance bias inside the
    query's block, values that are the raw keys) on scattered pages against the plain mixer, with a scale
    that makes every softmax lean on one or two keys: a key just outside a block that is let in, one just
    inside that is lost, or a slope of another head moves rows by far more than any rounding.  A prompt of
    several blocks, then single tokens across a block's edge."""
    t, c, eps = DTYPES[dtype], 40, 1e-4
    gen = torch.Generator().manual_seed(block)
    m = {"heads": heads, "kv_heads": groups, "dim": d, "vdim": d, "scale": (9.0 if dtype == "float32" else 4.0) / math.sqrt(d),
         "mask": {"size": block}}
    shapes = {"q": (heads * d, c), "q.b": (heads * d,), "k": (groups * d, c), "k.b": (groups * d,), "q.norm": (d,),
              "k.norm": (d,), "o": (c, heads * d), "o.b": (c,)}
    w = {k: torch.randn(*s, generator=gen) / math.sqrt(s[-1] if len(s) > 1 else 4.0) for k, s in shapes.items()}
    w["q.norm"], w["k.norm"] = 1.0 + w["q.norm"], 1.0 + w["k.norm"]
    n_prompt, n_total = 2 * block + block // 2 + 1, 3 * block + 3
    h = torch.randn(n_total, c, generator=gen)
    wd = {k: v.double() for k, v in w.items()}
    want = plain.attention_mixer(h.double(), wd, "", m, eps)
    pages = -(-n_total // pt)
    order = torch.randperm(pages + 3, generator=gen).tolist()
    k_pages = torch.full((pages + 3, groups, pt, d), float("nan"), dtype=t, device="cuda:0")
    v_pages = torch.full((pages + 3, groups, pt, d), float("nan"), dtype=t, device="cuda:0")
    cache = PagedKVView(k_pages, v_pages, 0, pt, None, True)
    slopes = dev(torch.tensor([2.0 ** (-8.0 * (a + 1) / heads) for a in range(heads)], dtype=torch.float32))
    ops.use_mma_attention = path == "tensor cores"
    try:
        outs, pos = [], 0
        for n in [n_prompt] + [1] * (n_total - n_prompt):
            x = h[pos: pos + n].double()
            proj = dev(torch.cat([x @ wd["q"].T + wd["q.b"], x @ wd["k"].T + wd["k.b"]], dim=1), t)
            ctx = batch([n], [pos], [0], tables=[order[:pages]])
            slots = ints([order[p // pt] * pt + p % pt for p in range(pos, pos + n)])
            ops.head_prepare(proj, heads, groups, d, d, 0, heads * d, heads * d, True, eps, cache, slots, ctx.positions,
                             q_gain=dev(w["q.norm"]), k_gain=dev(w["k.norm"]))
            out = ops.paged_attention_general(proj, heads, groups, d, d, m["scale"], cache, ctx, slopes=slopes, block=block)
            outs.append(out.double().cpu() @ wd["o"].T + wd["o.b"])
            pos += n
    finally:
        ops.use_mma_attention = True
    got = torch.cat(outs)
    err = (got - want).abs().amax(-1) / want.abs().amax(-1)
    assert float(err.max()) < (1e-4 if dtype == "float32" else 6e-2), f"row {int(err.argmax())}: {float(err.max()):.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,groups,scoring", [(6, 2, (3, 2), "sigmoid"), (4, 1, (1, 1), "sigmoid"),
                                                        (40, 6, (8, 3), "sigmoid"), (5, 3, None, "sigmoid"),
                                                        (12, 4, (12, 5), "sigmoid"), (8, 2, (4, 2), "softmax_top")])
def test_scored_router(ops, dtype, experts, top, groups, scoring):
    gen = torch.Generator().manual_seed(experts)
    n, c = 33, 48
    y = torch.randn(n, c, generator=gen).to(DTYPES[dtype])
    router, corr = torch.randn(experts, c, generator=gen) / 3.0, 0.5 * torch.randn(experts, generator=gen)
    positions = torch.arange(n, dtype=torch.int32)
    positions[7] = -1
    ids, weights, gate = ops.moe_route_scored(dev(y), dev(router), None, dev(positions), top, scoring, dev(corr), groups, 1.9)
    assert gate is None and ids[7].tolist() == [-1] * top
    r = {"experts": experts, "top": top, "scale": 1.9}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    if scoring == "sigmoid":
        want_ids, want_w = plain.route(y.double(), {"router": router.double(), "correction": corr.double()}, "", r)
    else:                                                     # the same choice over the logits themselves
        z = y.double() @ router.double().T
        choice = z + corr.double()
        per = experts // groups[0]
        score = choice.view(n, groups[0], per).topk(2, dim=-1).values.sum(-1)
        allowed = torch.zeros(n, groups[0], dtype=torch.bool).scatter_(1, score.topk(groups[1], dim=-1).indices, True)
        choice = choice.view(n, groups[0], per).masked_fill(~allowed[:, :, None], -math.inf).reshape(n, experts)
        want_ids = choice.topk(top, dim=-1).indices
        want_w = 1.9 * torch.softmax(z.gather(1, want_ids), dim=-1)
    live = positions >= 0
    assert torch.equal(ids.cpu().long()[live], want_ids[live])
    assert torch.allclose(weights.cpu().double()[live], want_w[live], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,ff,shared,c", [(6, 2, 24, 40, 64), (3, 3, 20, None, 72), (9, 1, 64, 8, 40)])
def test_clamped_experts_with_a_shared_one(ops, dtype, experts, top, ff, shared, c):
    """Router, grouped products with the clamped gate, combine and the shared expert against the plain
    feed-forward; activations large enough that both clamps act on many features."""
    t = DTYPES[dtype]
    gen = torch.Generator().manual_seed(ff)
    f = {"kind": "moe", "expert": {"ff": ff, "limit": 0.8}, "router": {"experts": experts, "top": top, "scale": 1.4}}
    w = {"router": torch.randn(experts, c, generator=gen) / 4.0, "correction": 0.3 * torch.randn(experts, generator=gen)}
    units = [(f"e{j}.", ff) for j in range(experts)]
    if shared:
        f["shared"] = {"ff": shared, "limit": 1.1}
        units.append(("shared.", shared))
    for p, width in units:
        w[p + "gate"], w[p + "up"] = (torch.randn(width, c, generator=gen) / 3.0 for _ in range(2))
        w[p + "down"] = torch.randn(c, width, generator=gen) / math.sqrt(width)
    if dtype == "bfloat16":
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    y = torch.randn(21, c, generator=gen).to(t)
    want = plain.routed_ff(y.double(), {k: v.double() for k, v in w.items()}, "", f)
    hidden = plain.clamped_expert(y.double(), {k: v.double() for k, v in w.items()}, "e0.", 1e9)
    assert float((y.double() @ w["e0.gate"].double().T > 0.8).double().mean()) > 0.1 and hidden.abs().max() > 1.0
    ids, weights, _ = ops.moe_route_scored(dev(y), dev(w["router"]), None, None, top, "sigmoid", dev(w["correction"]), None, 1.4)
    residual = torch.zeros(21, c, device="cuda:0")
    w_in = dev(torch.stack([torch.cat([w[f"e{j}.gate"], w[f"e{j}.up"]]) for j in range(experts)]), t)
    w_out = dev(torch.stack([w[f"e{j}.down"] for j in range(experts)]), t)
    ops.moe_experts_residual(dev(y), ids, weights, w_in, w_out, residual, activation="clamped_swish", limit=0.8)
    if shared:
        both = ops.linear(dev(y), dev(torch.cat([w["shared.gate"], w["shared.up"]]), t), None, "none", t)
        ops.linear_residual(ops.glu(both, activation="clamped_swish", limit=1.1), dev(w["shared.down"], t), None, residual)
    close(residual, want, dtype, "clamped experts", 3.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_gated_gelu_unit_and_pass_entry(ops, dtype):
    t = DTYPES[dtype]
    gen = torch.Generator().manual_seed(2)
    c, ff, n = 56, 88, 19
    w = {"gate": torch.randn(ff, c, generator=gen) / 4, "up": torch.randn(ff, c, generator=gen) / 4,
         "down": torch.randn(c, ff, generator=gen) / 8, "loop.in": torch.randn(c, 2 * c, generator=gen) / 8,
         "loop.step": torch.randn(3, c, generator=gen)}
    if dtype == "bfloat16":
        w = {k: (v.to(torch.bfloat16).float() if k != "loop.step" else v) for k, v in w.items()}
    y, x, x0 = (torch.randn(n, c, generator=gen) for _ in range(3))
    wd = {k: v.double() for k, v in w.items()}
    both = ops.linear(dev(y, t), dev(torch.cat([w["gate"], w["up"]]), t), None, "none", t)
    residual = torch.zeros(n, c, device="cuda:0")
    ops.linear_residual(ops.glu(both, activation="gelu_tanh"), dev(w["down"], t), None, residual)
    close(residual, plain.dense_ff(y.to(t).double(), wd, ""), dtype, "gated gelu unit")
    joined = ops.concat_cast(dev(x), dev(x0), t)
    got = ops.linear(joined, dev(w["loop.in"], t), dev(w["loop.step"])[2], "none", torch.float32)
    close(got, plain.pass_entry(x.to(t).double(), x0.to(t).double(), wd, 2), dtype, "pass entry")


# ---- the step function --------------------------------------------------------------------------
CASES = [(w, d) for w in "ABCDEF" for d in ("float32", "bfloat16")]
IDS = [f"{w}-{d}" for w, d in CASES]


def setup(which, dtype, num_pages=64, seed=3, max_requests=4):
    from mini_gpt_inference_b200.kernels.ops import default_ops

    raw = config(which, every_expert=dtype == "bfloat16")
    # (sharp softmaxes in 32-bit, where nothing but the order of sums differs; in bfloat16 they would magnify
    # the rounding of queries and keys)
    tensors = random_weights(raw, seed, sharp=3.0 if dtype == "float32" else 1.0, as_bfloat16=dtype == "bfloat16")
    loaded = load_model(config=ZenedraConfig.from_dict(raw), tensors=tensors, dtype=dtype, device="cuda:0")
    runner = make_runner(loaded, default_ops("cuda:0"), PAGE_TOKENS[which], num_pages, max_requests)
    return raw, tensors, runner, (TOL[dtype], 0.03 if dtype == "bfloat16" else 0.0)


@pytest.mark.parametrize("which,dtype", CASES, ids=IDS)
def test_whole_prompts(which, dtype):
    raw, tensors, runner, tol = setup(which, dtype, num_pages=100)
    pt = PAGE_TOKENS[which]
    longest = min(190, raw["max_positions"])
    for length, seed in [(150, 1), (37, 2), (1, 3), (2, 4), (pt + 1, 5), (pt, 6), (longest, 7)]:
        tokens = tokens_for(raw, length, seed)
        got = runner.step([StepEntry("r", tokens, list(range(length)))])
        runner.finish("r")
        assert got.shape == (length, raw["vocab"]) and got.dtype == torch.float32
        assert_rows_close(got, plain_logits(raw, tensors, tokens), tol[0], f"whole prompt of {length}", outliers=tol[1])
    runner.manager.check()
    assert runner.manager.stats()["allocated_blocks"] == 0


@pytest.mark.parametrize("which,dtype", CASES, ids=IDS)
def test_prefill_then_single_tokens(which, dtype):
    """A short prompt, then a long run of single tokens (replayed from a CUDA graph) across several blocks
    of the attention's mask, and the same sequence token by token from the very first token."""
    raw, tensors, runner, tol = setup(which, dtype)
    tokens = tokens_for(raw, 150, 7)
    want = plain_logits(raw, tensors, tokens)
    outs = [runner.step([StepEntry("r", tokens[:9], list(range(9)))])]
    outs += [runner.step([StepEntry("r", tokens[t: t + 1], [0])]) for t in range(9, 150)]
    assert_rows_close(torch.cat(outs), want, tol[0], "prefill then single tokens", outliers=tol[1])
    assert runner.graph_replays > 100
    one_by_one = torch.cat([runner.step([StepEntry("s", tokens[t: t + 1], [0])]) for t in range(40)])
    assert_rows_close(one_by_one, want[:40], tol[0], "single tokens from the first", outliers=tol[1])
    if dtype == "float32":
        # in 32-bit the cut into steps changes no bit
        assert torch.equal(one_by_one, torch.cat(outs)[:40])


@pytest.mark.parametrize("which,dtype", CASES, ids=IDS)
def test_portions_of_changing_size(which, dtype):
    raw, tensors, runner, tol = setup(which, dtype)
    tokens = tokens_for(raw, 131, 8)
    want = plain_logits(raw, tensors, tokens)
    sizes = itertools.cycle([13, 7, 2, 5, 2, 1, 3, 16, 2, 9, 33])
    outs, pos = [], 0
    while pos < len(tokens):
        n = min(next(sizes), len(tokens) - pos)
        outs.append(runner.step([StepEntry("r", tokens[pos: pos + n], list(range(n)))]))
        pos += n
    assert_rows_close(torch.cat(outs), want, tol[0], "portions of changing size", outliers=tol[1])


@pytest.mark.parametrize("which,dtype", CASES, ids=IDS)
def test_mixed_batches_reuse_pages_and_slots(which, dtype):
    """Up to four live requests, portions of some beside single tokens of others, requests left out of
    steps; pages and state slots are handed out again.  Every cache row and state slot starts as NaN and
    turns NaN again when its request ends."""
    pt = PAGE_TOKENS[which]
    lengths = [90, 29, 71, 3, 41, 2 * pt, 17, 55, 1]
    pool = sum(sorted(-(-n // pt) for n in lengths)[-4:])
    raw, tensors, runner, tol = setup(which, dtype, num_pages=pool)
    for pages in runner.storage.k + runner.storage.v:
        pages.fill_(float("nan"))
    for state in runner.storage.state.values():
        state.fill_(float("nan") if state.is_floating_point() else -1)
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
                held = runner.manager.get(rid)
                tables, slot = [list(t) for t in held.tables], held.state_slot
                runner.finish(rid)
                del live[rid]
                for g, table in enumerate(tables):
                    for page in table:
                        if page >= 0:
                            runner.storage.k[g][:, page] = float("nan")
                            runner.storage.v[g][:, page] = float("nan")
                for state in runner.storage.state.values():
                    state[slot] = float("nan") if state.is_floating_point() else -1
    for rid in reqs:
        assert_rows_close(torch.cat(got[rid]), want[rid], tol[0], f"request {rid} in mixed batches", outliers=tol[1])
    runner.manager.check()
    assert runner.manager.stats()["allocated_blocks"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batch_of_unequal_requests_equals_each_alone(dtype):
    raw, tensors, runner, tol = setup("A", dtype, num_pages=64, max_requests=8)
    prompts = [tokens_for(raw, n, 70 + n) for n in (1, 2, 33, 64, 7)]
    alone = []
    for i, p in enumerate(prompts):
        alone.append(runner.step([StepEntry(f"a{i}", p, list(range(len(p))))]))
        runner.finish(f"a{i}")
    together = runner.step([StepEntry(f"b{i}", p, list(range(len(p)))) for i, p in enumerate(prompts)])
    if dtype == "float32":
        assert torch.equal(together, torch.cat(alone))
    else:
        assert float(relative_error(together, torch.cat(alone).cpu()).max()) < tol[0]


# ---- generation through the entry point, its scheduler and sampler ---------------------------------
@pytest.mark.parametrize("which", "ABC")
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine(which, dtype):
    raw = config(which, every_expert=dtype == "bfloat16")
    tensors = random_weights(raw, 11, as_bfloat16=dtype == "bfloat16")
    loaded = load_model(config=ZenedraConfig.from_dict(raw), tensors=tensors, dtype=dtype, device="cuda:0")
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


def test_preemption_and_recompute_through_the_engine():
    """A pool too small for the three running requests (the attention's block made longer than any sequence, so
    that no page comes back early): requests are preempted, give back their pages and state slot, and are
    computed again from their first token in a slot that another request used meanwhile."""
    raw = config("A")
    raw["layers"][1]["mixer"]["mask"]["size"] = 1000
    tensors = random_weights(raw, 14)
    loaded = load_model(config=ZenedraConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cuda:0")
    engine = LLMEngine(loaded, EngineConfig(dtype="float32", block_size=8, num_blocks=10, max_batch_size=3,
                                            max_num_batched_tokens=16, max_prefill_chunk=7))
    prompts = [tokens_for(raw, n, 60 + i) for i, n in enumerate([20, 25, 18, 9])]
    outs = engine.generate(prompts, SamplingParams(max_tokens=16, temperature=0.0))
    assert engine.scheduler.num_preemptions > 0
    for prompt, out in zip(prompts, outs):
        assert out["token_ids"] == plain_greedy(raw, tensors, prompt, 16)
    assert engine.stats()["allocated_blocks"] == 0
    engine.runner.manager.check()


def test_long_decoding_through_the_engine():
    raw = config("B")
    tensors = random_weights(raw, 12)
    loaded = load_model(config=ZenedraConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cuda:0")
    engine = LLMEngine(loaded, EngineConfig(dtype="float32", block_size=8, num_blocks=40, max_batch_size=2))
    prompt = tokens_for(raw, 3, 9)
    out = engine.generate([prompt], SamplingParams(max_tokens=200, temperature=0.0))[0]
    assert out["token_ids"] == plain_greedy(raw, tensors, prompt, 200)


def test_trace_replay(tmp_path):
    """The replay program on a model folder: two requests, portions beside single tokens, a slot and pages
    used again by a third request."""
    from mini_gpt_inference_b200.engine.trace import main
    from mini_gpt_inference_b200.weights.safetensors_io import save_file

    raw = config("A")
    tensors = random_weights(raw, 13, as_bfloat16=True)
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(raw))
    save_file({k: v.to(torch.bfloat16) for k, v in tensors.items()}, folder / "model.safetensors")
    a, b, c = tokens_for(raw, 50, 1), tokens_for(raw, 20, 2), tokens_for(raw, 64, 3)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[:7], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[7:], "want": [12]}, {"id": "a", "tokens": a[31:], "want": [18]}], "end": ["a", "b"]},
        {"step": 3, "entries": [{"id": "c", "tokens": c[:62], "want": [61]}], "end": []},
        {"step": 4, "entries": [{"id": "c", "tokens": c[62:], "want": [0, 1]}], "end": ["c"]},
    ]
    for dtype in ("float32", "bfloat16"):
        if dtype == "bfloat16":                              # (see zenedra_cases.config on every_expert)
            raw = config("A", every_expert=True)
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
    """bin/generate: a random-weights folder from a config.json, then greedy tokens from it that equal the
    plain implementation's on the folder's own tensors."""
    import subprocess
    import sys
    from pathlib import Path

    from mini_gpt_inference_b200.weights import load_file

    root = Path(__file__).resolve().parent.parent
    raw = config("D")
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


@pytest.mark.parametrize("rows,width,out", [(1, 64, 96), (8, 320, 200), (16, 1024, 512), (5, 1600, 3200), (3, 72, 40), (40, 128, 64)])
def test_rms_norm_inside_the_projections(ops, rows, width, out):
    """The RMS norm as the prologue of the small-batch projection kernels (and, where they refuse, as a kernel
    of its own in front) against norm then product in float64; rows gathered first, as the head does."""
    gen = torch.Generator().manual_seed(width + rows)
    x = 2 * torch.randn(rows + 3, width, generator=gen)
    w, weight = 0.3 * torch.randn(width, generator=gen), torch.randn(out, width, generator=gen) / math.sqrt(width)
    weight = weight.to(torch.bfloat16)
    pick = torch.randperm(rows + 3, generator=gen)[:rows].to(torch.int32)
    want = plain.rms_norm(x[pick.long()].double(), w.double(), 1e-4, 1.0).to(torch.bfloat16).double() @ weight.double().T
    for rows_arg, xin in ((dev(pick), dev(x)), (None, dev(x[pick.long()]))):
        y = ops.defer_rmsnorm(xin, dev(w), 1e-4, 1.0, torch.bfloat16, rows_arg)
        got = ops.linear(y, dev(weight), None, "none", torch.float32)
        close(got, want, "bfloat16", "rms norm inside a projection", 0.5)
