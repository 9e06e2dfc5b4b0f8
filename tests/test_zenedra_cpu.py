"""Zenedra without a GPU: the plain implementation's mechanisms against restatements by hand, the
configuration and the loader, and the model through the step function, the cache manager, the scheduler
and the entry point with the torch test double in place of the CUDA kernel set."""

from __future__ import annotations

import itertools
import json
import math

import pytest
import torch

import plain_zenedra as pz
from torch_ops import TorchOps
from zenedra_cases import (PAGE_TOKENS, assert_rows_close, config, plain_greedy, plain_logits, random_weights,
                           tokens_for)

from mini_gpt_inference_b200 import EngineConfig, LLMEngine, SamplingParams, ZenedraConfig
from mini_gpt_inference_b200.cache.manager import CacheManager
from mini_gpt_inference_b200.cache.spec import PagedKVSpec
from mini_gpt_inference_b200.config import ConfigError, lookup
from mini_gpt_inference_b200.engine.build import load_model, make_runner
from mini_gpt_inference_b200.engine.runner import StepEntry
from mini_gpt_inference_b200.parts import DecoderModel
from mini_gpt_inference_b200.weights import WeightsError, check_and_bind, load_file, write_random_model


# ---- the plain mechanisms against restatements by hand ---------------------------------------------------
def test_pair_rows_and_run_order():
    assert pz.bigram_rows([5, 7, 7, 2], 10, 3, 4) == [10, (5 * 3 + 7 * 4) % 10, (7 * 3 + 7 * 4) % 10, (7 * 3 + 2 * 4) % 10]
    raw = config("D")
    assert [(i, p) for i, p, _ in pz.run_order(raw)] == [(0, None), (1, 0), (1, 1), (1, 2), (2, None)]
    assert [b for _, _, b in pz.run_order(raw)] == [False, True, True, True, False]
    assert [b for _, _, b in pz.run_order(config("A"))] == [True, False, True, False, False]
    assert ZenedraConfig.from_dict(raw).run_order() == [(i, p) for i, p, _ in pz.run_order(raw)]


def test_gla_is_a_decayed_sum_over_the_past():
    torch.manual_seed(0)
    T, c, m = 9, 12, {"heads": 2, "dim": 3, "vdim": 5, "tau": 4.0}
    w = {"q": torch.randn(6, c), "k": torch.randn(6, c), "v": torch.randn(10, c), "g": torch.randn(10, c),
         "o": torch.randn(c, 10), "norm": torch.randn(5), "a1": torch.randn(2, c), "a2": torch.randn(6, 2),
         "a2.b": torch.randn(6)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, c, dtype=torch.float64)
    got = pz.gla_mixer(h, w, "", m, 1e-5)
    q = (h @ w["q"].T).view(T, 2, 3) / math.sqrt(3)
    k, v = (h @ w["k"].T).view(T, 2, 3), (h @ w["v"].T).view(T, 2, 5)
    la = (torch.nn.functional.logsigmoid((h @ w["a1"].T) @ w["a2"].T + w["a2.b"]) / 4.0).view(T, 2, 3)
    o = torch.zeros(T, 2, 5, dtype=torch.float64)
    for t in range(T):
        for j in range(t + 1):
            decay = torch.exp(la[j + 1: t + 1].sum(0))                  # [heads, dim]: what key j has lost by time t
            o[t] += ((q[t] * decay * k[j]).sum(-1))[:, None] * v[j]
    o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5) * w["norm"]
    g = h @ w["g"].T
    want = (o.reshape(T, 10) * g * torch.sigmoid(g)) @ w["o"].T
    assert torch.allclose(got, want, atol=1e-10)


def test_mlstm_equals_the_unstabilised_recurrence_where_the_floor_is_idle():
    torch.manual_seed(1)
    T, c, m = 7, 10, {"heads": 2, "dim": 4, "vdim": 3, "gate_cap": 6.0}
    w = {k: torch.randn(*s).double() for k, s in
         {"q": (8, c), "k": (8, c), "v": (6, c), "g": (6, c), "o": (c, 6), "norm": (6,), "i": (2, c), "i.b": (2,),
          "f": (2, c), "f.b": (2,)}.items()}
    h = torch.randn(T, c, dtype=torch.float64)
    got = pz.mlstm_mixer(h, w, "", m, 1e-5)
    q, k = (h @ w["q"].T).view(T, 2, 4) / 2.0, (h @ w["k"].T).view(T, 2, 4)
    v = (h @ w["v"].T).view(T, 2, 3)
    gi = 6.0 * torch.tanh((h @ w["i"].T + w["i.b"]) / 6.0)
    gf = torch.nn.functional.logsigmoid(6.0 * torch.tanh((h @ w["f"].T + w["f.b"]) / 6.0))
    S, n = torch.zeros(2, 4, 3, dtype=torch.float64), torch.zeros(2, 4, dtype=torch.float64)
    mx = torch.zeros(2, dtype=torch.float64)
    o = torch.zeros(T, 2, 3, dtype=torch.float64)
    for t in range(T):
        S = torch.exp(gf[t])[:, None, None] * S + torch.exp(gi[t])[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = torch.exp(gf[t])[:, None] * n + torch.exp(gi[t])[:, None] * k[t]
        mx = torch.maximum(gf[t] + mx, gi[t])
        # the true-scale denominator: max(|n . q|, 1) in true scale, plus the small constant at the stabilised scale
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.ones(2, dtype=torch.float64)) + 1e-6 * torch.exp(mx)
        o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    o = (o / torch.sqrt((o * o).mean(-1, keepdim=True) + 1e-5)).reshape(T, 6) * w["norm"]
    want = (o * torch.sigmoid(h @ w["g"].T)) @ w["o"].T
    assert torch.allclose(got, want, atol=1e-9)


def test_attention_sees_its_own_block_only_and_values_are_raw_keys():
    torch.manual_seed(2)
    T, c = 11, 8
    m = {"heads": 2, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 0.7, "mask": {"size": 4}}
    w = {k: torch.randn(*s).double() for k, s in
         {"q": (8, c), "q.b": (8,), "k": (4, c), "k.b": (4,), "q.norm": (4,), "k.norm": (4,), "o": (c, 8), "o.b": (c,)}.items()}
    h = torch.randn(T, c, dtype=torch.float64)
    got = pz.attention_mixer(h, w, "", m, 1e-5)
    # a key outside the query's block does not matter, however large it is
    h2 = h.clone()
    h2[3] *= 50.0
    again = pz.attention_mixer(h2, w, "", m, 1e-5)
    assert torch.allclose(got[4:], again[4:], atol=1e-12) and not torch.allclose(got[3], again[3])
    # the first position of a block attends to itself alone: its output is its own raw key through W_o
    k = h @ w["k"].T + w["k.b"]
    for t in (0, 4, 8):
        assert torch.allclose(got[t], torch.cat([k[t], k[t]]) @ w["o"].T + w["o.b"], atol=1e-10)
    # the distance bias by hand at one position
    qn = pz.rms_norm((h @ w["q"].T + w["q.b"]).view(T, 2, 4), w["q.norm"], 1e-5)
    kn = pz.rms_norm(k, w["k.norm"], 1e-5)
    t, out = 6, []
    for a in range(2):
        s = torch.stack([0.7 * (qn[t, a] @ kn[j]) - 2.0 ** (-8 * (a + 1) / 2) * (t - j) for j in (4, 5, 6)])
        out.append(torch.softmax(s, 0) @ k[4:7])
    assert torch.allclose(got[t], torch.cat(out) @ w["o"].T + w["o.b"], atol=1e-10)


def test_router_groups_correction_and_weights():
    r = {"experts": 6, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}}
    w = {"router": torch.eye(6, dtype=torch.float64), "correction": torch.tensor([0., 0., 0., 0., 5., 0.], dtype=torch.float64)}
    h = torch.tensor([[3.0, 2.95, 2.9, 2.8, -4.0, -4.0]], dtype=torch.float64)
    ids, weights = pz.route(h, w, "", r)
    # the correction lifts the last group (sigmoid(-4) + 5) above the others; its second expert is chosen too,
    # although four experts of other groups score higher, and the weights do not contain the correction
    assert ids.tolist() == [[4, 5]]
    assert torch.allclose(weights, 3.0 * torch.sigmoid(torch.tensor([[-4.0, -4.0]], dtype=torch.float64)))
    r["groups"] = {"count": 3, "keep": 3}
    assert pz.route(h, w, "", r)[0].tolist() == [[4, 0]]
    # negative choice scores still beat experts of groups that are not kept
    w["correction"] = torch.full((6,), -3.0, dtype=torch.float64)
    r["groups"] = {"count": 3, "keep": 1}
    assert sorted(pz.route(h, w, "", r)[0].tolist()[0]) == [0, 1]


def test_clamped_expert_by_hand():
    w = {"gate": torch.tensor([[1.0], [1.0]]).double(), "up": torch.tensor([[1.0], [-1.0]]).double(),
         "down": torch.tensor([[1.0, 0.0], [0.0, 1.0]]).double()}
    out = pz.clamped_expert(torch.tensor([[5.0]], dtype=torch.float64), w, "", 2.0)
    g = 2.0 / (1.0 + math.exp(-1.702 * 2.0))
    assert torch.allclose(out, torch.tensor([[g * 3.0, g * -1.0]], dtype=torch.float64))


# ---- configuration, registry, names, loader ------------------------------------------------------------------
@pytest.mark.parametrize("which", "ABCDEF")
def test_config_round_trip_and_names(which, tmp_path):
    raw = config(which)
    cfg = ZenedraConfig.from_dict(raw)
    assert ZenedraConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))) == cfg
    assert lookup("Zenedra").config_class is ZenedraConfig
    model = DecoderModel(lookup(cfg.architecture).describe(cfg))
    tensors = random_weights(raw, 1)
    specs = model.tensor_specs()
    needed = {k for k, v in specs.items() if not v.optional}
    assert needed == set(tensors)
    bound = check_and_bind(tensors, specs)                              # the decay matrices' inner size is the checkpoint's
    assert all(specs[k].fits(v.shape) for k, v in bound.items())
    assert len(model.cache_specs()) == len(pz.run_order(raw)) + 1       # one entry per layer run, one for the embedding
    folder = write_random_model(tmp_path / which, cfg, 3, "bfloat16")
    again = load_file(folder / "model.safetensors")
    assert set(again) == needed and cfg.num_parameters() > 0
    assert ZenedraConfig.from_json(folder) == cfg


def test_config_errors_and_loader_errors():
    raw = config("A")
    for breaker in (lambda r: r.pop("max_positions"), lambda r: r["layers"][0].update(type="conv"),
                    lambda r: r["layers"][1]["mixer"].update(vdim=8), lambda r: r["loop"].update(stop=9),
                    lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(count=4),
                    lambda r: r["layers"][1]["mlp"]["router"]["groups"].update(keep=0),
                    lambda r: r["layers"][2]["mixer"].pop("tau"), lambda r: r["embedding"]["bigram"].update(buckets=0)):
        broken = json.loads(json.dumps(raw))
        breaker(broken)
        with pytest.raises(ConfigError):
            ZenedraConfig.from_dict(broken)
    cfg = ZenedraConfig.from_dict(raw)
    tensors = random_weights(raw, 2)
    tensors["l2.mix.a2"] = tensors["l2.mix.a2"][:, :3].contiguous()     # inner sizes that disagree
    del tensors["l1.mlp.correction"]
    tensors["l0.mix.norm"] = tensors["l0.mix.norm"][:5]
    with pytest.raises(WeightsError) as err:
        load_model(config=cfg, tensors={k: v for k, v in tensors.items() if k != "l2.mix.a2"}, dtype="float32", device="cpu")
    assert "l1.mlp.correction" in str(err.value) and "l0.mix.norm" in str(err.value) and "l2.mix.a2" in str(err.value)
    tensors = random_weights(raw, 2)
    tensors["l2.mix.a2"] = tensors["l2.mix.a2"][:, :3].contiguous()
    with pytest.raises(ValueError, match="inner size"):
        load_model(config=cfg, tensors=tensors, dtype="float32", device="cpu")


def test_a_layer_without_a_feed_forward_may_still_carry_its_second_norm():
    raw = config("E")
    tensors = random_weights(raw, 6)
    assert "l1.norm2" not in tensors
    toks = tokens_for(raw, 12, 1)
    want = plain_logits(raw, tensors, toks)
    for extra in ({}, {"l1.norm2": torch.randn(raw["width"])}):
        loaded = load_model(config=ZenedraConfig.from_dict(raw), tensors={**tensors, **extra}, dtype="float32", device="cpu")
        runner = make_runner(loaded, TorchOps(), 8, 4, 2)
        assert_rows_close(runner.step([StepEntry("r", toks, list(range(12)))]), want, 2e-4, "with and without the norm")


def test_block_mask_gives_pages_back():
    m = CacheManager([PagedKVSpec(2, 8, block=12)], page_tokens=4, num_pages=8, max_requests=2)
    m.admit("a")
    assert m.reserve("a", 11)
    m.advance("a", 11)
    assert m.num_free_pages() == 5                  # positions 0..10: pages 0..2, all of the first block
    assert m.reserve("a", 13)
    m.advance("a", 13)                              # the next query is at 13, in block 12..23: pages 0..2 are over
    assert m.num_free_pages() == 7 and m.block_table("a", 0)[:3] == [-1, -1, -1]
    m.check()
    m.release("a")
    assert m.num_free_pages() == 8


# ---- the model through the step function on the test double ----------------------------------------------------
def cpu_runner(raw, tensors, page_tokens, num_pages, max_requests=4):
    loaded = load_model(config=ZenedraConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cpu")
    return make_runner(loaded, TorchOps(), page_tokens, num_pages, max_requests)


@pytest.mark.parametrize("which", "ABCEF")
def test_cuttings_agree_with_plain(which):
    raw = config(which)
    tensors = random_weights(raw, 3, sharp=3.0)
    pt = PAGE_TOKENS[which]
    lengths = {"a": 41, "b": 36, "c": 9, "d": 2 * pt + 1}
    runner = cpu_runner(raw, tensors, pt, sum(-(-n // pt) for n in lengths.values()))
    reqs = {k: tokens_for(raw, n, i) for i, (k, n) in enumerate(lengths.items())}
    want = {k: plain_logits(raw, tensors, v) for k, v in reqs.items()}
    got = {k: [] for k in reqs}
    pos = dict.fromkeys(reqs, 0)
    sizes = itertools.cycle([13, 1, 2, 7, 1, 1, 5, 2])
    while any(pos[k] < len(reqs[k]) for k in reqs):
        entries, order = [], []
        for k in reqs:
            if pos[k] == len(reqs[k]):
                continue
            m = min(next(sizes), len(reqs[k]) - pos[k])
            entries.append(StepEntry(k, reqs[k][pos[k]: pos[k] + m], list(range(m))))
            order.append((k, m))
            pos[k] += m
        out = runner.step(entries)
        row = 0
        for k, m in order:
            got[k].append(out[row: row + m])
            row += m
        runner.manager.check()
    for k in reqs:
        assert_rows_close(torch.cat(got[k]), want[k], 2e-4, f"request {k}")
        runner.finish(k)
    assert runner.manager.stats()["allocated_blocks"] == 0


def test_slots_and_pages_used_again():
    raw = config("A")
    tensors = random_weights(raw, 5)
    runner = cpu_runner(raw, tensors, 8, 6, max_requests=2)
    for n, name in enumerate(["p", "q", "r", "s", "t"]):                # five requests through two slots
        toks = tokens_for(raw, 17 + n, 40 + n)
        want = plain_logits(raw, tensors, toks)
        first = runner.step([StepEntry(name, toks[:9], list(range(9)))])
        rest = [runner.step([StepEntry(name, [t], [0])]) for t in toks[9:]]
        assert_rows_close(torch.cat([first] + rest), want, 2e-4, name)
        if n % 2 == 0:
            runner.finish(name)
        else:                                                           # two live at once, the older one ends later
            other = tokens_for(raw, 5, 90 + n)
            got = runner.step([StepEntry(name + "x", other, [4])])
            assert_rows_close(got, plain_logits(raw, tensors, other, [4]), 2e-4, name + "x")
            runner.finish(name)
            runner.finish(name + "x")
        runner.manager.check()


def test_generation_through_the_engine_on_the_double():
    raw = config("A")
    tensors = random_weights(raw, 4)
    loaded = load_model(config=ZenedraConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cpu")
    engine = LLMEngine(loaded, EngineConfig(dtype="float32", device="cpu", block_size=8, num_blocks=12, max_batch_size=2,
                                            max_num_batched_tokens=12, max_prefill_chunk=5), ops=TorchOps())
    prompts = [tokens_for(raw, n, 30 + n) for n in (7, 1, 18)]
    outs = engine.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0))
    for prompt, out in zip(prompts, outs):
        assert out["token_ids"] == plain_greedy(raw, tensors, prompt, 6)
    assert engine.stats()["allocated_blocks"] == 0
