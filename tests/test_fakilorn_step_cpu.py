"""Fakilorn through the step function, the cache manager, the scheduler and the entry point on the
CPU, with the torch test double in place of the CUDA kernel set (the product has no CPU path): the
wiring of the parts, the published values, the page tables of several cache groups and the cutting
logic, without a GPU."""

from __future__ import annotations

import itertools

import pytest
import torch

from fakilorn_cases import PAGE_TOKENS, assert_rows_close, config, plain_greedy, plain_logits, random_weights, tokens_for
from torch_ops import TorchOps

from mini_gpt_inference_b200 import EngineConfig, FakilornConfig, LLMEngine, SamplingParams
from mini_gpt_inference_b200.engine.build import load_model, make_runner
from mini_gpt_inference_b200.engine.runner import StepEntry


def cpu_runner(raw, tensors, page_tokens, num_pages, max_requests=4):
    loaded = load_model(config=FakilornConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cpu")
    return make_runner(loaded, TorchOps(), page_tokens, num_pages, max_requests)


@pytest.mark.parametrize("which", "ABC")
def test_cuttings_agree_with_plain(which):
    raw = config(which, 3.0)
    tensors = random_weights(raw, 3)
    pt = PAGE_TOKENS[which]
    lengths = {"a": 41, "b": 36, "c": 9, "d": 2 * pt + 1}
    runner = cpu_runner(raw, tensors, pt, sum(-(-n // pt) for n in lengths.values()))
    # layers that differ in their key/value sizes keep their pages in groups of their own
    assert len(runner.manager.groups) == {"A": 3, "B": 2, "C": 2}[which]
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
        assert_rows_close(torch.cat(got[k]), want[k], 1e-4, f"request {k}")
        runner.finish(k)
    assert runner.manager.stats()["allocated_blocks"] == 0


def test_generation_through_the_engine_on_the_double():
    raw = config("A", 2.0)
    tensors = random_weights(raw, 4)
    loaded = load_model(config=FakilornConfig.from_dict(raw), tensors=tensors, dtype="float32", device="cpu")
    engine = LLMEngine(loaded, EngineConfig(dtype="float32", device="cpu", block_size=16, num_blocks=12, max_batch_size=2,
                                            max_num_batched_tokens=12, max_prefill_chunk=5), ops=TorchOps())
    prompts = [tokens_for(raw, n, 30 + n) for n in (7, 1, 18)]
    outs = engine.generate(prompts, SamplingParams(max_tokens=6, temperature=0.0))
    for prompt, out in zip(prompts, outs):
        assert out["token_ids"] == plain_greedy(raw, tensors, prompt, 6)
    assert engine.stats()["allocated_blocks"] == 0
