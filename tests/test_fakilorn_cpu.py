"""Fakilorn without a GPU: its configuration, registry entry, tensor names and loader, and the
plain implementation's own mechanisms against brute-force restatements."""

from __future__ import annotations

import copy
import json
import math

import pytest
import torch

import plain_fakilorn as plain
from fakilorn_cases import config, plain_logits, random_weights, tensor_shapes, tokens_for

from mini_gpt_inference_b200.config import ConfigError, FakilornConfig, lookup
from mini_gpt_inference_b200.config.registry import architecture_name, load_config
from mini_gpt_inference_b200.parts import DecoderModel
from mini_gpt_inference_b200.weights import load_file, write_random_model
from mini_gpt_inference_b200.weights.loader import WeightsError, check_and_bind


def build(which):
    cfg = FakilornConfig.from_dict(config(which))
    return cfg, DecoderModel(lookup(cfg.architecture).describe(cfg))


@pytest.mark.parametrize("which", "ABC")
def test_config_round_trip_and_registry(which):
    raw = config(which)
    assert architecture_name(raw) == "Fakilorn"
    cfg = FakilornConfig.from_dict(raw)
    assert FakilornConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.vocab_size == raw["vocab"] and len(cfg.layers) == len(raw["layers"])
    assert lookup("Fakilorn").config_class is FakilornConfig
    shapes = tensor_shapes(raw)
    assert cfg.num_parameters() == sum(math.prod(s) for s in shapes.values())


def test_config_errors():
    raw = config("A")
    for path, value in [(("layers", 0, "mixer", "heads"), 3), (("layers", 1, "mlp", "router", "top"), 9),
                        (("layers", 0, "type"), "recurrent"), (("norm", "eps"), 0.0), (("vocab",), -1),
                        (("layers", 2, "mixer", "vdim"), 8)]:
        bad = copy.deepcopy(raw)
        node = bad
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ConfigError):
            FakilornConfig.from_dict(bad)
    missing = copy.deepcopy(raw)
    del missing["logit_scale"]
    with pytest.raises(ConfigError):
        FakilornConfig.from_dict(missing)


@pytest.mark.parametrize("which", "ABC")
def test_tensor_names_and_shapes(which):
    raw = config(which)
    cfg, model = build(which)
    specs = {n: tuple(s.shape) for n, s in model.tensor_specs().items() if not s.optional}
    assert specs == tensor_shapes(raw)
    bound = check_and_bind(random_weights(raw, 1), model.tensor_specs())
    model.bind(bound)
    mixers = [layer.mixer for layer in model.layers]
    blends = [m.value_blend for m in mixers]
    assert blends == {"A": [None, "source", "blend", "blend"], "B": ["source", "blend", "blend"],
                      "C": [None, None]}[which]
    m0, r0 = mixers[0], raw["layers"][0]["mixer"]
    assert m0.fused_weight.shape == (r0["heads"] * (r0["dim"] + r0["vdim"]) + r0["kv_heads"] * (r0["dim"] + r0["vdim"]),
                                     raw["width"])
    assert [layer.run.__name__ for layer in model.layers].count("pre_norm_mixer_only") == (1 if which == "A" else 0)


def test_loader_reports_and_tolerates():
    raw = config("A")
    _, model = build("A")
    tensors = random_weights(raw, 2)
    # tensors that the model never reads may be present: the blend scalar of a layer that does not
    # blend, the second norm of a layer without a feed-forward
    extra = dict(tensors)
    extra["l0.mix.vmix"] = torch.tensor(0.5, dtype=torch.bfloat16)
    extra["l2.norm2"] = torch.ones(raw["width"], dtype=torch.bfloat16)
    extra["l2.norm2.b"] = torch.zeros(raw["width"], dtype=torch.bfloat16)
    check_and_bind(extra, model.tensor_specs())
    broken = dict(tensors)
    del broken["l1.mlp.e3.up"]
    broken["l1.mlp.e9.up"] = tensors["l1.mlp.e0.up"]
    broken["l3.mix.k"] = tensors["l3.mix.k"][:-1]
    with pytest.raises(WeightsError) as err:
        check_and_bind(broken, model.tensor_specs())
    assert err.value.missing == ["l1.mlp.e3.up"] and err.value.unexpected == ["l1.mlp.e9.up"]
    assert len(err.value.wrong_shape) == 1 and "l3.mix.k" in err.value.wrong_shape[0]


def test_random_model_folder(tmp_path):
    cfg = FakilornConfig.from_dict(config("B"))
    folder = write_random_model(tmp_path / "m", cfg, 3, "bfloat16")
    family, again = load_config(folder)
    assert family.name == "Fakilorn" and again == cfg
    assert json.loads((folder / "config.json").read_text())["architecture"] == "Fakilorn"
    stored = load_file(folder / "model.safetensors")
    assert {n: tuple(t.shape) for n, t in stored.items()} == tensor_shapes(config("B"))
    assert all(0.0 < float(stored[f"l{i}.mix.vmix"]) < 1.0 for i in range(3))


# ---- the plain implementation's mechanisms, each against a restatement by hand ---------------------
def test_plain_norms():
    x = torch.randn(5, 7, dtype=torch.float64)
    w, b = torch.randn(7, dtype=torch.float64), torch.randn(7, dtype=torch.float64)
    want = torch.nn.functional.layer_norm(x, (7,), w, b, 1e-3)
    assert torch.allclose(plain.layer_norm(x, w, b, 1e-3), want, atol=1e-12)
    u = plain.unit_rms(x, 0.0)
    assert torch.allclose((u * u).mean(-1), torch.ones(5, dtype=torch.float64), atol=1e-12)
    assert torch.allclose(plain.unit_rms(x, 0.5), x / torch.sqrt((x * x).mean(-1, keepdim=True) + 0.5))


def test_plain_route_and_experts():
    gen = torch.Generator().manual_seed(0)
    h = torch.randn(9, 12, generator=gen, dtype=torch.float64)
    router = torch.randn(6, 12, generator=gen, dtype=torch.float64)
    ids, weights = plain.route(h, router, 3)
    z = h @ router.T
    for t in range(9):
        order = sorted(range(6), key=lambda e: -float(z[t, e]))[:3]
        assert ids[t].tolist() == order
        e = torch.exp(z[t, order] - z[t, order].max())
        assert torch.allclose(weights[t], e / e.sum(), atol=1e-12)
    assert torch.allclose(weights.sum(-1), torch.ones(9, dtype=torch.float64))
    # with every expert chosen the weights are the softmax over all logits
    ids, weights = plain.route(h, router, 6)
    assert torch.allclose(weights.gather(1, ids.argsort(-1)), torch.softmax(z, -1), atol=1e-12)


def test_plain_attention_is_causal_and_grouped():
    raw = config("A", sharp=3.0)
    tensors = random_weights(raw, 5)
    tokens = tokens_for(raw, 40, 1)
    full = plain_logits(raw, tensors, tokens)
    # logits at a position depend on no later token
    changed = list(tokens)
    changed[30:] = tokens_for(raw, 10, 2)
    assert torch.equal(full[:30], plain_logits(raw, tensors, changed)[:30])
    assert not torch.allclose(full[30:], plain_logits(raw, tensors, changed)[30:])
    assert torch.allclose(full[:17], plain_logits(raw, tensors, tokens[:17]), atol=1e-9)
    # the blend scalar of the layer that publishes its values is never read
    other = dict(tensors)
    other["l1.mix.vmix"] = torch.tensor(0.9, dtype=torch.bfloat16)
    assert torch.equal(full, plain_logits(raw, other, tokens))
    other["l2.mix.vmix"] = torch.tensor(0.9, dtype=torch.bfloat16)
    assert not torch.allclose(full, plain_logits(raw, other, tokens))
