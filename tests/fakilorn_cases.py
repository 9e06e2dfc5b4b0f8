"""Small Fakilorn configurations and random weights for the tests, made here (names and shapes
written out from the design, not taken from the engine's own list), and the plain logits."""

from __future__ import annotations

import math

import torch

import plain_fakilorn


def _attn(heads, kv_heads, dim, vdim, v_mix, sharp=1.0):
    # q and k have unit RMS: a score is scale * dim * cos; `sharp` makes the softmax lean on few keys
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "v_mix": v_mix,
            "scale": sharp / math.sqrt(dim)}


def _moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def config(which: str, sharp: float = 1.0, every_expert: bool = False) -> dict:
    """``every_expert``: each router chooses all its experts (the weights stay a softmax).  A choice
    among experts is discrete: where two router logits are close, the rounding of bfloat16
    activations flips it and the token's output jumps, which says nothing about the kernels.  Whole
    models in bfloat16 are therefore compared with every expert chosen; the choice itself is
    compared in 32-bit on whole models and in both formats on the router alone."""
    raw = _config(which, sharp)
    if every_expert:
        for layer in raw["layers"]:
            if layer["mlp"] is not None and layer["mlp"]["kind"] == "moe":
                layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return raw


def _config(which: str, sharp: float) -> dict:
    """A: grouped heads, keys larger than values, a blending chain that starts at the second layer,
    every kind of feed-forward.  B: as many key heads as query heads, equal key and value sizes, one
    chosen expert, all experts chosen, no shared expert.  C: sizes that are multiples of nothing.  D: keys
    and values of 64 features."""
    if which == "A":
        layers = [
            {"type": "attention", "mixer": _attn(4, 2, 24, 16, False, sharp), "mlp": {"kind": "dense", "ff": 96}},
            {"type": "attention", "mixer": _attn(4, 2, 24, 16, True, sharp), "mlp": _moe(5, 2, 40, 24)},
            {"type": "attention", "mixer": _attn(6, 2, 8, 16, True, sharp), "mlp": None},
            {"type": "attention", "mixer": _attn(2, 2, 40, 16, True, sharp), "mlp": _moe(3, 3, 16)},
        ]
        return {"architecture": "Fakilorn", "vocab": 211, "width": 64, "layers": layers,
                "embedding": {"scale": 1.7}, "logit_scale": 0.6, "norm": {"eps": 1e-4}}
    if which == "B":
        layers = [
            {"type": "attention", "mixer": _attn(3, 3, 32, 32, True, sharp), "mlp": _moe(4, 1, 48, 32)},
            {"type": "attention", "mixer": _attn(3, 3, 32, 32, True, sharp), "mlp": {"kind": "dense", "ff": 200}},
            {"type": "attention", "mixer": _attn(6, 3, 16, 32, True, sharp), "mlp": _moe(6, 6, 24)},
        ]
        return {"architecture": "Fakilorn", "vocab": 300, "width": 96, "layers": layers,
                "embedding": {"scale": 0.8}, "logit_scale": 1.0, "norm": {"eps": 1e-6}}
    if which == "C":
        layers = [
            {"type": "attention", "mixer": _attn(5, 1, 10, 6, False, sharp), "mlp": _moe(7, 3, 11, 9)},
            {"type": "attention", "mixer": _attn(3, 3, 14, 22, False, sharp), "mlp": {"kind": "dense", "ff": 37}},
        ]
        return {"architecture": "Fakilorn", "vocab": 97, "width": 50, "layers": layers,
                "embedding": {"scale": 3.0}, "logit_scale": 0.37, "norm": {"eps": 1e-5}}
    if which == "D":
        # keys and values of 64 features each: the sizes that the tcgen05 prompt attention takes
        layers = [
            {"type": "attention", "mixer": _attn(4, 2, 64, 64, True, sharp), "mlp": {"kind": "dense", "ff": 160}},
            {"type": "attention", "mixer": _attn(4, 2, 64, 64, True, sharp), "mlp": _moe(4, 2, 64, 32)},
        ]
        return {"architecture": "Fakilorn", "vocab": 173, "width": 128, "layers": layers,
                "embedding": {"scale": 1.3}, "logit_scale": 0.9, "norm": {"eps": 1e-5}}
    raise KeyError(which)


PAGE_TOKENS = {"A": 16, "B": 8, "C": 4, "D": 16}


def tensor_shapes(cfg: dict) -> dict[str, tuple]:
    c = cfg["width"]
    shapes = {"embed": (cfg["vocab"], c), "final.norm": (c,), "final.norm.b": (c,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1.b"] = (c,)
        shapes[p + "mix.q"] = (m["heads"] * m["dim"], c)
        shapes[p + "mix.k"] = (m["kv_heads"] * m["dim"], c)
        shapes[p + "mix.v"] = (m["kv_heads"] * m["vdim"], c)
        shapes[p + "mix.g"] = (m["heads"] * m["vdim"], c)
        shapes[p + "mix.o"] = (c, m["heads"] * m["vdim"])
        if m["v_mix"]:
            shapes[p + "mix.vmix"] = ()
        mlp = layer["mlp"]
        if mlp is None:
            continue
        shapes[p + "norm2"] = shapes[p + "norm2.b"] = (c,)
        if mlp["kind"] == "dense":
            shapes[p + "mlp.up"] = (mlp["ff"], c)
            shapes[p + "mlp.down"] = (c, mlp["ff"])
            continue
        f = mlp["expert"]["ff"]
        shapes[p + "mlp.router"] = (mlp["router"]["experts"], c)
        for e in range(mlp["router"]["experts"]):
            shapes[f"{p}mlp.e{e}.gate"] = shapes[f"{p}mlp.e{e}.up"] = (f, c)
            shapes[f"{p}mlp.e{e}.down"] = (c, f)
        if mlp.get("shared"):
            s = mlp["shared"]["ff"]
            shapes[p + "mlp.shared.gate"] = shapes[p + "mlp.shared.up"] = (s, c)
            shapes[p + "mlp.shared.down"] = (c, s)
            shapes[p + "mlp.shared.sg"] = (1, c)
    return shapes


def random_weights(cfg: dict, seed: int, dtype=torch.bfloat16) -> dict[str, torch.Tensor]:
    """Matrices N(0, 1/fan_in) (routers and gates a little larger, so that choices are not close
    calls), norm gains around one, shifts and blend scalars away from zero and one."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in sorted(tensor_shapes(cfg).items()):
        noise = torch.randn(shape, generator=gen)
        if name.endswith(".b"):
            t = 0.2 * noise
        elif "norm" in name:
            t = 1.0 + 0.2 * noise
        elif name.endswith("vmix"):
            t = 0.25 + 0.5 * torch.sigmoid(noise)
        elif name == "embed":
            t = noise
        elif name.endswith("router") or name.endswith(".sg"):
            t = noise * (2.0 / math.sqrt(shape[-1]))
        else:
            t = noise / math.sqrt(shape[-1])
        out[name] = t.to(dtype)
    return out


def tokens_for(cfg: dict, length: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (length,), generator=gen).tolist()


def plain_logits(cfg: dict, tensors: dict, tokens) -> torch.Tensor:
    return plain_fakilorn.forward(cfg, tensors, tokens)[0]


def plain_greedy(cfg: dict, tensors: dict, prompt, n: int) -> list[int]:
    seq, out = list(prompt), []
    for _ in range(n):
        out.append(int(plain_logits(cfg, tensors, seq)[-1].argmax()))
        seq.append(out[-1])
    return out


def relative_error(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: the largest difference of the logits over the rows' own spread."""
    want = want.double()
    return (got.double().cpu() - want).abs().amax(-1) / want.std(-1)


def assert_rows_close(got, want, tol, what: str, places=None) -> None:
    err = relative_error(got, want)
    bad = (~(err <= tol)).nonzero()
    if bad.numel():
        i = int(bad[0])
        raise AssertionError(f"{what}: first wrong logits at {places[i] if places is not None else i}: "
                             f"error {float(err[i]):.3e} of the row's spread > {tol:.1e}")
