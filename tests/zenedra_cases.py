"""Small Zenedra configurations and random weights for the tests, made here (names and shapes written
out from the design, not taken from the engine's own list), and the plain logits."""

from __future__ import annotations

import math

import torch

import plain_zenedra


def _gla(heads, dim, vdim, tau):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def _mlstm(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def _attn(heads, kv_heads, dim, block, scale):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
                                           "mask": {"size": block}, "scale": scale}}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, top, ff, limit, scale, groups=None, shared=None):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def config(which: str, every_expert: bool = False) -> dict:
    """A: every mixer and feed-forward, a loop over the first two layers, grouped key heads, groups of
    experts.  B: no loop, attention first, as many key heads as query heads, one group of experts, one
    chosen expert, a block of 1 page, multipliers of 1 and 0.  C: a loop of one pass over all layers, heads
    of 80 key channels and 33 value channels, a layer without a feed-forward, experts without groups or a
    shared one.  D: heads of 64 and 128 channels, a block mask longer than any test's sequence.
    ``every_expert``: each router chooses all its experts (in bfloat16 a close call between two experts
    flips with the rounding of the activations, which says nothing about the kernels)."""
    raw = _config(which)
    if every_expert:
        for layer in raw["layers"]:
            mlp = layer.get("mlp")
            if mlp is not None and mlp["kind"] == "moe":
                mlp["router"]["top"] = mlp["router"]["experts"]
                mlp["router"].pop("groups", None)
    return raw


def _config(which: str) -> dict:
    if which == "A":
        layers = [
            {**_mlstm(2, 24, 40, 10.0), "mlp": _dense(96)},
            {**_attn(6, 2, 16, 8, 0.3), "mlp": _moe(6, 2, 24, 1.5, 1.7, (3, 2), (40, 2.5))},
            {**_gla(3, 16, 24, 8.0), "mlp": _moe(6, 2, 24, 1.5, 1.7, (3, 2), (40, 2.5))},
        ]
        return {"architecture": "Zenedra", "vocab": 211, "width": 64, "max_positions": 256, "layers": layers,
                "loop": {"start": 0, "stop": 2, "times": 2}, "norm": {"eps": 1e-4},
                "embedding": {"bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 5}}}
    if which == "B":
        layers = [
            {**_attn(3, 3, 32, 16, 0.2), "mlp": _moe(4, 1, 48, 3.0, 0.8, (1, 1))},
            {**_gla(1, 40, 32, 3.0), "mlp": _dense(200)},
            {**_mlstm(1, 32, 96, 4.0), "mlp": _moe(4, 1, 48, 3.0, 0.8, (1, 1))},
        ]
        return {"architecture": "Zenedra", "vocab": 300, "width": 96, "max_positions": 300, "layers": layers,
                "norm": {"eps": 1e-6}, "embedding": {"bigram": {"buckets": 1, "mul_prev": 1, "mul_cur": 0}}}
    if which == "C":
        layers = [
            {**_gla(2, 80, 33, 20.0), "mlp": None},
            {**_attn(5, 1, 24, 23, 0.25), "mlp": _moe(5, 3, 20, 0.7, 2.0)},
            {**_mlstm(3, 80, 33, 30.0), "mlp": _dense(72)},
        ]
        return {"architecture": "Zenedra", "vocab": 97, "width": 72, "max_positions": 200, "layers": layers,
                "loop": {"start": 0, "stop": 3, "times": 1}, "norm": {"eps": 1e-5},
                "embedding": {"bigram": {"buckets": 1000, "mul_prev": 1009, "mul_cur": 10007}}}
    if which == "D":
        layers = [
            {**_attn(4, 2, 64, 4096, 0.125), "mlp": _dense(256)},
            {**_gla(2, 64, 128, 12.0), "mlp": _dense(256)},
            {**_mlstm(2, 128, 64, 20.0), "mlp": _moe(8, 2, 64, 2.5, 1.5, (4, 2), (64, 1.0))},
        ]
        return {"architecture": "Zenedra", "vocab": 384, "width": 128, "max_positions": 640, "layers": layers,
                "loop": {"start": 1, "stop": 2, "times": 3}, "norm": {"eps": 1e-5},
                "embedding": {"bigram": {"buckets": 256, "mul_prev": 3, "mul_cur": 11}}}
    if which == "E":                                        # no attention at all: nothing is kept in pages
        layers = [
            {**_gla(2, 16, 16, 2.0), "mlp": _dense(64)},
            {**_mlstm(2, 16, 24, 5.0), "mlp": None},
        ]
        return {"architecture": "Zenedra", "vocab": 64, "width": 40, "max_positions": 200, "layers": layers,
                "norm": {"eps": 1e-5}, "embedding": {"bigram": {"buckets": 13, "mul_prev": 2, "mul_cur": 3}}}
    if which == "F":                                        # attention alone, three passes over the one layer
        layers = [{**_attn(2, 1, 32, 10, 0.2), "mlp": _dense(48)}]
        return {"architecture": "Zenedra", "vocab": 80, "width": 48, "max_positions": 200, "layers": layers,
                "loop": {"start": 0, "stop": 1, "times": 3}, "norm": {"eps": 1e-5},
                "embedding": {"bigram": {"buckets": 31, "mul_prev": 7, "mul_cur": 1}}}
    raise KeyError(which)


PAGE_TOKENS = {"A": 8, "B": 16, "C": 4, "D": 16, "E": 8, "F": 4}
DECAY_RANK = {"A": 4, "B": 7, "C": 16, "D": 8}


def random_weights(raw: dict, seed: int, dtype=torch.float32, rank: int = 5, sharp: float = 1.0,
                   as_bfloat16: bool = False) -> dict:
    """Weights with unit-variance activations: matrices ``N(0, 1 / inputs)``, output projections smaller by the
    depth, norm weights and biases ``N(0, 0.3)``, embeddings ``N(0, 1)``.  ``sharp`` scales the query projections
    of the attention layers, so that a softmax leans on few keys.  ``as_bfloat16``: every number is one that
    bfloat16 holds (an engine that computes in bfloat16 and the plain side then use the same weights)."""
    gen = torch.Generator().manual_seed(seed)
    c = raw["width"]
    depth = len(plain_zenedra.run_order(raw))

    def mat(rows, cols, scale=1.0):
        return torch.randn(rows, cols, generator=gen) * (scale / math.sqrt(cols))

    def vec(n, scale=0.3):
        return torch.randn(n, generator=gen) * scale

    b = raw["embedding"]["bigram"]
    w = {"embed": torch.randn(raw["vocab"], c, generator=gen), "bigram": torch.randn(b["buckets"] + 1, c, generator=gen),
         "pos": torch.randn(raw["max_positions"], c, generator=gen) * 0.5,
         "final.norm": vec(c), "head": mat(raw["vocab"], c)}
    if raw.get("loop"):
        w["loop.in"] = mat(c, 2 * c, math.sqrt(2.0))
        w["loop.step"] = vec(raw["loop"]["times"] * c).view(raw["loop"]["times"], c)
    out_scale = 1.0 / math.sqrt(2 * depth)
    for i, layer in enumerate(raw["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        w[p + "norm1"] = vec(c)
        x = p + "mix."
        h, d, dv = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            g = m["kv_heads"]
            w[x + "q"], w[x + "q.b"] = mat(h * d, c, sharp), vec(h * d)
            w[x + "k"], w[x + "k.b"] = mat(g * d, c), vec(g * d)
            w[x + "q.norm"], w[x + "k.norm"] = 1.0 + vec(d), 1.0 + vec(d)
            w[x + "o"], w[x + "o.b"] = mat(c, h * d, out_scale), vec(c, 0.05)
        else:
            w[x + "q"], w[x + "k"] = mat(h * d, c), mat(h * d, c)
            w[x + "v"], w[x + "g"] = mat(h * dv, c), mat(h * dv, c)
            w[x + "o"] = mat(c, h * dv, out_scale)
            if layer["type"] == "gla":
                w[x + "norm"] = 1.0 + vec(dv)
                w[x + "a1"], w[x + "a2"] = mat(rank, c), mat(h * d, rank, 2.0)
                w[x + "a2.b"] = vec(h * d, 1.5) + 1.0
            else:
                w[x + "norm"] = 1.0 + vec(h * dv)
                for name in ("i", "f"):
                    w[x + name], w[x + name + ".b"] = mat(h, c, 2.0), vec(h, 1.5)
        f = layer.get("mlp")
        if f is None:
            continue
        w[p + "norm2"] = vec(c)
        y = p + "mlp."
        if f["kind"] == "dense":
            w[y + "gate"], w[y + "up"] = mat(f["ff"], c), mat(f["ff"], c)
            w[y + "down"] = mat(c, f["ff"], out_scale)
            continue
        r, e = f["router"], f["expert"]
        w[y + "router"], w[y + "correction"] = mat(r["experts"], c, 2.0), vec(r["experts"], 0.4)
        units = [(f"{y}e{j}.", e["ff"]) for j in range(r["experts"])]
        if f.get("shared") is not None:
            units.append((y + "shared.", f["shared"]["ff"]))
        for q, ff in units:
            w[q + "gate"], w[q + "up"] = mat(ff, c, 1.5), mat(ff, c, 1.5)
            w[q + "down"] = mat(c, ff, out_scale)
    if as_bfloat16:
        w = {k: v.to(torch.bfloat16).float() for k, v in w.items()}
    return {k: v.to(dtype).contiguous() for k, v in w.items()}


def tokens_for(raw: dict, length: int, seed: int) -> list[int]:
    gen = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, raw["vocab"], (length,), generator=gen).tolist()


def plain_logits(raw: dict, tensors: dict, tokens, rows=None, dtype=torch.float64) -> torch.Tensor:
    out = plain_zenedra.forward(tokens, tensors, raw, dtype)
    return out if rows is None else out[list(rows)]


def plain_greedy(raw: dict, tensors: dict, prompt, new_tokens: int) -> list[int]:
    return plain_zenedra.greedy(prompt, tensors, raw, new_tokens)


def relative_error(got: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
    """Per row: the largest difference of the logits over the row's own spread."""
    want = want.double()
    return (got.double().cpu() - want).abs().amax(-1) / want.std(-1)


def assert_rows_close(got, want, tol, what: str, places=None, outliers: float = 0.0) -> None:
    """``outliers``: the share of rows (at least one, if not zero) that may miss ``tol``, though not five times
    ``tol``.  For bfloat16 runs: where a head's read-out nearly cancels (a query at right angles to the one key
    its memory holds), the norm that follows magnifies the rounding of that one token by a hundred."""
    err = relative_error(got, want)
    bad = (~(err <= tol)).nonzero()
    if outliers and 0 < bad.numel() <= max(1, int(outliers * err.numel())):
        bad = (~(err <= 5 * tol)).nonzero()
    if bad.numel():
        i = int(bad[0])
        raise AssertionError(f"{what}: first wrong logits at {places[i] if places is not None else i}: "
                             f"error {float(err[i]):.3e} of the row's spread > {tol:.1e}")
