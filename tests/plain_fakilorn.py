"""A plain, slow Fakilorn: one function per mechanism, whole sequences, float64 by default.

It takes the model as a config dict (the keys of ``config.json``) and a dict of tensors by
their checkpoint names, and shares no code with the engine.  Notation: ``x`` is the
residual stream ``[T, width]`` of one sequence, ``h`` a mixer's or feed-forward's input.

* norm:      ``(x - mean) / sqrt(var + eps) * w + b`` (biased variance)
* unit rms:  ``x / sqrt(mean(x^2) + eps)`` over the last axis, no gain
* attention: per head ``softmax_j<=i(scale * unit(q_i) . unit(k_j)) v_j``, grouped key/value
  heads, values blended with the first blending layer's values, heads gated by
  ``sigmoid(W_g h)`` before the output projection
* dense ff:  ``W_down relu(W_up h)^2``
* routed ff: the ``top`` largest router logits choose experts, softmax over the chosen logits
  weighs them; expert ``W_down (silu(W_gate h) * W_up h)``; a shared expert of the same form
  is added for every token, times ``sigmoid(W_sg h)``
"""

from __future__ import annotations

import math

import torch


def layer_norm(x, w, b, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    y = (x - mean) / torch.sqrt(var + eps) * w
    return y if b is None else y + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def embed(tokens, table, scale):
    return table[torch.as_tensor(tokens, dtype=torch.long)] * scale


def attention_scores(q, k, scale):
    """q [T, D], k [T, D] of one head pair -> causal softmax weights [T, T]."""
    s = (q @ k.T) * scale
    t = q.shape[0]
    mask = torch.ones(t, t, dtype=torch.bool).tril()
    s = s.masked_fill(~mask, -math.inf)
    return torch.softmax(s, dim=-1)


def blend_values(v, v_first, lam):
    return (1.0 - lam) * v + lam * v_first


def attention_mixer(h, w, prefix, m, eps, v_first, is_first):
    """Returns (output [T, width], the values this layer caches [T, G * vdim])."""
    heads, groups, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = h.shape[0]
    q = (h @ w[prefix + "q"].T).view(t, heads, d)
    k = (h @ w[prefix + "k"].T).view(t, groups, d)
    v = h @ w[prefix + "v"].T
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    if m.get("v_mix") and not is_first:
        v = blend_values(v, v_first, w[prefix + "vmix"])
    vh = v.view(t, groups, dv)
    out = torch.empty(t, heads, dv, dtype=h.dtype)
    per = heads // groups
    for a in range(heads):
        g = a // per
        out[:, a] = attention_scores(q[:, a], k[:, g], m["scale"]) @ vh[:, g]
    gate = torch.sigmoid(h @ w[prefix + "g"].T)
    return (out.reshape(t, heads * dv) * gate) @ w[prefix + "o"].T, v


def dense_ff(h, w, prefix):
    return (torch.relu(h @ w[prefix + "up"].T) ** 2) @ w[prefix + "down"].T


def expert_ff(h, w, prefix):
    a = h @ w[prefix + "gate"].T
    return ((a * torch.sigmoid(a)) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(h, router_w, top):
    """Returns (chosen expert ids [T, top], their weights [T, top])."""
    z = h @ router_w.T
    vals, ids = torch.topk(z, top, dim=-1)
    return ids, torch.softmax(vals, dim=-1)


def routed_ff(h, w, prefix, mlp):
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    ids, weights = route(h, w[prefix + "router"], top)
    out = torch.zeros(h.shape[0], w[prefix + "e0.down"].shape[0], dtype=h.dtype)
    for e in range(n):
        y = expert_ff(h, w, f"{prefix}e{e}.")
        share = (weights * (ids == e)).sum(-1, keepdim=True)
        out = out + share * y
    if mlp.get("shared"):
        sg = torch.sigmoid(h @ w[prefix + "shared.sg"].T)             # [T, 1]
        out = out + sg * expert_ff(h, w, prefix + "shared.")
    return out


def forward(config, tensors, tokens, dtype=torch.float64):
    """Logits [T, vocab] and the residual stream after every layer [L, T, width]."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = config["norm"]["eps"]
    x = embed(tokens, w["embed"], config["embedding"]["scale"])
    v_first, streams = None, []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        if layer["type"] != "attention":
            raise ValueError(f"unknown mixer {layer['type']!r}")
        m = layer["mixer"]
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        first = bool(m.get("v_mix")) and v_first is None
        y, v = attention_mixer(h, w, p + "mix.", m, eps, v_first, first)
        if first:
            v_first = v
        x = x + y
        mlp = layer.get("mlp")
        if mlp is not None:
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            if mlp["kind"] == "dense":
                x = x + dense_ff(h, w, p + "mlp.")
            elif mlp["kind"] == "moe":
                x = x + routed_ff(h, w, p + "mlp.", mlp)
            else:
                raise ValueError(f"unknown feed-forward {mlp['kind']!r}")
        streams.append(x)
    y = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    logits = (y @ w["embed"].T) * config["logit_scale"]
    return logits, torch.stack(streams)
