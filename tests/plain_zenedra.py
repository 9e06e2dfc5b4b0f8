"""A plain, slow Zenedra: one function per mechanism, whole sequences, float64 by default.

It takes the model as a config dict (the keys of ``config.json``) and a dict of tensors by their
checkpoint names, and shares no code with the engine.  Notation: ``x`` is the residual stream
``[T, width]`` of one sequence, ``h`` the input of a mixer or feed-forward, ``t`` a position.

* embedding:  ``E[tok_t] + B[r_t] + P[t]`` with ``r_0 = buckets`` and ``r_t = (tok_(t-1) * mul_prev +
  tok_t * mul_cur) mod buckets``
* rms norm:   ``x / sqrt(mean(x^2) + eps) * (offset + w)``; offset 1 for the layers' norms and the
  final one, 0 for norms inside mixers
* run order:  layers before ``start`` once, layers ``start .. stop-1`` ``times`` times, the rest once;
  in front of pass ``p``: ``x = W_in [x ; x_emb] + step[p]``
* gla:        ``S_t = diag(a_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t``, ``a = sigmoid(z)^(1/tau)``
* attention:  values are the keys before their norm; scores ``scale * qn . kn - slope_h * (t - j)``
  over the keys of the query's own block of ``mask.size`` positions
* mlstm:      stabilised matrix memory with scalar gates per head
* dense ff:   ``W_down (gelu_tanh(W_gate h) * W_up h)``
* routed ff:  sigmoid scores, a correction only for the choice, groups of neighbours, weights
  ``scale * s`` of the chosen experts, clamped experts, a shared expert
"""

from __future__ import annotations

import math

import torch


# ---- pieces --------------------------------------------------------------------------------------
def rms_norm(x, w, eps, offset=0.0):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * (offset + w)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    rows = [buckets]
    for t in range(1, len(tokens)):
        rows.append((int(tokens[t - 1]) * mul_prev + int(tokens[t]) * mul_cur) % buckets)
    return rows


def embedding(tokens, w, cfg):
    b = cfg["embedding"]["bigram"]
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    rows = torch.as_tensor(bigram_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"]), dtype=torch.long)
    return w["embed"][ids] + w["bigram"][rows] + w["pos"][: len(tokens)]


def run_order(cfg):
    """[(layer, pass number or None, whether a pass begins here)]"""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    order = [(i, None, False) for i in range(loop["start"])]
    for p in range(loop["times"]):
        order += [(i, p, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None, False) for i in range(loop["stop"], n)]


def pass_entry(x, x_emb, w, p):
    return torch.cat([x, x_emb], dim=-1) @ w["loop.in"].T + w["loop.step"][p]


# ---- mixers --------------------------------------------------------------------------------------
def gla_mixer(h, w, p, m, eps):
    heads, d, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, heads, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(T, heads, d)
    v = (h @ w[p + "v"].T).view(T, heads, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.exp(torch.nn.functional.logsigmoid(z) / tau).view(T, heads, d)
    S = torch.zeros(heads, d, dv, dtype=h.dtype)
    o = torch.empty(T, heads, dv, dtype=h.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, w[p + "norm"], eps)
    g = h @ w[p + "g"].T
    return (o.reshape(T, heads * dv) * (g * torch.sigmoid(g))) @ w[p + "o"].T


def distance_slopes(heads):
    return torch.tensor([2.0 ** (-8.0 * (a + 1) / heads) for a in range(heads)], dtype=torch.float64)


def attention_mixer(h, w, p, m, eps):
    heads, groups, d = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, heads, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, groups, d)
    v = k
    qn, kn = rms_norm(q, w[p + "q.norm"], eps), rms_norm(k, w[p + "k.norm"], eps)
    pos = torch.arange(T)
    dist = (pos[:, None] - pos[None, :]).to(h.dtype)
    block = m["mask"]["size"]
    seen = (pos[None, :] <= pos[:, None]) & ((pos[:, None] // block) == (pos[None, :] // block))
    slopes = distance_slopes(heads).to(h.dtype)
    out = torch.empty(T, heads, d, dtype=h.dtype)
    per = heads // groups
    for a in range(heads):
        s = (qn[:, a] @ kn[:, a // per].T) * m["scale"] - slopes[a] * dist
        s = s.masked_fill(~seen, -math.inf)
        out[:, a] = torch.softmax(s, dim=-1) @ v[:, a // per]
    return out.reshape(T, heads * d) @ w[p + "o"].T + w[p + "o.b"]


def soft_cap(x, cap):
    return cap * torch.tanh(x / cap)


def mlstm_mixer(h, w, p, m, eps):
    heads, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    T = h.shape[0]
    q = (h @ w[p + "q"].T).view(T, heads, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(T, heads, d)
    v = (h @ w[p + "v"].T).view(T, heads, dv)
    gi = soft_cap(h @ w[p + "i"].T + w[p + "i.b"], cap)
    gf = torch.nn.functional.logsigmoid(soft_cap(h @ w[p + "f"].T + w[p + "f.b"], cap))
    S = torch.zeros(heads, d, dv, dtype=h.dtype)
    n = torch.zeros(heads, d, dtype=h.dtype)
    mx = torch.zeros(heads, dtype=h.dtype)
    o = torch.empty(T, heads, dv, dtype=h.dtype)
    for t in range(T):
        m_new = torch.maximum(gf[t] + mx, gi[t])
        keep, take = torch.exp(gf[t] + mx - m_new), torch.exp(gi[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = m_new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    o = rms_norm(o, None, eps).reshape(T, heads * dv) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


# ---- feed-forwards ---------------------------------------------------------------------------------
def dense_ff(h, w, p):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def clamped_expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(h, w, p, r):
    """Returns (ids [T, top], weights [T, top]) in the order of falling choice scores."""
    experts, top = r["experts"], r["top"]
    s = torch.sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    groups = r.get("groups")
    if groups is not None:
        count, keep = groups["count"], groups["keep"]
        per = experts // count
        grouped = choice.view(-1, count, per)
        score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
        best = score.topk(keep, dim=-1).indices
        allowed = torch.zeros_like(score, dtype=torch.bool).scatter_(1, best, True)
        choice = grouped.masked_fill(~allowed[:, :, None], -math.inf).reshape(-1, experts)
    ids = choice.topk(top, dim=-1).indices
    return ids, s.gather(1, ids) * r["scale"]


def routed_ff(h, w, p, f):
    ids, weights = route(h, w, p, f["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            e = int(ids[t, j])
            out[t] += weights[t, j] * clamped_expert(h[t: t + 1], w, f"{p}e{e}.", f["expert"]["limit"])[0]
    if f.get("shared") is not None:
        out = out + clamped_expert(h, w, p + "shared.", f["shared"]["limit"])
    return out


# ---- the whole model -------------------------------------------------------------------------------
MIXERS = {"gla": gla_mixer, "attention": attention_mixer, "mlstm": mlstm_mixer}


def layer(x, w, i, spec, eps):
    p = f"l{i}."
    x = x + MIXERS[spec["type"]](rms_norm(x, w[p + "norm1"], eps, 1.0), w, p + "mix.", spec["mixer"], eps)
    f = spec.get("mlp")
    if f is None:
        return x
    h = rms_norm(x, w[p + "norm2"], eps, 1.0)
    return x + (dense_ff(h, w, p + "mlp.") if f["kind"] == "dense" else routed_ff(h, w, p + "mlp.", f))


def forward(tokens, tensors, cfg, dtype=torch.float64, keep_layers=False):
    """Logits ``[T, vocab]`` of one sequence (and the stream after every layer run, if asked)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x_emb = embedding(tokens, w, cfg)
    x = x_emb
    streams = []
    for i, p, begins in run_order(cfg):
        if begins:
            x = pass_entry(x, x_emb, w, p)
        x = layer(x, w, i, cfg["layers"][i], eps)
        if keep_layers:
            streams.append(x)
    logits = rms_norm(x, w["final.norm"], eps, 1.0) @ w["head"].T
    return (logits, torch.stack(streams)) if keep_layers else logits


def greedy(tokens, tensors, cfg, new_tokens, dtype=torch.float64):
    tokens = list(tokens)
    out = []
    for _ in range(new_tokens):
        out.append(int(forward(tokens, tensors, cfg, dtype)[-1].argmax()))
        tokens.append(out[-1])
    return out
