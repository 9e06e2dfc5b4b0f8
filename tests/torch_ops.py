"""A kernel set written with plain torch, for tests that run the engine's step function,
cache and parts without a GPU.  It is a test double: the product path has no such set and
refuses to run without its CUDA extension.  It follows the same calling conventions and
cache layout as the CUDA kernel set, and shares nothing with ``plain_gpt``.
"""

from __future__ import annotations

import math

import torch


class TorchOps:
    name = "torch-test-double"

    def embed(self, token_ids, positions, tok_emb, pos_table, scale=1.0):
        x = tok_emb.float()[token_ids.long()] * scale
        if pos_table is not None:
            x = x + pos_table.float()[positions.long()]
        return x

    def layernorm(self, x32, gain, shift, eps, out_dtype):
        mean = x32.mean(-1, keepdim=True)
        var = ((x32 - mean) ** 2).mean(-1, keepdim=True)
        y = (x32 - mean) * torch.rsqrt(var + eps) * gain
        if shift is not None:
            y = y + shift
        return y.to(out_dtype)

    def linear(self, x, weight, bias, activation, out_dtype):
        y = x.float() @ weight.float().T
        if bias is not None:
            y = y + bias
        if activation == "gelu_tanh":
            y = 0.5 * y * (1 + torch.tanh(math.sqrt(2 / math.pi) * (y + 0.044715 * y ** 3)))
        elif activation == "relu_sq":
            y = torch.relu(y) ** 2
        elif activation != "none":
            raise ValueError(activation)
        return y.to(out_dtype)

    def linear_residual(self, x, weight, bias, residual32):
        y = x.float() @ weight.float().T
        if bias is not None:
            y = y + bias
        residual32 += y

    def kv_store(self, qkv, n_head, n_kv_head, head_dim, cache, slot_mapping):
        N = qkv.shape[0]
        k = qkv[:, n_head * head_dim: (n_head + n_kv_head) * head_dim].reshape(N, n_kv_head, head_dim)
        v = qkv[:, (n_head + n_kv_head) * head_dim:].reshape(N, n_kv_head, head_dim)
        slots = slot_mapping.long()
        page, off = slots // cache.page_tokens, slots % cache.page_tokens
        cache.k_pages[page, :, off] = k.to(cache.k_pages.dtype)
        cache.v_pages[page, :, off] = v.to(cache.v_pages.dtype)

    def paged_attention(self, qkv, n_head, n_kv_head, head_dim, scale, cache, ctx):
        N = qkv.shape[0]
        q = qkv[:, : n_head * head_dim].reshape(N, n_head, head_dim).float()
        out = torch.zeros(N, n_head, head_dim)
        table = ctx.block_tables[cache.group].long()
        pt = cache.page_tokens
        for i in range(N):
            r = int(ctx.token_request[i])
            p = int(ctx.positions[i])
            lo = 0 if cache.window is None else max(0, p - cache.window + 1)
            keys = torch.arange(lo, p + 1)
            pages = table[r, keys // pt]
            assert (pages >= 0).all(), "attention reads a page that is not there"
            k = cache.k_pages[pages, :, keys % pt].float()      # [keys, Hkv, D]
            v = cache.v_pages[pages, :, keys % pt].float()
            for h in range(n_head):
                kh = h // (n_head // n_kv_head)
                s = (k[:, kh] @ q[i, h]) * scale
                out[i, h] = torch.softmax(s, dim=0) @ v[:, kh]
        return out.reshape(N, n_head * head_dim).to(qkv.dtype)

    def gather_rows(self, x32, rows):
        return x32[rows.long()]

    def logits(self, y, tok_emb, scale=1.0):
        return (y.float() @ tok_emb.float().T) * scale

    # ---- what the second architecture adds (same conventions as the CUDA kernel set) ---------------
    def head_prepare(self, proj, n_head, n_kv_head, head_dim, v_dim, q_off, k_off, v_off, unit_norm, eps,
                     cache, slots, positions, v_other=None, blend=None, q_gain=None, k_gain=None):
        n = proj.shape[0]
        live = positions >= 0

        def unit(x, gain=None):
            x = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) if unit_norm else x
            return x if gain is None else x * gain

        q = proj[:, q_off: q_off + n_head * head_dim].float().reshape(n, n_head, head_dim)
        v = proj[:, v_off: v_off + n_kv_head * v_dim].float()
        k = unit(proj[:, k_off: k_off + n_kv_head * head_dim].float().reshape(n, n_kv_head, head_dim), k_gain)
        if v_other is not None:
            v = (1.0 - blend[0]) * v + blend[0] * v_other.float()
        v = v.reshape(n, n_kv_head, v_dim)
        proj[live, q_off: q_off + n_head * head_dim] = unit(q, q_gain)[live].reshape(int(live.sum()), -1).to(proj.dtype)
        if cache is not None and cache.writes:
            keep = live & (slots >= 0)
            page, off = slots[keep].long() // cache.page_tokens, slots[keep].long() % cache.page_tokens
            cache.k_pages[page, :, off] = k[keep].to(cache.k_pages.dtype)
            cache.v_pages[page, :, off] = v[keep].to(cache.v_pages.dtype)

    def paged_attention_general(self, q, n_head, n_kv_head, head_dim, v_dim, scale, cache, ctx, gate=None,
                                slopes=None, block=None):
        n = q.shape[0]
        qh = q[:, : n_head * head_dim].reshape(n, n_head, head_dim).float()
        out = torch.zeros(n, n_head, v_dim)
        table = ctx.block_tables[cache.group].long()
        pt = cache.page_tokens
        for i in range(n):
            r, p = int(ctx.token_request[i]), int(ctx.positions[i])
            if p < 0:
                continue
            lo = 0 if cache.window is None else max(0, p - cache.window + 1)
            if block:
                lo = max(lo, p // block * block)
            keys = torch.arange(lo, p + 1)
            pages = table[r, keys // pt]
            assert (pages >= 0).all(), "attention reads a page that is not there"
            k = cache.k_pages[pages, :, keys % pt].float()
            v = cache.v_pages[pages, :, keys % pt].float()
            for h in range(n_head):
                kh = h // (n_head // n_kv_head)
                scores = (k[:, kh] @ qh[i, h]) * scale
                if slopes is not None:
                    scores = scores - slopes[h] * (p - keys).float()
                out[i, h] = torch.softmax(scores, dim=0) @ v[:, kh]
        out = out.reshape(n, n_head * v_dim)
        if gate is not None:
            out = out * torch.sigmoid(gate.float())
        return out.to(q.dtype)

    def moe_route(self, y, router_weight, gate_weight, positions, top):
        z = y.float() @ router_weight.float().T
        vals, ids = torch.topk(z, top, dim=-1)
        weights = torch.softmax(vals, dim=-1)
        ids = ids.to(torch.int32)
        ids[positions < 0] = -1
        gate = torch.sigmoid(y.float() @ gate_weight.float()) if gate_weight is not None else None
        return ids, weights, gate

    @staticmethod
    def _gated(a, u, activation, limit):
        if activation == "silu":
            return a * torch.sigmoid(a) * u
        if activation == "gelu_tanh":
            return 0.5 * a * (1 + torch.tanh(math.sqrt(2 / math.pi) * (a + 0.044715 * a ** 3))) * u
        if activation == "clamped_swish":
            a, u = a.clamp(max=limit), u.clamp(-limit, limit)
            return a * torch.sigmoid(1.702 * a) * (u + 1.0)
        raise ValueError(activation)

    def moe_experts_residual(self, y, ids, weights, w_in, w_out, residual32, activation="silu", limit=0.0):
        inner = w_in.shape[1] // 2
        for t in range(y.shape[0]):
            for k in range(ids.shape[1]):
                e = int(ids[t, k])
                if e < 0:
                    continue
                a = w_in[e].float() @ y[t].float()
                hidden = self._gated(a[:inner], a[inner:], activation, limit).to(y.dtype).float()
                residual32[t] += weights[t, k] * (w_out[e].float() @ hidden)

    def moe_route_scored(self, y, router_weight, gate_weight, positions, top, scoring, correction, groups, scale):
        z = y.float() @ router_weight.float().T
        n, experts = z.shape
        s = torch.sigmoid(z) if scoring == "sigmoid" else z
        choice = s if correction is None else s + correction
        if groups is not None:
            count, keep = groups
            per = experts // count
            grouped = choice.view(n, count, per)
            score = grouped.topk(min(2, per), dim=-1).values.sum(-1)
            allowed = torch.zeros(n, count, dtype=torch.bool).scatter_(1, score.topk(keep, dim=-1).indices, True)
            choice = grouped.masked_fill(~allowed[:, :, None], -math.inf).reshape(n, experts)
        ids = choice.topk(top, dim=-1).indices
        picked = s.gather(1, ids)
        weights = (picked if scoring == "sigmoid" else torch.softmax(picked, dim=-1)) * scale
        ids = ids.to(torch.int32)
        ids[positions < 0] = -1
        gate = torch.sigmoid(y.float() @ gate_weight.float()) if gate_weight is not None else None
        return ids, weights, gate

    def scale_(self, x32, scale):
        x32 *= scale
        return x32

    def clone(self, x):
        return x.clone()

    def embed_pairs(self, ctx, tok_emb, pair_emb, pos_table, buckets, mul_prev, mul_cur, state, source=None,
                    previous=None):
        ids = ctx.token_ids.long()
        x = tok_emb.float()[ids] + pos_table.float()[ctx.positions.long().clamp(min=0)]
        for r in range(ctx.num_requests):
            start, count = int(ctx.req_q_start[r]), int(ctx.req_q_len[r])
            slot = int(ctx.req_state_slot[r])
            if count == 0:
                continue
            before = None if int(ctx.req_ctx_before[r]) == 0 else int(state[slot, 0])
            for i in range(start, start + count):
                row = buckets if before is None else (before * mul_prev + int(ids[i]) * mul_cur) % buckets
                x[i] += pair_emb[row].float()
                before = int(ids[i])
            state[slot, 0] = before
        return x

    def rmsnorm(self, x32, weight, eps, offset, out_dtype):
        return (x32 / torch.sqrt((x32 * x32).mean(-1, keepdim=True) + eps) * (offset + weight)).to(out_dtype)

    def concat_cast(self, a32, b32, out_dtype):
        return torch.cat([a32, b32], dim=-1).to(out_dtype)

    def matrix_memory_scan(self, ctx, mode, proj, q_off, k_off, v_off, n_head, head_dim, v_dim, gates, constant, state):
        n = proj.shape[0]
        q = proj[:, q_off: q_off + n_head * head_dim].float().reshape(n, n_head, head_dim) * head_dim ** -0.5
        k = proj[:, k_off: k_off + n_head * head_dim].float().reshape(n, n_head, head_dim)
        v = proj[:, v_off: v_off + n_head * v_dim].float().reshape(n, n_head, v_dim)
        out = torch.zeros(n, n_head, v_dim)
        aux = torch.zeros(n, n_head, 2) if mode == "mlstm" else None
        cols = v_dim + (1 if mode == "mlstm" else 0)
        for r in range(ctx.num_requests):
            start, count = int(ctx.req_q_start[r]), int(ctx.req_q_len[r])
            if count == 0:
                continue
            slot = int(ctx.req_state_slot[r])
            flat = state[slot]
            S = flat[: n_head * cols * head_dim].view(n_head, cols, head_dim).clone()
            m = flat[n_head * cols * head_dim:].clone() if mode == "mlstm" else None
            if int(ctx.req_ctx_before[r]) == 0:
                S.zero_()
                if m is not None:
                    m.zero_()
            for i in range(start, start + count):
                if mode == "gla":
                    decay = torch.exp(torch.nn.functional.logsigmoid(gates[i].float()) / constant).view(n_head, head_dim)
                    S = decay[:, None, :] * S + v[i][:, :, None] * k[i][:, None, :]
                    out[i] = torch.einsum("hvd,hd->hv", S, q[i])
                else:
                    cap = constant
                    gi = cap * torch.tanh(gates[i, :n_head].float() / cap)
                    gf = torch.nn.functional.logsigmoid(cap * torch.tanh(gates[i, n_head:].float() / cap))
                    m_new = torch.maximum(gf + m, gi)
                    keep, take = torch.exp(gf + m - m_new), torch.exp(gi - m_new)
                    v1 = torch.cat([v[i], torch.ones(n_head, 1)], dim=1)
                    S = keep[:, None, None] * S + take[:, None, None] * v1[:, :, None] * k[i][:, None, :]
                    m = m_new
                    full = torch.einsum("hvd,hd->hv", S, q[i])
                    out[i] = full[:, :v_dim]
                    aux[i, :, 0], aux[i, :, 1] = full[:, v_dim], m
            flat[: n_head * cols * head_dim] = S.reshape(-1)
            if m is not None:
                flat[n_head * cols * head_dim:] = m
        return out.reshape(n, n_head * v_dim), aux

    def head_norm_gate(self, out32, aux, gate, gain, n_head, v_dim, eps, per_head_gain, gate_activation, out_dtype,
                       positions=None):
        n = out32.shape[0]
        o = out32.view(n, n_head, v_dim)
        if aux is not None:
            o = o / (torch.maximum(aux[:, :, 0].abs(), torch.exp(-aux[:, :, 1])) + 1e-6)[:, :, None]
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps)
        o = o * (gain.view(n_head, v_dim) if per_head_gain else gain)
        g = gate.float().view(n, n_head, v_dim)
        g = g * torch.sigmoid(g) if gate_activation == "silu" else torch.sigmoid(g)
        return (o * g).reshape(n, n_head * v_dim).to(out_dtype)

    def glu(self, gate_up, row_scale=None, activation="silu", limit=0.0):
        inner = gate_up.shape[1] // 2
        a, u = gate_up[:, :inner].float(), gate_up[:, inner:].float()
        out = self._gated(a, u, activation, limit)
        if row_scale is not None:
            out = out * row_scale[:, None]
        return out.to(gate_up.dtype)

    def argmax(self, logits, vocab_limit=None, out=None):
        v = logits if vocab_limit is None else logits[:, :vocab_limit]
        ids = v.argmax(-1).to(torch.int32)
        if out is None:
            return ids
        out.copy_(ids)
        return out
