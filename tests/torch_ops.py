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
                     cache, slots, positions, v_other=None, blend=None):
        n = proj.shape[0]
        live = positions >= 0

        def unit(x):
            return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) if unit_norm else x

        q = proj[:, q_off: q_off + n_head * head_dim].float().reshape(n, n_head, head_dim)
        k = unit(proj[:, k_off: k_off + n_kv_head * head_dim].float().reshape(n, n_kv_head, head_dim))
        v = proj[:, v_off: v_off + n_kv_head * v_dim].float()
        if v_other is not None:
            v = (1.0 - blend[0]) * v + blend[0] * v_other.float()
        v = v.reshape(n, n_kv_head, v_dim)
        proj[live, q_off: q_off + n_head * head_dim] = unit(q)[live].reshape(int(live.sum()), -1).to(proj.dtype)
        if cache is not None and cache.writes:
            keep = live & (slots >= 0)
            page, off = slots[keep].long() // cache.page_tokens, slots[keep].long() % cache.page_tokens
            cache.k_pages[page, :, off] = k[keep].to(cache.k_pages.dtype)
            cache.v_pages[page, :, off] = v[keep].to(cache.v_pages.dtype)

    def paged_attention_general(self, q, n_head, n_kv_head, head_dim, v_dim, scale, cache, ctx, gate=None):
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
            keys = torch.arange(lo, p + 1)
            pages = table[r, keys // pt]
            assert (pages >= 0).all(), "attention reads a page that is not there"
            k = cache.k_pages[pages, :, keys % pt].float()
            v = cache.v_pages[pages, :, keys % pt].float()
            for h in range(n_head):
                kh = h // (n_head // n_kv_head)
                out[i, h] = torch.softmax((k[:, kh] @ qh[i, h]) * scale, dim=0) @ v[:, kh]
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

    def moe_experts_residual(self, y, ids, weights, w_in, w_out, residual32):
        inner = w_in.shape[1] // 2
        for t in range(y.shape[0]):
            for k in range(ids.shape[1]):
                e = int(ids[t, k])
                if e < 0:
                    continue
                a = w_in[e].float() @ y[t].float()
                hidden = a[:inner] * torch.sigmoid(a[:inner]) * a[inner:]
                residual32[t] += weights[t, k] * (w_out[e].float() @ hidden)

    def glu(self, gate_up, row_scale=None):
        inner = gate_up.shape[1] // 2
        a, u = gate_up[:, :inner].float(), gate_up[:, inner:].float()
        out = a * torch.sigmoid(a) * u
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
