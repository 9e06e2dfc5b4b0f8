"""Causal attention with unit-RMS queries and keys, an output gate and blended values.

One fused projection gives ``[q | k | v | g]`` of a token: ``n_head`` query heads and
``n_kv_head`` key heads of ``head_dim`` features, ``n_kv_head`` value heads of
``v_head_dim`` features (keys and values may differ in size) and, with ``gate``, one gate
value per output feature.  Then, per token:

* ``unit_norm``: every query and key head is divided by its root mean square,
  ``u / sqrt(mean(u^2) + eps)``, in 32-bit, without a gain;
* ``value_blend``: ``"source"`` publishes this layer's values for the layers after it,
  ``"blend"`` replaces ``v`` by ``(1 - t) v + t v_source`` with the published values of the
  same token and this layer's own scalar ``t``; the blended values are what the cache holds;
* keys and values go to their pages, and every query attends to the keys of its own request
  at positions up to its own, ``softmax(scale * q . k)`` in 32-bit, read from the pages
  whichever step brought them;
* ``gate``: the concatenated heads are multiplied by ``sigmoid(g)`` before the output
  projection, which adds into the residual stream.

Further variants, all parameters: ``bias`` (the q, k and output projections have biases, named after
their matrices with ``.b``); ``norm_weights`` (the unit-RMS query and key heads are multiplied by a
stored gain of ``head_dim`` numbers each, shared by the heads, named ``q.norm`` and ``k.norm``);
``values="keys"`` (there is no value projection: a token's values are its keys as projected, before
their norm); ``slope_rate`` (a distance bias: ``slope_h * (i - j)`` is taken off the score of query
``i`` and key ``j``, ``slope_h = 2 ** (-slope_rate * (h + 1) / n_head)``); ``block_mask`` (a query sees
only the keys of its own block of that many positions, blocks counted from position 0: the cache
gives back the pages of blocks that are over).

Positions do not enter otherwise unless the model's position encoding rotates q and k.  The four
matrices are stored apart in the checkpoint (``q``, ``k``, ``v``, ``g``, then ``o`` and the
scalar ``vmix``, under names given by ``names``) and joined once when they are bound.
"""

from __future__ import annotations

import math

import torch

from ..cache.spec import PagedKVSpec
from .base import Mixer, register_mixer
from .spec import TensorSpec

_DEFAULT_NAMES = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "blend": "vmix"}
VALUE_SOURCE = "attention_value_source"     # key in ctx.shared


@register_mixer("gated_unit_attention")
class GatedUnitAttention(Mixer):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step
    accepts_deferred_norm = True

    def __init__(self, prefix: str, width: int, n_head: int, head_dim: int, n_kv_head: int | None = None,
                 v_head_dim: int | None = None, scale: float | None = None, eps: float = 1e-6,
                 unit_norm: bool = True, gate: bool = True, value_blend: str | None = None,
                 blend_tensor: bool = False, window: int | None = None,
                 cache_page_tokens: int | None = None, cache_pages: int | None = None,
                 names: dict | None = None, position=None, bias: bool = False, norm_weights: bool = False,
                 values: str = "projected", slope_rate: float | None = None, block_mask: int | None = None,
                 init: str = "normal") -> None:
        super().__init__(prefix)
        self.width, self.n_head, self.head_dim = width, n_head, head_dim
        self.n_kv_head = n_head if n_kv_head is None else n_kv_head
        self.v_head_dim = head_dim if v_head_dim is None else v_head_dim
        if self.n_head % self.n_kv_head != 0:
            raise ValueError(f"n_head {n_head} is not a multiple of n_kv_head {self.n_kv_head}")
        if value_blend not in (None, "source", "blend"):
            raise ValueError(f"value_blend {value_blend!r}: None, 'source' or 'blend'")
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.eps, self.unit_norm, self.has_gate = float(eps), bool(unit_norm), bool(gate)
        self.value_blend = value_blend
        # whether a layer that does not blend may still carry the scalar in its checkpoint
        self.has_blend_tensor = bool(blend_tensor)
        self.window = window
        if values not in ("projected", "keys"):
            raise ValueError(f"values {values!r}: 'projected' or 'keys'")
        if values == "keys" and (self.v_head_dim != head_dim or value_blend is not None):
            raise ValueError("values that are the keys have the keys' size and are not blended")
        if norm_weights and not unit_norm:
            raise ValueError("norm_weights without unit_norm")
        self.has_bias, self.has_norm_weights, self.values_are_keys = bool(bias), bool(norm_weights), values == "keys"
        self.slope_rate = None if slope_rate is None else float(slope_rate)
        self.block_mask = block_mask
        self._init = init
        self.cache_page_tokens, self.cache_pages = cache_page_tokens, cache_pages
        self.position = position
        self.names = {**_DEFAULT_NAMES, **(names or {})}
        self.q_width = n_head * head_dim
        self.k_width = self.n_kv_head * head_dim
        self.v_width = self.n_kv_head * self.v_head_dim
        self.o_width = n_head * self.v_head_dim
        self.k_off, self.v_off = self.q_width, self.q_width + self.k_width
        if self.values_are_keys:
            self.v_off, self.g_off = self.k_off, self.k_off + self.k_width
        else:
            self.g_off = self.v_off + self.v_width
        self.fused_weight = self.out_weight = self.blend = None
        self.fused_bias = self.out_bias = self.q_gain = self.k_gain = self.slopes = None

    def _name(self, which: str) -> str:
        return self.prefix + self.names[which]

    def tensor_specs(self):
        init, init_out = self._init, ("residual_proj" if self._init == "normal" else self._init + "_residual")
        specs = {
            self._name("q"): TensorSpec((self.q_width, self.width), "matrix", init),
            self._name("k"): TensorSpec((self.k_width, self.width), "matrix", init),
            self._name("out"): TensorSpec((self.width, self.o_width), "matrix", init_out),
        }
        if not self.values_are_keys:
            specs[self._name("v")] = TensorSpec((self.v_width, self.width), "matrix", init)
        if self.has_bias:
            specs[self._name("q") + ".b"] = TensorSpec((self.q_width,), "vector", "norm_shift")
            specs[self._name("k") + ".b"] = TensorSpec((self.k_width,), "vector", "norm_shift")
            specs[self._name("out") + ".b"] = TensorSpec((self.width,), "vector", "bias")
        if self.has_norm_weights:
            specs[self._name("q") + ".norm"] = TensorSpec((self.head_dim,), "vector", "norm_gain")
            specs[self._name("k") + ".norm"] = TensorSpec((self.head_dim,), "vector", "norm_gain")
        if self.has_gate:
            specs[self._name("gate")] = TensorSpec((self.o_width, self.width), "matrix")
        if self.value_blend is not None or self.has_blend_tensor:
            # a layer that does not blend may still find the scalar in its checkpoint, unused
            specs[self._name("blend")] = TensorSpec((), "vector", "unit_interval",
                                                    optional=self.value_blend is None)
        return specs

    def bind(self, tensors) -> None:
        rows = [tensors.get(self._name(w)) for w in (("q", "k") if self.values_are_keys else ("q", "k", "v"))]
        if self.has_gate:
            rows.append(tensors.get(self._name("gate")))
        # one matrix for the step's one projection: a layout made once, when the weights arrive
        self.fused_weight = torch.cat(rows, dim=0).contiguous() if all(r is not None for r in rows) else None
        self.out_weight = tensors.get(self._name("out"))
        if self.has_bias and self.fused_weight is not None:
            qb, kb = tensors.get(self._name("q") + ".b"), tensors.get(self._name("k") + ".b")
            self.fused_bias = torch.zeros(self.fused_weight.shape[0], dtype=torch.float32, device=self.fused_weight.device)
            self.fused_bias[: self.q_width] = qb
            self.fused_bias[self.k_off: self.k_off + self.k_width] = kb
            self.out_bias = tensors.get(self._name("out") + ".b")
        if self.has_norm_weights:
            self.q_gain, self.k_gain = tensors.get(self._name("q") + ".norm"), tensors.get(self._name("k") + ".norm")
        if self.slope_rate is not None and self.out_weight is not None:
            slopes = [2.0 ** (-self.slope_rate * (h + 1) / self.n_head) for h in range(self.n_head)]
            self.slopes = torch.tensor(slopes, dtype=torch.float64).to(dtype=torch.float32, device=self.out_weight.device)
        blend = tensors.get(self._name("blend")) if self.value_blend == "blend" else None
        self.blend = blend.reshape(1).contiguous() if blend is not None else None

    def cache_spec(self):
        return PagedKVSpec(self.n_kv_head, self.head_dim, self.window, self.cache_page_tokens,
                           self.cache_pages,
                           None if self.v_head_dim == self.head_dim else self.v_head_dim, self.block_mask)

    def plan_step(self, batch, plan, ops) -> None:
        # where keys and values have one size, the kernel set may cut prompt portions into the tiles of
        # its tiled attention kernel (the same work list as the plain causal attention's)
        planner = getattr(ops, "plan_prompt_attention", None)
        if planner is not None and self.head_dim == self.v_head_dim and self.slopes is None and self.block_mask is None:
            planner(batch, plan, self.n_head, self.n_kv_head, self.head_dim)

    def forward(self, ctx, cache, y, residual32) -> None:
        ops = ctx.ops
        proj = ops.linear(y, self.fused_weight, self.fused_bias, "none", ctx.act_dtype)
        if self.position is not None:
            self.position.rotate(ctx, proj, self.n_head, self.n_kv_head, self.head_dim)
        other = blend = None
        if self.value_blend == "blend":
            other = ctx.shared.get(VALUE_SOURCE)
            if other is None:
                raise RuntimeError(f"{self.prefix}: no layer before this one published its values")
            if other.shape[1] != self.v_width:
                raise RuntimeError(f"{self.prefix}: the published values have another size")
            blend = self.blend
        elif self.value_blend == "source":
            ctx.shared[VALUE_SOURCE] = proj[:, self.v_off: self.v_off + self.v_width]
        extra = {"q_gain": self.q_gain, "k_gain": self.k_gain} if self.has_norm_weights else {}
        ops.head_prepare(proj, self.n_head, self.n_kv_head, self.head_dim, self.v_head_dim, 0, self.k_off,
                         self.v_off, self.unit_norm, self.eps, cache, ctx.slot_mapping[cache.group],
                         ctx.positions, v_other=other, blend=blend, **extra)
        gate = proj[:, self.g_off: self.g_off + self.o_width] if self.has_gate else None
        extra = {}
        if self.slopes is not None:
            extra["slopes"] = self.slopes
        if self.block_mask is not None:
            extra["block"] = self.block_mask
        out = ops.paged_attention_general(proj, self.n_head, self.n_kv_head, self.head_dim, self.v_head_dim,
                                          self.scale, cache, ctx, gate=gate, **extra)
        ops.linear_residual(out, self.out_weight, self.out_bias, residual32)
