"""Feed-forward of routed experts, with an optional expert that every token uses.

``z = W_router y`` in 32-bit; the ``top`` experts with the largest ``z`` are chosen and weighted
by the softmax over the chosen ``z`` alone.  An expert is a gated unit without biases,
``W_down (silu(W_gate y) * (W_up y))``; the part adds ``sum_k weight_k expert_k(y)`` to the
residual stream.  With ``shared_inner`` an expert of the same form (its own hidden width) runs for
every token and is added too, times ``sigmoid(w_sg . y)``, one number per token, if
``shared_gate``.

Variants, all parameters: ``scoring="sigmoid"`` scores every expert ``s = sigmoid(z)`` on its own and
weighs the chosen ones by ``route_scale * s`` without renormalising; ``correction`` adds a stored
vector to the scores for the choice only; ``groups=(count, keep)`` cuts the experts into ``count``
equal groups of neighbours, scores a group by the sum of its two largest choice scores and lets only
the experts of the best ``keep`` groups be chosen.  ``activation="clamped_swish"`` makes an expert
``W_down (g * sigmoid(1.702 g) * (u + 1))`` with ``g = min(W_gate y, limit)``,
``u = clamp(W_up y, -limit, limit)``; the shared expert has a limit of its own.

In the checkpoint expert ``e`` has ``e<e>.gate``, ``e<e>.up``, ``e<e>.down`` under the part's
prefix, the router ``router``, the shared expert ``shared.gate``, ``shared.up``, ``shared.down``
and ``shared.sg``.  When bound, the experts' matrices are stacked (``[E, 2F, C]`` with gate rows
first, ``[E, C, F]``), because the kernels walk them by expert number; the router and the shared
gate stay 32-bit.
"""

from __future__ import annotations

import torch

from .base import FeedForward, register_feed_forward
from .spec import TensorSpec


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True      # the tokens are grouped by expert on the device; the host decides nothing per step
    accepts_deferred_norm = False      # the router reads the normalised rows themselves

    def __init__(self, prefix: str, width: int, n_experts: int, top: int, inner: int,
                 shared_inner: int | None = None, shared_gate: bool = True, scoring: str = "softmax_top",
                 route_scale: float = 1.0, correction: bool = False, groups: tuple | None = None,
                 activation: str = "silu", limit: float = 0.0, shared_limit: float | None = None,
                 init: str = "normal") -> None:
        super().__init__(prefix)
        if not 0 < top <= n_experts:
            raise ValueError(f"top {top} must lie in 1..n_experts ({n_experts})")
        if scoring not in ("softmax_top", "sigmoid"):
            raise ValueError(f"scoring {scoring!r}: softmax_top or sigmoid")
        if activation not in ("silu", "clamped_swish"):
            raise ValueError(f"activation {activation!r}: silu or clamped_swish")
        if groups is not None:
            count, keep = groups
            if n_experts % count or not 0 < keep <= count or keep * (n_experts // count) < top:
                raise ValueError(f"groups {groups!r} do not fit {n_experts} experts with {top} choices")
        self.scoring, self.route_scale, self.has_correction = scoring, float(route_scale), bool(correction)
        self.groups = None if groups is None else (int(groups[0]), int(groups[1]))
        self.activation, self.limit = activation, float(limit)
        self.shared_limit = self.limit if shared_limit is None else float(shared_limit)
        self._init = init
        self.correction = None
        self.width, self.n_experts, self.top, self.inner = width, n_experts, top, inner
        self.shared_inner = shared_inner
        self.shared_gate = bool(shared_gate) and shared_inner is not None
        self.router = self.w_in = self.w_out = None
        self.shared_in = self.shared_out = self.shared_gate_weight = None

    def tensor_specs(self):
        p, c, f = self.prefix, self.width, self.inner
        init, init_out = self._init, ("residual_proj" if self._init == "normal" else self._init + "_residual")
        specs = {p + "router": TensorSpec((self.n_experts, c), "vector", init)}
        if self.has_correction:
            specs[p + "correction"] = TensorSpec((self.n_experts,), "vector", "norm_shift")
        for e in range(self.n_experts):
            specs[f"{p}e{e}.gate"] = TensorSpec((f, c), "matrix", init)
            specs[f"{p}e{e}.up"] = TensorSpec((f, c), "matrix", init)
            specs[f"{p}e{e}.down"] = TensorSpec((c, f), "matrix", init_out)
        if self.shared_inner is not None:
            s = self.shared_inner
            specs[p + "shared.gate"] = TensorSpec((s, c), "matrix", init)
            specs[p + "shared.up"] = TensorSpec((s, c), "matrix", init)
            specs[p + "shared.down"] = TensorSpec((c, s), "matrix", init_out)
            if self.shared_gate:
                specs[p + "shared.sg"] = TensorSpec((1, c), "vector", "normal")
        return specs

    def bind(self, tensors) -> None:
        p = self.prefix
        if tensors.get(p + "router") is None:
            return
        self.router = tensors[p + "router"]
        self.correction = tensors.get(p + "correction") if self.has_correction else None
        self.w_in = torch.stack([torch.cat([tensors[f"{p}e{e}.gate"], tensors[f"{p}e{e}.up"]], dim=0)
                                 for e in range(self.n_experts)]).contiguous()
        self.w_out = torch.stack([tensors[f"{p}e{e}.down"] for e in range(self.n_experts)]).contiguous()
        if self.shared_inner is not None:
            self.shared_in = torch.cat([tensors[p + "shared.gate"], tensors[p + "shared.up"]], dim=0).contiguous()
            self.shared_out = tensors[p + "shared.down"]
            if self.shared_gate:
                self.shared_gate_weight = tensors[p + "shared.sg"].reshape(-1).contiguous()

    def forward(self, ctx, y, residual32) -> None:
        ops = ctx.ops
        if self.scoring == "softmax_top" and not self.has_correction and self.groups is None:
            ids, weights, gate = ops.moe_route(y, self.router, self.shared_gate_weight, ctx.positions, self.top)
            if self.route_scale != 1.0:
                ops.scale_(weights, self.route_scale)
        else:
            ids, weights, gate = ops.moe_route_scored(y, self.router, self.shared_gate_weight, ctx.positions, self.top,
                                                      self.scoring, self.correction, self.groups, self.route_scale)
        plain = self.activation == "silu"
        ops.moe_experts_residual(y, ids, weights, self.w_in, self.w_out, residual32,
                                 **({} if plain else {"activation": self.activation, "limit": self.limit}))
        if self.shared_inner is not None:
            # the shared expert is an ordinary gated unit over all tokens: the projection kernels
            # serve it; its per-token gate rides on the hidden features (W (g h) = g (W h))
            hidden = ops.glu(ops.linear(y, self.shared_in, None, "none", ctx.act_dtype), gate,
                             **({} if plain else {"activation": self.activation, "limit": self.shared_limit}))
            ops.linear_residual(hidden, self.shared_out, None, residual32)
        return None
