"""Mixers whose memory is a matrix per head, carried from token to token: gated linear attention and
the matrix memory of xLSTM (mLSTM).

Both project ``q`` and ``k`` (``n_head x head_dim``, ``q`` times ``head_dim ** -0.5``), ``v`` and an
output gate ``g`` (``n_head x v_head_dim``), keep per head a state ``S`` of ``head_dim x v_head_dim``
numbers in 32-bit in the request's slot of the state pool, and read ``o_t = S_t^T q_t``.

``gated_linear_attention``: ``S_t = diag(a_t) S_(t-1) + k_t v_t^T`` with one decay per key channel,
``a = sigmoid(z) ** (1 / tau)``, ``z = W_a2 (W_a1 h) + b`` (a product of two thin matrices whose inner
size the checkpoint gives).  Every head's ``o`` is RMS-normed over its features with a gain shared by
the heads, the heads are multiplied by ``silu(g)`` and projected.

``mlstm``: scalar gates per head, ``i = cap * tanh(x_i / cap)`` and ``f = logsigmoid(cap * tanh(x_f /
cap))`` (logarithms of the input and forget gates), a running maximum ``m_t = max(f + m_(t-1), i)``
that starts at 0, ``S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k_t v_t^T``, ``n_t`` the same
with ``k_t`` alone, ``o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)``.  Every head's ``o`` is
divided by its root mean square, the concatenated heads are multiplied by a gain of their whole
size and by ``sigmoid(g)`` and projected.

Decays, gates, their exponentials, the state and the norms are 32-bit whatever the compute dtype.
The state starts at zero when a request brings its first token; nothing else distinguishes a prompt
portion from a decoded token.
"""

from __future__ import annotations

import torch

from ..cache.spec import FixedStateSpec
from .base import Mixer, register_mixer
from .spec import TensorSpec


class _MatrixMemoryMixer(Mixer):
    graph_safe = True      # launches kernels only; the state slot and the token counts are read on the device
    accepts_deferred_norm = True
    mode = ""

    def __init__(self, prefix: str, width: int, n_head: int, head_dim: int, v_head_dim: int, eps: float,
                 position=None) -> None:
        super().__init__(prefix)
        self.width, self.n_head, self.head_dim, self.v_head_dim = width, n_head, head_dim, v_head_dim
        self.eps = float(eps)
        self.qk_width, self.v_width = n_head * head_dim, n_head * v_head_dim
        self.k_off, self.v_off, self.g_off = self.qk_width, 2 * self.qk_width, 2 * self.qk_width + self.v_width
        self.fused_weight = self.out_weight = self.norm_gain = None

    def _main_specs(self):
        p, c = self.prefix, self.width
        return {p + "q": TensorSpec((self.qk_width, c), "matrix", "fan_in"),
                p + "k": TensorSpec((self.qk_width, c), "matrix", "fan_in"),
                p + "v": TensorSpec((self.v_width, c), "matrix", "fan_in"),
                p + "g": TensorSpec((self.v_width, c), "matrix", "fan_in"),
                p + "o": TensorSpec((c, self.v_width), "matrix", "fan_in_residual")}

    def _bind_main(self, tensors) -> bool:
        p = self.prefix
        rows = [tensors.get(p + n) for n in ("q", "k", "v", "g")]
        if any(r is None for r in rows):
            return False
        self.fused_weight = torch.cat(rows, dim=0).contiguous()
        self.out_weight = tensors.get(p + "o")
        self.norm_gain = tensors.get(p + "norm")
        return True

    def plan_step(self, batch, plan, ops) -> None:
        # the kernel set may cut prompt portions into chunks that it scans side by side
        planner = getattr(ops, "plan_memory_chunks", None)
        if planner is not None:
            planner(batch, plan, self.head_dim, self.v_head_dim, self.mode == "mlstm")

    def _finish(self, ctx, proj, memory_out, aux, residual32, per_head_gain: bool, gate_activation: str):
        gate = proj[:, self.g_off: self.g_off + self.v_width]
        heads = ctx.ops.head_norm_gate(memory_out, aux, gate, self.norm_gain, self.n_head, self.v_head_dim,
                                       self.eps, per_head_gain, gate_activation, ctx.act_dtype,
                                       positions=ctx.positions)
        ctx.ops.linear_residual(heads, self.out_weight, None, residual32)


@register_mixer("gated_linear_attention")
class GatedLinearAttention(_MatrixMemoryMixer):
    mode = "gla"
    DEFAULT_DECAY_RANK = 16      # what random-weights mode gives the two decay matrices (a checkpoint's shapes win)

    def __init__(self, prefix: str, width: int, n_head: int, head_dim: int, v_head_dim: int, tau: float,
                 eps: float, position=None) -> None:
        super().__init__(prefix, width, n_head, head_dim, v_head_dim, eps)
        self.tau = float(tau)
        self.decay_in = self.decay_out = self.decay_bias = None

    def tensor_specs(self):
        p, r = self.prefix, self.DEFAULT_DECAY_RANK
        specs = self._main_specs()
        specs[p + "norm"] = TensorSpec((self.v_head_dim,), "vector", "norm_gain")
        specs[p + "a1"] = TensorSpec((-1, self.width), "matrix", "fan_in", fill=(r, self.width))
        specs[p + "a2"] = TensorSpec((self.qk_width, -1), "matrix", "fan_in", fill=(self.qk_width, r))
        specs[p + "a2.b"] = TensorSpec((self.qk_width,), "vector", "unit_normal")
        return specs

    def bind(self, tensors) -> None:
        if not self._bind_main(tensors):
            return
        p = self.prefix
        self.decay_in, self.decay_out, self.decay_bias = tensors[p + "a1"], tensors[p + "a2"], tensors[p + "a2.b"]
        if self.decay_in.shape[0] != self.decay_out.shape[1]:
            raise ValueError(f"{p}a1 {tuple(self.decay_in.shape)} and {p}a2 {tuple(self.decay_out.shape)} "
                             "do not share their inner size")

    def cache_spec(self):
        return FixedStateSpec((self.n_head * self.v_head_dim * self.head_dim,), "float32")

    def forward(self, ctx, cache, y, residual32) -> None:
        ops = ctx.ops
        if hasattr(y, "materialize"):
            y = y.materialize()                      # three projections read the normalised rows
        proj = ops.linear(y, self.fused_weight, None, "none", ctx.act_dtype)
        thin = ops.linear(y, self.decay_in, None, "none", ctx.act_dtype)
        z = ops.linear(thin, self.decay_out, self.decay_bias, "none", torch.float32)
        out, aux = ops.matrix_memory_scan(ctx, "gla", proj, 0, self.k_off, self.v_off, self.n_head, self.head_dim,
                                          self.v_head_dim, z, self.tau, cache.state)
        self._finish(ctx, proj, out, aux, residual32, False, "silu")


@register_mixer("mlstm")
class MLSTM(_MatrixMemoryMixer):
    mode = "mlstm"

    def __init__(self, prefix: str, width: int, n_head: int, head_dim: int, v_head_dim: int, gate_cap: float,
                 eps: float, position=None) -> None:
        super().__init__(prefix, width, n_head, head_dim, v_head_dim, eps)
        self.gate_cap = float(gate_cap)
        self.gate_weight = self.gate_bias = None

    def tensor_specs(self):
        p = self.prefix
        specs = self._main_specs()
        specs[p + "norm"] = TensorSpec((self.v_width,), "vector", "norm_gain")
        for name in ("i", "f"):
            specs[p + name] = TensorSpec((self.n_head, self.width), "matrix", "fan_in")
            specs[p + name + ".b"] = TensorSpec((self.n_head,), "vector", "unit_normal")
        return specs

    def bind(self, tensors) -> None:
        if not self._bind_main(tensors):
            return
        p = self.prefix
        self.gate_weight = torch.cat([tensors[p + "i"], tensors[p + "f"]], dim=0).contiguous()
        self.gate_bias = torch.cat([tensors[p + "i.b"], tensors[p + "f.b"]], dim=0).contiguous()

    def cache_spec(self):
        # per head: head_dim x (v_head_dim + 1) numbers (the last column is the normaliser n) and the maximum m
        return FixedStateSpec((self.n_head * (self.v_head_dim + 1) * self.head_dim + self.n_head,), "float32")

    def forward(self, ctx, cache, y, residual32) -> None:
        ops = ctx.ops
        if hasattr(y, "materialize"):
            y = y.materialize()
        proj = ops.linear(y, self.fused_weight, None, "none", ctx.act_dtype)
        gates = ops.linear(y, self.gate_weight, self.gate_bias, "none", torch.float32)
        out, aux = ops.matrix_memory_scan(ctx, "mlstm", proj, 0, self.k_off, self.v_off, self.n_head, self.head_dim,
                                          self.v_head_dim, gates, self.gate_cap, cache.state)
        self._finish(ctx, proj, out, aux, residual32, True, "sigmoid")
