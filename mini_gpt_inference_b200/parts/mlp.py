"""Dense feed-forward: ``proj(act(fc(y)))`` added into the residual stream.

The reference's MLP (src/minigpt_infer/model.py:93-101) with its hidden width and its
activation as parameters; ``gelu_tanh(u) = 0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3)))``
is evaluated in 32-bit inside the first projection's epilogue, and so is ``relu_sq(u) =
max(u, 0)^2``.  ``fc_name`` and ``proj_name`` name the two matrices inside the part's prefix
where they are not ``fc`` and ``proj`` (then without a ``.weight`` suffix).
"""

from __future__ import annotations

from .base import FeedForward, register_feed_forward
from .spec import TensorSpec

_ACTIVATIONS = {"gelu_tanh": "gelu_tanh", "gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh",
                "relu_sq": "relu_sq", "relu2": "relu_sq"}


@register_feed_forward("dense_mlp")
class DenseMLP(FeedForward):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step

    def __init__(self, prefix: str, width: int, inner: int, bias: bool,
                 activation: str = "gelu_tanh", fc_name: str | None = None,
                 proj_name: str | None = None) -> None:
        super().__init__(prefix)
        if activation not in _ACTIVATIONS:
            raise ValueError(f"activation {activation!r} has no kernel epilogue; known: "
                             + ", ".join(sorted(_ACTIVATIONS)))
        self.width, self.inner, self.has_bias = width, inner, bool(bias)
        self.activation = _ACTIVATIONS[activation]
        self.fc_weight = self.fc_bias = self.proj_weight = self.proj_bias = None
        p = self.prefix
        self._names = {
            "fc_weight": p + (fc_name if fc_name is not None else "fc.weight"),
            "proj_weight": p + (proj_name if proj_name is not None else "proj.weight"),
            "fc_bias": p + (fc_name + ".bias" if fc_name is not None else "fc.bias"),
            "proj_bias": p + (proj_name + ".bias" if proj_name is not None else "proj.bias"),
        }

    def tensor_specs(self):
        n = self._names
        specs = {
            n["fc_weight"]: TensorSpec((self.inner, self.width), "matrix"),
            n["proj_weight"]: TensorSpec((self.width, self.inner), "matrix", "residual_proj"),
        }
        if self.has_bias:
            specs[n["fc_bias"]] = TensorSpec((self.inner,), "vector", "bias")
            specs[n["proj_bias"]] = TensorSpec((self.width,), "vector", "bias")
        return specs

    def bind(self, tensors) -> None:
        for attr, name in self._names.items():
            setattr(self, attr, tensors.get(name))

    accepts_deferred_norm = True

    def forward(self, ctx, y, residual32):
        whole = getattr(ctx.ops, "mlp_residual", None)
        if whole is not None:
            # the kernel set may run both projections as one kernel; it returns where the sum lies
            return whole(y, self.fc_weight, self.fc_bias, self.proj_weight, self.proj_bias, self.activation,
                         residual32, ctx.act_dtype)
        h = ctx.ops.linear(y, self.fc_weight, self.fc_bias, self.activation, ctx.act_dtype)
        ctx.ops.linear_residual(h, self.proj_weight, self.proj_bias, residual32)
        return None


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    """``down(act(gate(y)) * up(y))`` added into the residual stream, without biases.  ``activation``:
    ``gelu_tanh`` or ``silu``, evaluated in 32-bit.  The gate's and the up matrix are joined when bound, so
    a step runs one projection, the gated product and the second projection."""

    graph_safe = True
    accepts_deferred_norm = True

    def __init__(self, prefix: str, width: int, inner: int, activation: str = "gelu_tanh",
                 gate_name: str = "gate", up_name: str = "up", down_name: str = "down") -> None:
        super().__init__(prefix)
        if activation not in ("gelu_tanh", "silu"):
            raise ValueError(f"activation {activation!r} is not a gated unit's; known: gelu_tanh, silu")
        self.width, self.inner, self.activation = width, inner, activation
        p = self.prefix
        self._names = {"gate": p + gate_name, "up": p + up_name, "down": p + down_name}
        self.in_weight = self.down_weight = None

    def tensor_specs(self):
        n = self._names
        return {n["gate"]: TensorSpec((self.inner, self.width), "matrix", "fan_in"),
                n["up"]: TensorSpec((self.inner, self.width), "matrix", "fan_in"),
                n["down"]: TensorSpec((self.width, self.inner), "matrix", "fan_in_residual")}

    def bind(self, tensors) -> None:
        import torch

        gate, up = tensors.get(self._names["gate"]), tensors.get(self._names["up"])
        self.in_weight = torch.cat([gate, up], dim=0).contiguous() if gate is not None and up is not None else None
        self.down_weight = tensors.get(self._names["down"])

    def forward(self, ctx, y, residual32):
        ops = ctx.ops
        hidden = ops.glu(ops.linear(y, self.in_weight, None, "none", ctx.act_dtype), activation=self.activation)
        ops.linear_residual(hidden, self.down_weight, None, residual32)
        return None
