"""LayerNorm over the width, statistics in 32-bit.

``y = (x - mean) / sqrt(var + eps) * gain (+ shift)`` with the biased variance, as
``nn.LayerNorm`` in src/minigpt_infer/model.py:107-109, 127 (eps there is the library
default 1e-5; here it is a parameter).  The shift exists only if ``bias``.  ``gain_name`` and
``shift_name`` name the two tensors in the checkpoint where they are not ``<prefix>weight`` and
``<prefix>bias``.
"""

from __future__ import annotations

from .base import Norm, register_norm
from .spec import TensorSpec


@register_norm("layernorm")
class LayerNorm(Norm):
    graph_safe = True      # launches kernels only; nothing is decided on the host per step

    def __init__(self, prefix: str, width: int, eps: float, bias: bool, gain_name: str | None = None,
                 shift_name: str | None = None, optional: bool = False) -> None:
        super().__init__(prefix)
        self.width, self.eps, self.has_bias = width, float(eps), bool(bias)
        self.gain_name = gain_name if gain_name is not None else self.prefix + "weight"
        self.shift_name = shift_name if shift_name is not None else self.prefix + "bias"
        self.optional = bool(optional)     # a norm that a layer carries but never runs
        self.weight = None
        self.bias = None

    def tensor_specs(self):
        specs = {self.gain_name: TensorSpec((self.width,), "vector", "norm_gain", optional=self.optional)}
        if self.has_bias:
            specs[self.shift_name] = TensorSpec((self.width,), "vector", "norm_shift", optional=self.optional)
        return specs

    def bind(self, tensors) -> None:
        self.weight = tensors.get(self.gain_name)
        self.bias = tensors.get(self.shift_name) if self.has_bias else None

    def forward(self, ctx, x32):
        return ctx.ops.layernorm(x32, self.weight, self.bias, self.eps, ctx.act_dtype)

    def defer(self, ctx, x32, rows=None):
        if not hasattr(ctx.ops, "defer_layernorm"):
            return super().defer(ctx, x32, rows)
        return ctx.ops.defer_layernorm(x32, self.weight, self.bias, self.eps, ctx.act_dtype, rows)
