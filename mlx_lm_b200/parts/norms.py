"""Norms.  ``LayerNorm``: mean and biased variance over the last axis in
float32, gain and optional bias — what ``nn.LayerNorm(D, eps)`` is at its
call sites in mlx_lm/models/gpt2.py:92-96, 123."""

from __future__ import annotations

from typing import List

from .. import ops
from .base import VECTOR, Init, Norm, ParamSpec, register_part


class LayerNorm(Norm):
    replayable = True
    kernel_libs = ("norm",)

    def __init__(self, name: str, width: int, eps: float, bias: bool = True, gain_init: Init = Init(1.0, 0.0),
                 bias_init: Init = Init()):
        self.name, self.width, self.eps, self.has_bias = name, width, float(eps), bias
        self.gain_init, self.bias_init = gain_init, bias_init
        self.gain = self.bias = None

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec(self.name + ".weight", (self.width,), VECTOR, self.gain_init)]
        if self.has_bias:
            specs.append(ParamSpec(self.name + ".bias", (self.width,), VECTOR, self.bias_init))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        self.gain = tensors[self.name + ".weight"]
        self.bias = tensors[self.name + ".bias"] if self.has_bias else None

    def fold_args(self):
        return (self.gain, self.bias, self.eps)

    def forward(self, ctx, x, rows=None, tag: str = "normed"):
        n = x.shape[0] if rows is None else rows.numel()
        out = ctx.ws.get(tag, n, self.width, x.dtype)
        ops.label(self.name, 8.0 * n * self.width, 2.0 * x.element_size() * n * self.width)
        ops.layernorm(x, self.gain, self.bias, out, self.eps, ctx.stream, rows=rows)
        return out


register_part("norm", "layer_norm", LayerNorm)
