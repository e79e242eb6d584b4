"""Norms.  ``LayerNorm``: mean and biased variance over the last axis in
float32, gain and optional bias — what ``nn.LayerNorm(D, eps)`` is at its
call sites in mlx_lm/models/gpt2.py:92-96, 123."""

from __future__ import annotations

from typing import List, Optional

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


class RMSNorm(Norm):
    """``x / sqrt(mean(x^2) + eps) * (offset + weight)`` over float32 rows, result in the run's dtype.
    ``offset = 1``: the weight is stored as its distance from one; ``offset = 0``: as it is."""
    replayable = True
    kernel_libs = ("rms",)

    def __init__(self, name: str, width: int, eps: float, offset: float = 0.0, weight_suffix: str = "",
                 init: Optional[Init] = None):
        self.name, self.width, self.eps, self.offset = name, width, float(eps), float(offset)
        self.weight_name = name + weight_suffix
        self.init = init if init is not None else Init(1.0 - self.offset, 0.1)
        self.weight = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.weight_name, (self.width,), VECTOR, self.init)]

    def bind(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.weight_name]

    def forward(self, ctx, x, rows=None, tag: str = "normed"):
        n = x.shape[0] if rows is None else rows.numel()
        out = ctx.ws.get(tag, n, self.width, ctx.dtype)
        ops.label(self.name, 4.0 * n * self.width, (4.0 + out.element_size()) * n * self.width)
        ops.rmsnorm(x, self.weight, out, self.eps, ctx.stream, offset=self.offset, rows=rows)
        return out


class DynamicTanh(Norm):
    """A norm without statistics: ``tanh(alpha * x) * weight + bias`` element by element, with one learned number
    ``alpha`` (``<name>.alpha``, no shape), a weight ``<name>`` and a bias ``<name>.b`` per column.  Reads float32
    rows, computes in float32, gives the run's dtype.  ``out_scale`` multiplies the result before it is rounded (a
    model whose logits are scaled hands that factor to its final norm).  Being elementwise it can also run inside
    the update of the residual stream (``SandwichBlock``): ``stream_args()`` gives ``(alpha, weight, bias)``."""
    replayable = True
    kernel_libs = ("dyt",)

    def __init__(self, name: str, width: int, bias: bool = True, out_scale: float = 1.0, alpha_init: Init = Init(1.0, 0.2),
                 weight_init: Init = Init(1.0, 0.1), bias_init: Init = Init(0.0, 0.1)):
        self.name, self.width, self.has_bias, self.out_scale = name, width, bias, float(out_scale)
        self.alpha_init, self.weight_init, self.bias_init = alpha_init, weight_init, bias_init
        self.alpha = self.weight = self.bias = None

    def param_specs(self) -> List[ParamSpec]:
        specs = [ParamSpec(self.name, (self.width,), VECTOR, self.weight_init)]
        if self.has_bias:
            specs.append(ParamSpec(self.name + ".b", (self.width,), VECTOR, self.bias_init))
        specs.append(ParamSpec(self.name + ".alpha", (), VECTOR, self.alpha_init))
        return specs

    def bind(self, tensors, dtype, device) -> None:
        self.weight = tensors[self.name]
        self.bias = tensors[self.name + ".b"] if self.has_bias else None
        self.alpha = tensors[self.name + ".alpha"].reshape(1)

    def stream_args(self):
        if self.out_scale != 1.0:
            raise ValueError(f"{self.name}: a norm with an output scale does not run inside a stream update")
        return (self.alpha, self.weight, self.bias)

    def forward(self, ctx, x, rows=None, tag: str = "normed"):
        n = x.shape[0] if rows is None else rows.numel()
        out = ctx.ws.get(tag, n, self.width, ctx.dtype)
        ops.label(self.name, 10.0 * n * self.width, (4.0 + out.element_size()) * n * self.width)
        ops.dyt_norm(x, self.alpha, self.weight, self.bias, out, ctx.stream, rows=rows, out_scale=self.out_scale)
        return out


register_part("norm", "layer_norm", LayerNorm)
register_part("norm", "dynamic_tanh", DynamicTanh)
register_part("norm", "rms_norm", RMSNorm)
