"""Norms."""
from __future__ import annotations

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import Norm, register_part


@register_part("norm", "rms")
class RMSNorm(Norm):
    """y = x * w / sqrt(mean(x^2) + eps): the weight multiplies (no 1 + w), no bias
    (reference: src/kernels/rmsnorm.cpp:10-17).  Input is the float32 residual stream, sums
    are float32, the output has the activation type."""

    def __init__(self, width: int, eps: float):
        self.width, self.eps = int(width), float(eps)
        self.weight = None

    def weight_specs(self):
        return [WeightSpec("weight", (self.width,), "vector", ("one_plus_normal", 0.05))]

    def bind(self, tensors, rt):
        self.weight = tensors["weight"].float().contiguous()

    def forward(self, x, rt, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = rt.arena.alloc((n, self.width), rt.dtype)
        rt.launches += 1
        ops.rmsnorm(x, self.weight, out, self.eps, rows)
        return out

    def add_normed(self, y, x, rt, h=None, clear=False):
        """x += norm(y), for layers that norm a sublayer's output instead of its input; x, y float32
        [T, width].  ``h`` receives the new x in h's type (the next sublayer's input); ``clear`` zeroes y."""
        rt.launches += 1
        ops.rmsnorm_add(y, self.weight, x, self.eps, h=h, clear_y=clear)


@register_part("norm", "layer")
class LayerNorm(Norm):
    """y = (x - mean) / sqrt(var + eps) * w, the variance being the mean of the squared deviations; a weight and no
    bias.  ``scale``: a constant folded into the weight (a model that multiplies its logits by a constant puts it on
    the final norm).  Input is the float32 residual stream, sums are float32, the output has the activation type."""

    def __init__(self, width: int, eps: float, scale: float = 1.0):
        self.width, self.eps, self.scale = int(width), float(eps), float(scale)
        self.weight = None

    def weight_specs(self):
        return [WeightSpec("weight", (self.width,), "vector", ("one_plus_normal", 0.05))]

    def kernel_needs(self, run_dtype):
        return [("rowwise.cu", ())]

    def bind(self, tensors, rt):
        w = tensors["weight"].float()
        self.weight = (w * self.scale if self.scale != 1.0 else w).contiguous()

    def forward(self, x, rt, rows=None):
        n = x.shape[0] if rows is None else rows.numel()
        out = rt.arena.alloc((n, self.width), rt.dtype)
        rt.launches += 1
        ops.layernorm(x, self.weight, out, self.eps, rows)
        return out
