"""Feed-forward parts."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import FeedForward, register_part


@register_part("feed_forward", "gated_silu")
class GatedSiLU(FeedForward):
    """down(silu(gate(h)) * up(h)), no biases, added to the residual stream
    (reference: src/model/qwen_block.cpp:165-182, src/kernels/elementwise.cpp:62-68).
    Gate and up are held as one matrix [gate ; up]; the gate product is formed in float32
    from the float32 accumulators and rounded once."""

    graph_safe = True        # launches kernels only; no host work that depends on the data


    def __init__(self, width: int, inner: int):
        self.width, self.inner = int(width), int(inner)
        self.wgu = self.wd = None

    def weight_specs(self):
        return [WeightSpec("gate_proj.weight", (self.inner, self.width)),
                WeightSpec("up_proj.weight", (self.inner, self.width)),
                WeightSpec("down_proj.weight", (self.width, self.inner))]

    def bind(self, tensors, rt):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            raise ValueError("gate and up projections must share one element type")
        self.wd = tensors["down_proj.weight"].contiguous()
        # On the tensor-core path blocks of 64 gate rows and 64 up rows alternate, so that one
        # 128-row tile of the product holds both halves of 64 features (see gemm_tcgen05.cu).
        self.interleaved = (rt.use_tensor_cores and g.dtype == torch.bfloat16 and self.inner % 64 == 0
                            and self.width % 8 == 0)
        if self.interleaved:
            n = self.inner // 64
            self.wgu = torch.stack([g.view(n, 64, self.width), u.view(n, 64, self.width)], dim=1) \
                .reshape(2 * self.inner, self.width).contiguous()
        else:
            self.wgu = torch.cat([g, u], dim=0).contiguous()

    def forward(self, h, residual, batch, rt):
        T = h.shape[0]
        a = rt.arena.alloc((T, self.inner), rt.dtype)
        if self.interleaved:
            rt.matmul(h, self.wgu, a, ops.EPI_SWIGLU_IL)
        else:
            rt.matmul(h, self.wgu[:self.inner], a, ops.EPI_SWIGLU, w2=self.wgu[self.inner:])
        rt.matmul(a, self.wd, residual, ops.EPI_ADD)


@register_part("feed_forward", "gated_clamped")
class GatedClamped(FeedForward):
    """down(g' * sigmoid(alpha g') * (u' + shift)) with g' = min(gate(h), limit) and
    u' = clamp(up(h), -limit, limit); no biases; added to the stream it is handed.  Gate and up are one
    matrix and one product; the gate product is formed in float32 from the float32 sums.  On the
    tensor-core path it is the product's epilogue (blocks of 64 gate rows and 64 up rows alternate, as in
    ``gated_silu``); elsewhere [gate ; up] goes out in float32 and a kernel of its own forms it."""

    graph_safe = True

    def __init__(self, width: int, inner: int, limit: float, alpha: float = 1.702, shift: float = 1.0):
        self.width, self.inner = int(width), int(inner)
        self.limit, self.alpha, self.shift = float(limit), float(alpha), float(shift)
        self.wgu = self.wd = None

    def weight_specs(self):
        return [WeightSpec("gate_proj.weight", (self.inner, self.width)),
                WeightSpec("up_proj.weight", (self.inner, self.width)),
                WeightSpec("down_proj.weight", (self.width, self.inner))]

    def bind(self, tensors, rt):
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        if g.dtype != u.dtype:
            raise ValueError("gate and up projections must share one element type")
        self.wd = tensors["down_proj.weight"].contiguous()
        self.interleaved = (rt.use_tensor_cores and g.dtype == torch.bfloat16 and self.inner % 64 == 0
                            and self.width % 8 == 0)
        if self.interleaved:
            n = self.inner // 64
            self.wgu = torch.stack([g.view(n, 64, self.width), u.view(n, 64, self.width)], dim=1) \
                .reshape(2 * self.inner, self.width).contiguous()
        else:
            self.wgu = torch.cat([g, u], dim=0).contiguous()

    def forward(self, h, residual, batch, rt):
        T = h.shape[0]
        if self.interleaved:
            a = rt.arena.alloc((T, self.inner), rt.dtype)
            rt.matmul(h, self.wgu, a, ops.EPI_SWIGLU_IL, gate=(self.limit, self.alpha, self.shift))
            rt.matmul(a, self.wd, residual, ops.EPI_ADD)
            return
        gu = rt.arena.alloc((T, 2 * self.inner), torch.float32)
        rt.matmul(h, self.wgu, gu)
        a = rt.arena.alloc((T, self.inner), rt.dtype)
        rt.launches += 1
        ops.glu_clamped(gu, a, self.limit, self.alpha, self.shift)
        rt.matmul(a, self.wd, residual, ops.EPI_ADD)


@register_part("feed_forward", "gated_relu")
class GatedReLU(GatedClamped):
    """down(max(gate(h), 0) * up(h)), no biases: the clamped gate product at its limits (no clamp, the
    sigmoid as steep as it gets, no shift), so it runs as the same two launches."""

    def __init__(self, width: int, inner: int):
        super().__init__(width, inner, limit=float("inf"), alpha=float("inf"), shift=0.0)


_ACTIVATIONS = {"gelu_erf": ops.UNARY_GELU_ERF, "relu_squared": ops.UNARY_RELU_SQUARED}


@register_part("feed_forward", "plain_mlp")
class PlainMLP(FeedForward):
    """down(act(up(h))), no gate and no biases, added to the stream it is handed; ``activation`` is "gelu_erf" (the exact
    GELU, 0.5 z (1 + erf(z / sqrt 2))) or "relu_squared" (max(z, 0)^2).  The activation is float32 arithmetic on the up
    product's float32 sums, rounded once to the activation type: on the tensor cores in the product's epilogue."""

    graph_safe = True

    def __init__(self, width: int, inner: int, activation: str):
        self.width, self.inner, self.activation = int(width), int(inner), str(activation)
        if self.activation not in _ACTIVATIONS:
            raise ValueError(f"plain_mlp: activation must be one of {', '.join(_ACTIVATIONS)}, got {activation!r}")

    def weight_specs(self):
        return [WeightSpec("up_proj.weight", (self.inner, self.width)),
                WeightSpec("down_proj.weight", (self.width, self.inner))]

    def kernel_needs(self, run_dtype):
        return [("rowwise.cu", ())]

    def bind(self, tensors, rt):
        self.wu = tensors["up_proj.weight"].contiguous()
        self.wd = tensors["down_proj.weight"].contiguous()

    def forward(self, h, residual, batch, rt):
        T = h.shape[0]
        a = rt.arena.alloc((T, self.inner), rt.dtype)
        rt.matmul(h, self.wu, a, unary=_ACTIVATIONS[self.activation])       # the activation in the product's epilogue
        rt.matmul(a, self.wd, residual, ops.EPI_ADD)
