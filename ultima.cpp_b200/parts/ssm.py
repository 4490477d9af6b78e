"""A selective state-space mixer with one decay a head (the state-space duality form of Mamba-2)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import Mixer, StateNeed, register_part


@register_part("mixer", "state_space_dual")
class StateSpaceDual(Mixer):
    """For each head a matrix S [state size N, value size P] in float32, zero at a sequence's start.  One
    projection of the mixer's input gives a row [z | x | B | C | dt]: an output gate z and values x of
    ``n_heads`` * P columns each, input and output rows B and C of ``n_groups`` * N columns each (head h uses
    group h // (heads / groups)), and one step size a head.  x, B and C pass a causal convolution of ``conv``
    taps over time (one filter a channel with a bias, the last tap on the current token, zeros before the
    sequence) and SiLU.  With dt = softplus(dt + dt_bias) (no clamp):

        S <- exp(-exp(a_log[h]) dt) S + dt B x^T;      y = S^T C + d_skip[h] x

    y silu(z) is divided by its root mean square in ``norm_groups`` equal parts of the row (``eps``),
    multiplied by a weight of the row's size and by ``out_scale``, and goes through the output projection
    into the stream the mixer is handed.  The convolution's last ``conv - 1`` inputs are state too.

    Everything between the two projections is float32; for few tokens the input projection runs in K
    slices that the kernels add up as they read."""

    graph_safe = True

    def __init__(self, width: int, n_heads: int, head_dim: int, state: int, n_groups: int, conv: int, norm_groups: int,
                 eps: float, out_scale: float = 1.0):
        self.width, self.nh, self.hd, self.n_state = int(width), int(n_heads), int(head_dim), int(state)
        self.ng, self.conv, self.norm_groups = int(n_groups), int(conv), int(norm_groups)
        self.eps, self.out_scale = float(eps), float(out_scale)
        if self.nh % self.ng:
            raise ValueError("state_space_dual: heads must be a multiple of groups")
        self.inner = self.nh * self.hd
        if self.norm_groups < 1 or self.inner % self.norm_groups:
            raise ValueError("state_space_dual: the row must divide into norm_groups equal parts")
        if not (1 <= self.conv <= 16):
            raise ValueError(f"state_space_dual: a convolution of {self.conv} taps is not one the kernels take (1 to 16)")
        if not (1 <= self.n_state <= 256):
            raise ValueError(f"state_space_dual: a state of {self.n_state} channels is more than the scan kernel holds (256)")
        self.channels = self.inner + 2 * self.ng * self.n_state
        self.rows = 2 * self.inner + 2 * self.ng * self.n_state + self.nh

    def weight_specs(self):
        W, V = WeightSpec, "vector"
        return [W("in_proj.weight", (self.rows, self.width)),
                W("conv.weight", (self.channels, self.conv), V, ("normal", 0.3)),
                W("conv.bias", (self.channels,), V, ("normal", 0.1)),
                W("dt_bias", (self.nh,), V, ("normal", 0.5)),
                W("a_log", (self.nh,), V, ("normal", 0.5)),
                W("d_skip", (self.nh,), V, ("one_plus_normal", 0.2)),
                W("o_norm.weight", (self.inner,), V, ("one_plus_normal", 0.05)),
                W("o_proj.weight", (self.width, self.inner))]

    def cache_need(self):
        taps = max(self.conv - 1, 1)
        return (StateNeed((self.nh, self.n_state, self.hd), "float32"), StateNeed((taps, self.channels), "float32"))

    def kernel_needs(self, run_dtype):
        return [("ssm.cu", ())]

    def bind(self, tensors, rt):
        self.w_in = tensors["in_proj.weight"].contiguous()
        self.wo = tensors["o_proj.weight"].contiguous()
        self.conv_w = tensors["conv.weight"].float().contiguous()
        self.conv_b = tensors["conv.bias"].float().contiguous()
        self.dt_bias = tensors["dt_bias"].float().contiguous()
        self.a_log = tensors["a_log"].float().contiguous()
        self.d_skip = tensors["d_skip"].float().contiguous()
        self.o_norm = tensors["o_norm.weight"].float().contiguous()
        x_off = self.inner
        b_off = x_off + self.inner
        c_off = b_off + self.ng * self.n_state
        self.shape = ops.ssm_shape(self.nh, self.hd, self.n_state, self.ng, self.conv,
                                   (0, x_off, b_off, c_off, c_off + self.ng * self.n_state))

    def input_weight(self):
        return self.w_in

    def adopt_input_weight(self, w):
        self.w_in = w

    def forward(self, h, residual, batch, cache, rt, projected=None):
        T = h.shape[0]
        S, conv_state = cache.states
        f32 = torch.float32
        p = projected if projected is not None else rt.matmul_parts(h, self.w_in)
        if p is None:
            p = rt.arena.alloc((T, self.rows), f32)
            rt.matmul(h, self.w_in, p)
        xbc = rt.arena.alloc((T, self.channels), f32)
        dtv = rt.arena.alloc((T, self.nh), f32)
        dec = rt.arena.alloc((T, self.nh), f32)
        y = rt.arena.alloc((T, self.inner), f32)
        ya = rt.arena.alloc((T, self.inner), rt.dtype)
        one_each = batch.max_new == 1 and batch.n_seqs == T
        rt.launches += 3 if one_each or self.conv == 1 else 4
        ops.ssm_prepare(p, self.shape, self.conv_w, self.conv_b, conv_state, self.dt_bias, self.a_log, batch, xbc, dtv, dec,
                        update_state=one_each)
        if not one_each and self.conv > 1:
            ops.ssm_conv_state_update(p, self.shape, conv_state, batch)
        ops.ssm_scan(xbc, dtv, dec, self.d_skip, y, S, batch, self.nh, self.hd, self.n_state, self.ng)
        ops.ssm_finish(y, p, self.shape, self.o_norm, ya, self.norm_groups, self.eps, self.out_scale)
        rt.matmul(ya, self.wo, residual, ops.EPI_ADD)


@register_part("mixer", "selective_scan")
class SelectiveScan(Mixer):
    """The selective scan with a decay for every (channel, state element) (the first Mamba form).  ``in_proj`` gives a row
    [x | z] of ``inner`` columns each; x passes a causal convolution of ``conv`` taps over time (one filter a channel with a
    bias, the last tap on the current token, zeros before the sequence) and SiLU; ``x_proj`` of that gives
    [dt | B | C] (``dt_rank``, ``state``, ``state`` columns); dt = softplus(dt_proj(dt) + dt_bias), one a channel;
    A = -exp(a_log) [inner, state].  For channel c and state element n, in float32, zero at a sequence's start:

        S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;     y_c = sum_n S[c, n] C_n + d_skip[c] x_c

    y silu(z) goes through the output projection into the stream the mixer is handed.  The convolution's last
    ``conv - 1`` inputs are state too.  Step sizes, softplus, exponentials and S are float32; the products' operands
    have the activation type (for few tokens the input product runs in K slices that the kernels add up)."""

    graph_safe = True

    def __init__(self, width: int, inner: int, state: int, dt_rank: int, conv: int):
        self.width, self.inner, self.n_state = int(width), int(inner), int(state)
        self.dt_rank, self.conv = int(dt_rank), int(conv)
        if not (1 <= self.conv <= 16):
            raise ValueError(f"selective_scan: a convolution of {self.conv} taps is not one the kernels take (1 to 16)")
        if not (1 <= self.n_state <= 256):
            raise ValueError(f"selective_scan: a state of {self.n_state} elements is more than the scan kernel holds (256)")
        if self.dt_rank < 1:
            raise ValueError("selective_scan: dt_rank must be at least 1")
        self.rank_pad = -(-self.dt_rank // 8) * 8

    def weight_specs(self):
        W, V = WeightSpec, "vector"
        return [W("in_proj.weight", (2 * self.inner, self.width)),
                W("conv.weight", (self.inner, self.conv), V, ("normal", 0.3)),
                W("conv.bias", (self.inner,), V, ("normal", 0.1)),
                W("x_proj.weight", (self.dt_rank + 2 * self.n_state, self.inner)),
                W("dt_proj.weight", (self.inner, self.dt_rank), "matrix", ("normal", 0.1)),
                W("dt_bias", (self.inner,), V, ("normal", 0.5)),
                W("a_log", (self.inner, self.n_state), V, ("normal", 0.5)),
                W("d_skip", (self.inner,), V, ("one_plus_normal", 0.2)),
                W("o_proj.weight", (self.width, self.inner))]

    def cache_need(self):
        S = StateNeed((self.inner, self.n_state), "float32")
        return (S, StateNeed((self.conv - 1, self.inner), "float32")) if self.conv > 1 else S

    def kernel_needs(self, run_dtype):
        return [("ssm.cu", ()), ("rowwise.cu", ())]

    def bind(self, tensors, rt):
        self.w_in = tensors["in_proj.weight"].contiguous()
        self.w_x = tensors["x_proj.weight"].contiguous()
        wd = tensors["dt_proj.weight"]
        if self.rank_pad != self.dt_rank:                 # an aligned operand: columns of zeros
            p = torch.zeros((self.inner, self.rank_pad), dtype=wd.dtype, device=wd.device)
            p[:, :self.dt_rank] = wd
            wd = p
        self.w_dt = wd.contiguous()
        self.wo = tensors["o_proj.weight"].contiguous()
        self.conv_w = tensors["conv.weight"].float().contiguous()
        self.conv_b = tensors["conv.bias"].float().contiguous()
        self.dt_bias = tensors["dt_bias"].float().contiguous()
        self.A = (-torch.exp(tensors["a_log"].float())).contiguous()
        self.d_skip = tensors["d_skip"].float().contiguous()

    def forward(self, h, residual, batch, cache, rt):
        T = h.shape[0]
        f32 = torch.float32
        S = cache.states[0]
        conv_state = cache.states[1] if self.conv > 1 else None
        p = rt.matmul_parts(h, self.w_in)               # few tokens: K in slices, summed by the kernels that read them
        if p is None:
            p = rt.arena.alloc((T, 2 * self.inner), f32)
            rt.matmul(h, self.w_in, p)
        xc = rt.arena.alloc((T, self.inner), rt.dtype)
        one_each = batch.max_new == 1 and batch.n_seqs == T           # one token a sequence: the kernel moves the state on itself
        rt.launches += 1
        ops.causal_conv(p, self.conv_w, conv_state, batch, xc, silu=True, out_bias=self.conv_b, update_state=one_each)
        if self.conv > 1 and not one_each:
            rt.launches += 1
            ops.causal_conv_state(p, conv_state, batch)
        bc = rt.arena.alloc((T, self.dt_rank + 2 * self.n_state), f32)
        rt.matmul(xc, self.w_x, bc)
        low = rt.arena.alloc((T, self.rank_pad), rt.dtype)
        rt.launches += 1
        ops.take_cols(bc, 0, self.dt_rank, low)
        dtp = rt.arena.alloc((T, self.inner), f32)
        rt.matmul(low, self.w_dt, dtp)
        y = rt.arena.alloc((T, self.inner), rt.dtype)
        z = p[..., self.inner:]
        # many tokens a sequence: softplus, dt * x and the gate leave the chain from token to token (three kernels)
        work = None if one_each or T < 4 * batch.n_seqs else rt.arena.alloc((2, T, self.inner), f32)
        rt.launches += 1 if work is None else 3
        ops.mamba1_scan(xc, dtp, self.dt_bias, bc, self.dt_rank, self.dt_rank + self.n_state, self.A, self.d_skip, z, y, S,
                        batch, self.n_state, work=work)
        rt.matmul(y, self.wo, residual, ops.EPI_ADD)
