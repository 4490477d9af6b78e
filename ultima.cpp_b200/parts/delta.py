"""The delta-rule mixers: recurrent layers with a matrix of state a head."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import Mixer, StateNeed, register_part


@register_part("mixer", "gated_delta")
class GatedDelta(Mixer):
    """For each head a matrix S [key size D, value size E] in float32, zero at a sequence's start.
    A token brings q, k (``n_kv_heads`` heads of size D; head h uses q/k head h // (heads / kv heads))
    and v (``n_heads`` heads of size E), each from its projection through a causal convolution of
    ``conv`` taps over time (one filter a channel, the last tap on the current token, zeros before the
    sequence) and SiLU; q and k are made unit vectors (x / sqrt(sum x^2 + unit_eps)), q also times
    D^-1/2.  With the write strength b = sigmoid(b_proj h) (one a head) and the decay
    a = exp(-exp(a_log[h]) * softplus(decay_up(decay_down h) + dt_bias)) (one a head and key channel):

        S[d, :] *= a[d];   u = b (v - S^T k);   S += k u^T;   o = S^T q

    o is divided by its root mean square over E (``eps``), multiplied by a weight of size E shared by
    the heads and by sigmoid(gate_up(gate_down h)), and goes through the output projection into the
    stream the mixer is handed.  The convolution's last ``conv - 1`` inputs are state too.

    Everything between the projections and the output projection is float32.  The projections that
    read the mixer's input run as two products, [q | k | v | b] with float32 results (for few tokens in
    K slices that the next kernel adds up) and [decay_down | gate_down] in the activation type, which
    the two up-projections then take as their input (each padded to a multiple of 8 columns with zero
    weights, so that both are aligned operands of the tensor-core product).

    Two further forms, each a parameter:
      decay="head"   one decay a head instead of one a head and key channel:
                     a = exp(-exp(a_log[h]) * softplus(a_proj h + dt_bias[h])), ``a_proj`` a matrix of ``heads`` rows
      gate="silu"    the output gate is silu(gate_proj h) with a full matrix of heads * value size rows instead of
                     the sigmoid of a low-rank product
    Their rows join the one input product [q | k | v | b | a | gate], whose float32 sums the kernels read.
    """

    graph_safe = True

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int, conv: int,
                 decay_rank: int | None = None, gate_rank: int | None = None, eps: float = 1e-6, unit_eps: float = 1e-6,
                 decay: str = "channel", gate: str = "sigmoid_lowrank"):
        if n_heads % n_kv_heads:
            raise ValueError("heads must be a multiple of kv heads")
        self.width, self.nh, self.nkv = int(width), int(n_heads), int(n_kv_heads)
        self.hd, self.hdv, self.conv = int(head_dim), int(v_head_dim), int(conv)
        if decay not in ("channel", "head") or gate not in ("sigmoid_lowrank", "silu"):
            raise ValueError("gated_delta: decay is 'channel' or 'head', gate is 'sigmoid_lowrank' or 'silu'")
        self.decay_per_head, self.gate_full = decay == "head", gate == "silu"
        self.decay_rank = None if self.decay_per_head else int(decay_rank or 0)
        self.gate_rank = None if self.gate_full else int(gate_rank or 0)
        self.eps, self.unit_eps = float(eps), float(unit_eps)
        self.qk_width, self.v_width = self.nkv * self.hd, self.nh * self.hdv
        self.channels = 2 * self.qk_width + self.v_width
        if not (1 <= self.conv <= 16):
            raise ValueError(f"gated_delta: a convolution of {self.conv} taps is not one the kernels take (1 to 16)")
        if self.hd > 256:
            raise ValueError(f"gated_delta: key size {self.hd} is more than the scan kernel holds (256)")
        if (self.decay_rank is not None and self.decay_rank < 1) or (self.gate_rank is not None and self.gate_rank < 1):
            raise ValueError("gated_delta: the low-rank products need inner sizes of at least 1")

    def weight_specs(self):
        W, V = WeightSpec, "vector"
        s = [W("q_proj.weight", (self.qk_width, self.width)), W("q_conv.weight", (self.qk_width, self.conv), V, ("normal", 0.3)),
             W("k_proj.weight", (self.qk_width, self.width)), W("k_conv.weight", (self.qk_width, self.conv), V, ("normal", 0.3)),
             W("v_proj.weight", (self.v_width, self.width)), W("v_conv.weight", (self.v_width, self.conv), V, ("normal", 0.3)),
             W("b_proj.weight", (self.nh, self.width)),
             W("a_log", (self.nh,), V, ("normal", 0.5)),
             W("o_norm.weight", (self.hdv,), V, ("one_plus_normal", 0.05))]
        if self.decay_per_head:
            s += [W("a_proj.weight", (self.nh, self.width)), W("dt_bias", (self.nh,), V, ("normal", 0.5))]
        else:
            s += [W("decay_down.weight", (self.decay_rank, self.width)),
                  W("decay_up.weight", (self.nh * self.hd, self.decay_rank), "matrix", ("normal", 0.1)),
                  W("dt_bias", (self.nh * self.hd,), V, ("normal", 0.5))]
        if self.gate_full:
            s.append(W("gate_proj.weight", (self.v_width, self.width)))
        else:
            s += [W("gate_down.weight", (self.gate_rank, self.width)),
                  W("gate_up.weight", (self.v_width, self.gate_rank), "matrix", ("normal", 0.1))]
        return s + [W("o_proj.weight", (self.width, self.v_width))]

    def cache_need(self):
        taps = max(self.conv - 1, 1)
        return (StateNeed((self.nh, self.hd, self.hdv), "float32"), StateNeed((taps, self.channels), "float32"))

    def kernel_needs(self, run_dtype):
        return [("delta.cu", ())]

    def bind(self, tensors, rt):
        names = ["q_proj", "k_proj", "v_proj", "b_proj"] + (["a_proj"] if self.decay_per_head else []) \
            + (["gate_proj"] if self.gate_full else [])
        low = ([] if self.decay_per_head else ["decay_down"]) + ([] if self.gate_full else ["gate_down"])
        ups = ([] if self.decay_per_head else ["decay_up"]) + ([] if self.gate_full else ["gate_up"])
        ws = {n: tensors[n + ".weight"] for n in names + low + ups}
        if len({w.dtype for w in ws.values()}) != 1:
            raise ValueError("gated_delta: the projections must share one element type")
        self.w_in = torch.cat([ws[n] for n in names], dim=0).contiguous()
        self.b_off = self.channels
        self.a_off = self.b_off + self.nh if self.decay_per_head else -1
        self.g_off = self.b_off + self.nh * (2 if self.decay_per_head else 1) if self.gate_full else -1

        def padded(w, rows, cols):
            out = torch.zeros((rows, cols), dtype=w.dtype, device=w.device)
            out[:w.shape[0], :w.shape[1]] = w
            return out
        ra = 0 if self.decay_per_head else -(-self.decay_rank // 8) * 8
        rg = 0 if self.gate_full else -(-self.gate_rank // 8) * 8
        self.low_split = ra
        self.w_low = self.decay_up = self.gate_up = None
        if low:
            self.w_low = torch.cat([padded(ws[n], r, self.width) for n, r in (("decay_down", ra), ("gate_down", rg)) if n in ws],
                                   dim=0).contiguous()
        if not self.decay_per_head:
            self.decay_up = padded(ws["decay_up"], ws["decay_up"].shape[0], ra).contiguous()
        if not self.gate_full:
            self.gate_up = padded(ws["gate_up"], ws["gate_up"].shape[0], rg).contiguous()
        self.conv_w = torch.cat([tensors[n].float() for n in ("q_conv.weight", "k_conv.weight", "v_conv.weight")],
                                dim=0).contiguous()
        self.dt_bias = tensors["dt_bias"].float().contiguous()
        self.a_log = tensors["a_log"].float().contiguous()
        self.o_norm = tensors["o_norm.weight"].float().contiguous()
        self.wo = tensors["o_proj.weight"].contiguous()
        self.shape = ops.delta_shape(self.nh, self.nkv, self.hd, self.hdv, self.conv,
                                     (0, self.qk_width, 2 * self.qk_width, self.b_off), a_off=self.a_off)

    def forward(self, h, residual, batch, cache, rt):
        T = h.shape[0]
        S, conv_state = cache.states
        f32 = torch.float32
        p = rt.matmul_parts(h, self.w_in)             # few tokens: K in slices, summed by the kernels that read them
        if p is None:
            p = rt.arena.alloc((T, self.w_in.shape[0]), f32)
            rt.matmul(h, self.w_in, p)
        decay_pre = None
        if self.w_low is not None:
            low = rt.arena.alloc((T, self.w_low.shape[0]), rt.dtype)
            rt.matmul(h, self.w_low, low)
        if not self.decay_per_head:
            decay_pre = rt.arena.alloc((T, self.nh * self.hd), f32)
            rt.matmul(low[:, :self.low_split], self.decay_up, decay_pre)
        if self.gate_full:
            gate_pre = p[..., self.g_off:self.g_off + self.v_width]       # columns of the input product, summed by the kernel
        else:
            gate_pre = rt.arena.alloc((T, self.v_width), f32)
            rt.matmul(low[:, self.low_split:], self.gate_up, gate_pre)
        qn = rt.arena.alloc((T, self.qk_width), f32)
        kn = rt.arena.alloc((T, self.qk_width), f32)
        vc = rt.arena.alloc((T, self.v_width), f32)
        beta = rt.arena.alloc((T, self.nh), f32)
        dec = rt.arena.alloc((T, self.nh * self.hd), f32)
        o = rt.arena.alloc((T, self.v_width), f32)
        oa = rt.arena.alloc((T, self.v_width), rt.dtype)
        # one token a sequence: a channel's state has one reader, which then also moves it on
        one_each = batch.max_new == 1 and batch.n_seqs == T
        rt.launches += 3 if one_each else 4
        ops.delta_prepare(p, self.shape, self.conv_w, conv_state, decay_pre, self.dt_bias, self.a_log, batch,
                          qn, kn, vc, beta, dec, self.unit_eps, self.hd ** -0.5, update_state=one_each)
        if not one_each:
            ops.conv_state_update(p, conv_state, batch, self.channels, self.conv)
        ops.delta_scan(qn, kn, vc, beta, dec, o, S, batch, self.nh, self.nkv, self.hd, self.hdv)
        ops.delta_finish(o, gate_pre, self.o_norm, oa, self.nh, self.hdv, self.eps, silu_gate=self.gate_full)
        rt.matmul(oa, self.wo, residual, ops.EPI_ADD)


@register_part("mixer", "general_delta")
class GeneralDelta(Mixer):
    """The generalised delta rule: for each head a matrix S [D, D] in float32, zero at a sequence's start.  A token brings
    r, k, v (``n_heads`` heads of size D each, plain projections), a decay for every head and key channel
    w = exp(-exp(-1/2) * sigmoid(w_up(tanh(w_down h)) + w_bias)) and a removal rate for every head and key channel
    a = sigmoid(a_proj h + a_bias).  With the unit key u = k / sqrt(sum k^2 + unit_eps) of each head:

        S <- diag(w) S - (a * u) (u^T S) + k v^T        (both terms read the old S);      o = S^T r

    Each head's o is divided by its root mean square (``eps``); the heads side by side are multiplied by a weight of all
    heads' size and by sigmoid(gate_proj h), and go through the output projection into the stream the mixer is handed.

    The projections that read the mixer's input are ONE product [r | k | v | gate | a | w_down] with float32 results (for
    few tokens in K slices that the kernels add up); tanh(w_down h) in the activation type is the operand of the small
    product w_up (padded to a multiple of 8 columns with zero weights).  Everything behind the products is float32."""

    graph_safe = True
    DECAY_SCALE = math.exp(-0.5)

    def __init__(self, width: int, n_heads: int, head_dim: int, decay_rank: int, eps: float, unit_eps: float = 1e-6):
        self.width, self.nh, self.hd, self.rank = int(width), int(n_heads), int(head_dim), int(decay_rank)
        self.eps, self.unit_eps = float(eps), float(unit_eps)
        self.inner = self.nh * self.hd
        if self.hd > 256:
            raise ValueError(f"general_delta: head size {self.hd} is more than the scan kernel holds (256)")
        if self.rank < 1:
            raise ValueError("general_delta: the decay's low-rank product needs an inner size of at least 1")
        self.rank_pad = -(-self.rank // 8) * 8

    def weight_specs(self):
        W, V, n = WeightSpec, "vector", self.inner
        return [W("r_proj.weight", (n, self.width)), W("k_proj.weight", (n, self.width)), W("v_proj.weight", (n, self.width)),
                W("gate_proj.weight", (n, self.width)), W("a_proj.weight", (n, self.width)),
                W("a_bias", (n,), V, ("normal", 0.5)),
                W("w_down.weight", (self.rank, self.width)),
                W("w_up.weight", (n, self.rank), "matrix", ("normal", 0.3)),
                W("w_bias", (n,), V, ("normal", 0.5)),
                W("o_norm.weight", (n,), V, ("one_plus_normal", 0.05)),
                W("o_proj.weight", (self.width, n))]

    def cache_need(self):
        return StateNeed((self.nh, self.hd, self.hd), "float32")

    def kernel_needs(self, run_dtype):
        return [("delta.cu", ()), ("rowwise.cu", ())]

    def bind(self, tensors, rt):
        names = ["r_proj", "k_proj", "v_proj", "gate_proj", "a_proj", "w_down"]
        ws = [tensors[n + ".weight"] for n in names]
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("general_delta: the projections must share one element type")
        self.w_in = torch.cat(ws, dim=0).contiguous()
        n = self.inner
        self.offs = (0, n, 2 * n, 4 * n)                 # r, k, v, removal rate
        self.g_off, self.low_off = 3 * n, 5 * n
        up = tensors["w_up.weight"]
        if self.rank_pad != self.rank:
            p = torch.zeros((n, self.rank_pad), dtype=up.dtype, device=up.device)
            p[:, :self.rank] = up
            up = p
        self.w_up = up.contiguous()
        self.a_bias = tensors["a_bias"].float().contiguous()
        self.w_bias = tensors["w_bias"].float().contiguous()
        self.o_norm = tensors["o_norm.weight"].float().contiguous()
        self.wo = tensors["o_proj.weight"].contiguous()

    def forward(self, h, residual, batch, cache, rt):
        T, n = h.shape[0], self.inner
        S = cache.states[0]
        f32 = torch.float32
        p = rt.matmul_parts(h, self.w_in)
        if p is None:
            p = rt.arena.alloc((T, self.w_in.shape[0]), f32)
            rt.matmul(h, self.w_in, p)
        low = rt.arena.alloc((T, self.rank_pad), rt.dtype)
        rt.launches += 1
        ops.take_cols(p, self.low_off, self.rank, low, tanh=True)
        wpre = rt.arena.alloc((T, n), f32)
        rt.matmul(low, self.w_up, wpre)
        rn, un, kraw, rem, dec, vc, o = (rt.arena.alloc((T, n), f32) for _ in range(7))
        oa = rt.arena.alloc((T, n), rt.dtype)
        rt.launches += 3
        ops.gdelta_prepare(p, self.offs, self.a_bias, wpre, self.w_bias, rn, un, kraw, rem, dec, vc, self.nh, self.hd,
                           self.unit_eps, self.DECAY_SCALE)
        ops.delta_scan(rn, un, vc, None, dec, o, S, batch, self.nh, self.nh, self.hd, self.hd, rem=rem, kraw=kraw)
        ops.delta_finish(o, p[..., self.g_off:self.g_off + n], self.o_norm, oa, self.nh, self.hd, self.eps)
        rt.matmul(oa, self.wo, residual, ops.EPI_ADD)
