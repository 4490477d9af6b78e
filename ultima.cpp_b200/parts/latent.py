"""The latent-attention mixer: keys and values kept as one small vector a position."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import Mixer, KVNeed, register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """Every position keeps c = rms_norm(W_dkv h [:rank]) (weight ``kv_norm``, the layer's eps) and one rotated key
    part k_r = rotate(W_dkv h [rank:]) of ``rot_dim`` numbers that all heads share; nothing else is cached.  Head h of
    ``n_heads`` has a query [q_u (``head_dim`` numbers) | q_r (``rot_dim``, rotated)], the unrotated key W_uk[h] c and
    the value W_uv[h] c (``v_head_dim`` numbers); the score is (q_u . W_uk[h] c + q_r . k_r) * scale, the softmax
    ordinary, the window optional.  The rotation turns the pairs (2i, 2i + 1) of the first ``rotary_dim`` columns of a
    rotated part; its frequencies theta^(-2i/rotary_dim) may be rescaled (``yarn`` = (factor, original, fast, slow):
    with p(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(p(fast)), 0), hi = min(ceil(p(slow)),
    rotary_dim - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), frequency i becomes
    f_i / factor * ramp_i + f_i (1 - ramp_i), and cos and sin are multiplied by 0.1 ln(factor) + 1).

    The attention runs in the latent space: q' = W_uk[h]^T q_u (``rank`` numbers) meets c directly, so all heads read
    ONE key row [c | k_r] a position and the weighted sum of the c goes through W_uv[h] afterwards.  Launches: one
    product [q | dkv] with float32 sums, the placement kernel (norm, rotation, cache row, query parts), the heads'
    W_uk^T products as one batched product, attention over one key head whose values are the leading columns of the
    key rows, the heads' W_uv products as one batched product, the output product into the stream."""

    graph_safe = True

    def __init__(self, width: int, n_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, rank: int, scale: float,
                 eps: float, theta: float, rotary_dim: int, max_positions: int, window: int | None = None,
                 yarn: tuple | None = None):
        self.width, self.nh, self.hd, self.rot = int(width), int(n_heads), int(head_dim), int(rot_dim)
        self.hdv, self.rank, self.scale, self.eps = int(v_head_dim), int(rank), float(scale), float(eps)
        self.theta, self.rd, self.max_positions = float(theta), int(rotary_dim), int(max_positions)
        self.window = int(window) if window else None
        self.yarn = tuple(float(v) for v in yarn) if yarn else None
        self.row = self.rank + self.rot                    # a position's key row
        if self.rd % 2 or not (2 <= self.rd <= self.rot):
            raise ValueError(f"latent_attention: rotary size {self.rd} must be even and at most the rotated part {self.rot}")
        if self.row > 1024 or self.rank > 512:
            raise ValueError(f"latent_attention: a key row of {self.row} numbers (latent {self.rank}) is more than the "
                             f"attention kernels take (1,024 and 512)")

    def weight_specs(self):
        W = WeightSpec
        return [W("q_proj.weight", (self.nh * (self.hd + self.rot), self.width)),
                W("kv_down.weight", (self.row, self.width)),
                W("kv_norm.weight", (self.rank,), "vector", ("one_plus_normal", 0.05)),
                W("k_up.weight", (self.nh * self.hd, self.rank), "matrix", ("normal", 0.08)),
                W("v_up.weight", (self.nh * self.hdv, self.rank), "matrix", ("normal", 0.08)),
                W("o_proj.weight", (self.width, self.nh * self.hdv))]

    def cache_need(self):
        return KVNeed(1, self.row, self.window, values_in_keys=True)

    def kernel_needs(self, run_dtype):
        from ..kernels import attn_tc
        out = [("latent.cu", ()), ("attn_simple.cu", ())]
        if run_dtype == torch.bfloat16:
            out += attn_tc.latent_needs(self.row, self.nh)
        return out

    def frequencies(self):
        """(frequency of every pair, amplitude of cos and sin), float64."""
        half = self.rd // 2
        i = torch.arange(half, dtype=torch.float64)
        f = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / self.rd)
        amp = 1.0
        if self.yarn is not None:
            factor, original, fast, slow = self.yarn

            def where(t):
                return self.rd * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(self.theta))
            lo = max(math.floor(where(fast)), 0)
            hi = min(math.ceil(where(slow)), self.rd - 1)
            ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            f = f / factor * ramp + f * (1.0 - ramp)
            amp = 0.1 * math.log(factor) + 1.0
        return f, amp

    def bind(self, tensors, rt):
        wq, wd = tensors["q_proj.weight"], tensors["kv_down.weight"]
        if wq.dtype != wd.dtype:
            raise ValueError("latent_attention: the projections must share one element type")
        self.w_in = torch.cat([wq, wd], dim=0).contiguous()
        self.c_off = wq.shape[0]
        self.kv_norm = tensors["kv_norm.weight"].float().contiguous()
        # a head's W_uk as the matrix its query part meets: [rank, head size]; W_uv as stored: [value size, rank]
        self.k_up_t = tensors["k_up.weight"].view(self.nh, self.hd, self.rank).transpose(1, 2).contiguous()
        self.v_up = tensors["v_up.weight"].view(self.nh, self.hdv, self.rank).contiguous()
        self.wo = tensors["o_proj.weight"].contiguous()
        key = ("latent_rotary", self.rd, self.theta, self.max_positions, self.yarn)

        def make():
            f, amp = self.frequencies()
            ang = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * f[None, :]
            return ((torch.cos(ang) * amp).float().contiguous().to(rt.device),
                    (torch.sin(ang) * amp).float().contiguous().to(rt.device))
        self.cos, self.sin = rt.shared(key, make)

    def forward(self, h, residual, batch, cache, rt):
        T = h.shape[0]
        kv = cache.kv
        x = rt.matmul_parts(h, self.w_in)              # few tokens: K in slices, summed by the placement kernel
        if x is None:
            x = rt.arena.alloc((T, self.w_in.shape[0]), torch.float32)
            rt.matmul(h, self.w_in, x)
        q_plain = rt.arena.alloc((T, self.nh, self.hd), rt.dtype)
        q_lat = rt.arena.alloc((T, self.nh, self.row), rt.dtype)
        rt.launches += 2
        ops.latent_place(x, 0, self.c_off, q_plain, q_lat, self.kv_norm, self.cos, self.sin, self.rd, batch.tok_pos,
                         batch.tok_seq, kv.k, kv.table, kv.ring, kv.page, self.nh, self.hd, self.rot, self.rank, self.eps)
        rt.matmul_heads(q_plain, self.k_up_t, q_lat[:, :, :self.rank])
        o_lat = rt.attention_latent(q_lat, kv, batch, self.nh, self.row, self.rank, self.scale, self.window)
        o = rt.arena.alloc((T, self.nh, self.hdv), rt.dtype)
        rt.launches += 1
        rt.matmul_heads(o_lat, self.v_up, o)
        rt.matmul(o.view(T, self.nh * self.hdv), self.wo, residual, ops.EPI_ADD)
