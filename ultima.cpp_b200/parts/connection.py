"""Connections: how a sublayer meets a residual stream that is kept in several copies."""
from __future__ import annotations

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import Connection, register_part


@register_part("connection", "hyper")
class HyperConnection(Connection):
    """With copies x_1 .. x_S of the stream and the tables ``in`` [S], ``out`` [S] and ``mix`` [S, S] (indexed
    [from, to]): the sublayer reads norm(sum_s in[s] x_s), and its result y goes back as
    x_t <- sum_s mix[s, t] x_s + out[t] y, all copies at once from the old ones.  One kernel a pass over the
    copies, float32 throughout; a write and the next sublayer's read can share a pass."""

    def __init__(self, streams: int):
        self.streams = int(streams)
        if not (1 <= self.streams <= 8):
            raise ValueError(f"hyper connection: {self.streams} copies of the stream are not what the kernel takes (1 to 8)")
        self.w_in = self.w_out = self.w_mix = None

    def weight_specs(self):
        S = self.streams
        return [WeightSpec("in", (S,), "vector", ("one_plus_normal", 0.1)), WeightSpec("out", (S,), "vector", ("one_plus_normal", 0.1)),
                WeightSpec("mix", (S, S), "vector", ("normal", 0.4))]

    def bind(self, tensors, rt):
        self.w_in = tensors["in"].float().contiguous()
        self.w_out = tensors["out"].float().contiguous()
        self.w_mix = tensors["mix"].float().contiguous()

    def kernel_needs(self, run_dtype):
        return [("streams.cu", ())]

    def read(self, xs, norm, rt):
        h = rt.arena.alloc(tuple(xs.shape[1:]), rt.dtype)
        rt.launches += 1
        ops.streams_pass(xs, read=(self.w_in, norm.weight, norm.eps), out=h)
        return h

    def write(self, xs, y, rt, then=None):
        rt.launches += 1
        if then is None:
            ops.streams_pass(xs, write=(self.w_mix, self.w_out, y))
            return None
        nxt, norm = then
        h = rt.arena.alloc(tuple(xs.shape[1:]), rt.dtype)
        ops.streams_pass(xs, write=(self.w_mix, self.w_out, y), read=(nxt.w_in, norm.weight, norm.eps), out=h)
        return h
