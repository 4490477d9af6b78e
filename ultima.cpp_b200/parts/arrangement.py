"""How a layer's parts are arranged around the residual stream."""
from __future__ import annotations

import os

from ..kernels import ops
import torch

from ..weights.spec import WeightSpec
from .base import Arrangement, Entry, ResidualGate, register_part


# ULTIMA_FUSE_INPUTS=0: every part of a parallel layer runs its own input product (for measurements)
FUSE_INPUTS = os.environ.get("ULTIMA_FUSE_INPUTS", "1") != "0"


@register_part("arrangement", "pre_norm")
class PreNorm(Arrangement):
    """x += mixer(norm(x)); x += feed_forward(norm(x)), the residual stream x in float32
    (reference: src/model/qwen_block.cpp:621-628, :782-792, :811-812)."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm",
             "feed_forward": "feed_forward"}

    def __init__(self):
        pass

    def run(self, layer, x, batch, cache, rt):
        mark = rt.arena.mark()
        h = layer.mixer_norm.forward(x, rt)
        layer.mixer.forward(h, x, batch, cache, rt)
        rt.arena.reset(mark)
        h = layer.feed_forward_norm.forward(x, rt)
        layer.feed_forward.forward(h, x, batch, rt)
        rt.arena.reset(mark)


class _NormAfter(Arrangement):
    """x += norm(mixer(x)); x += norm(feed_forward(x)): the sublayers read the residual stream itself
    and the norm stands on what they put out.  A sublayer adds its output into the stream it is handed;
    here that is a cleared float32 buffer y, which the norm then folds into x.  The same kernel writes
    the next sublayer's input (x in the activation type) and clears y again, and both buffers are kept
    from layer to layer of a pass, so a layer costs no conversion or clearing kernel of its own after
    the first."""

    def _buffers(self, x, rt):
        carry = getattr(rt, "_norm_after_carry", None)
        if carry is not None and carry[0] == (rt.pass_id, x.data_ptr(), tuple(x.shape)):
            return carry[1], carry[2]
        y = rt.arena.alloc(tuple(x.shape), x.dtype)
        y.zero_()
        if rt.dtype == x.dtype:
            h = x                                   # 32-bit run: the sublayers read x in place
        else:
            h = rt.arena.alloc(tuple(x.shape), rt.dtype)
            rt.launches += 1
            ops.convert(x, h)
        rt._norm_after_carry = ((rt.pass_id, x.data_ptr(), tuple(x.shape)), h, y)
        return h, y

    def run(self, layer, x, batch, cache, rt):
        h, y = self._buffers(x, rt)
        hn = None if h is x else h
        mark = rt.arena.mark()
        layer.mixer.forward(h, y, batch, cache, rt)
        layer.mixer_norm.add_normed(y, x, rt, h=hn, clear=True)
        rt.arena.reset(mark)
        ff = getattr(layer, "feed_forward", None)
        if ff is not None:
            ff.forward(h, y, batch, rt)
            layer.feed_forward_norm.add_normed(y, x, rt, h=hn, clear=True)
            rt.arena.reset(mark)


@register_part("arrangement", "norm_after")
class NormAfter(_NormAfter):
    roles = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "feed_forward_norm": "norm"}

    def __init__(self):
        pass


@register_part("arrangement", "norm_after_mixer_only")
class NormAfterMixerOnly(_NormAfter):
    """The same layer without a feed-forward."""
    roles = {"mixer": "mixer", "mixer_norm": "norm"}

    def __init__(self):
        pass


@register_part("residual_gate", "sigmoid_linear")
class SigmoidLinearGate(ResidualGate):
    """x += sigmoid(W h + b) * y, element by element: a square projection of the sublayer's own input opens
    or closes every channel of its result.  The projection's sums, the sigmoid and the sum into the stream
    are float32 (for few tokens the product runs in K slices that the joining kernel adds up)."""

    def __init__(self, width: int, bias: bool = True):
        self.width, self.bias = int(width), bool(bias)
        self.w = self.b = None

    def weight_specs(self):
        s = [WeightSpec("weight", (self.width, self.width))]
        if self.bias:
            s.append(WeightSpec("bias", (self.width,), "vector", ("normal", 0.5)))
        return s

    def bind(self, tensors, rt):
        self.w = tensors["weight"].contiguous()
        self.b = tensors["bias"].float().contiguous() if self.bias else None

    @staticmethod
    def _sums(h, w, rt):
        g = rt.matmul_parts(h, w)
        if g is None:
            g = rt.arena.alloc((h.shape[0], w.shape[0]), torch.float32)
            rt.matmul(h, w, g)
        return g

    def input_weight(self):
        return self.w

    def adopt_input_weight(self, w):
        self.w = w

    def join(self, h, y, x, rt, sums=None):
        g = sums if sums is not None else self._sums(h, self.w, rt)
        rt.launches += 1
        ops.gated_add(g, self.b, y, x, clear_y=True)


class _ParallelGated(Arrangement):
    """h = norm(x); x += gate_m(h) * mixer(h) + gate_f(h) * feed_forward(h): one norm, both sublayers read
    its output, and each result passes a gate of its own (family ``residual_gate``) into the stream.  A
    sublayer adds its output into the stream it is handed; here that is a cleared float32 buffer y, which
    the gate's kernel folds into x and clears again.  y is kept from layer to layer of a pass."""

    def _buffer(self, x, rt):
        carry = getattr(rt, "_parallel_gated_carry", None)
        if carry is not None and carry[0] == (rt.pass_id, x.data_ptr(), tuple(x.shape)):
            return carry[1]
        y = rt.arena.alloc(tuple(x.shape), x.dtype)
        y.zero_()
        rt._parallel_gated_carry = ((rt.pass_id, x.data_ptr(), tuple(x.shape)), y)
        return y

    def run(self, layer, x, batch, cache, rt):
        y = self._buffer(x, rt)
        mark = rt.arena.mark()
        h = layer.norm.forward(x, rt)
        ff = getattr(layer, "feed_forward", None)
        gates = [layer.mixer_gate] + ([layer.feed_forward_gate] if ff is not None else [])
        # one product for everything that reads h and takes float32 sums: the mixer's input projections and the gates'
        sums = self._input_sums(layer, [layer.mixer] + gates, h, rt)
        inner = rt.arena.mark()
        if sums[0] is not None:
            layer.mixer.forward(h, y, batch, cache, rt, projected=sums[0])
        else:
            layer.mixer.forward(h, y, batch, cache, rt)
        gates[0].join(h, y, x, rt, sums[1])
        rt.arena.reset(inner)
        if ff is not None:
            ff.forward(h, y, batch, rt)
            gates[1].join(h, y, x, rt, sums[2])
        rt.arena.reset(mark)

    @staticmethod
    def _input_sums(layer, parts, h, rt):
        """For each of ``parts`` the float32 sums of h with its ``input_weight`` (None where it has none), from ONE
        product over the stacked matrices.  The stack is made at the layer's first run; the parts then hold views
        of it instead of copies of their own."""
        plan = getattr(layer, "_stacked_inputs", None)
        if plan is None:
            ws = [p.input_weight() for p in parts]
            take = [i for i, w in enumerate(ws) if w is not None]
            plan = False
            if FUSE_INPUTS and len(take) > 1 and len({(ws[i].dtype, ws[i].shape[1], ws[i].device) for i in take}) == 1:
                stacked = torch.cat([ws[i] for i in take], dim=0).contiguous()
                spans, at = {}, 0
                for i in take:
                    spans[i] = (at, at + ws[i].shape[0])
                    parts[i].adopt_input_weight(stacked[at:at + ws[i].shape[0]])
                    at += ws[i].shape[0]
                plan = (stacked, spans)
            layer._stacked_inputs = plan
        if not plan:
            return [None] * len(parts)
        stacked, spans = plan
        s = rt.matmul_parts(h, stacked)
        if s is None:
            s = rt.arena.alloc((h.shape[0], stacked.shape[0]), torch.float32)
            rt.matmul(h, stacked, s)
        return [s[..., spans[i][0]:spans[i][1]] if i in spans else None for i in range(len(parts))]


@register_part("arrangement", "parallel_gated")
class ParallelGated(_ParallelGated):
    roles = {"norm": "norm", "mixer": "mixer", "mixer_gate": "residual_gate", "feed_forward": "feed_forward",
             "feed_forward_gate": "residual_gate"}

    def __init__(self):
        pass


@register_part("arrangement", "parallel_gated_mixer_only")
class ParallelGatedMixerOnly(_ParallelGated):
    """The same layer without a feed-forward."""
    roles = {"norm": "norm", "mixer": "mixer", "mixer_gate": "residual_gate"}

    def __init__(self):
        pass


@register_part("entry", "pass_marker")
class PassMarker(Entry):
    """Before pass ``index`` of a group of layers that runs ``times`` times: x += step[index], one learned row
    a pass (tensor ``step`` [times, width], shared by the passes' markers), and on every pass but the
    first the embedding's output is added to the stream again."""

    def __init__(self, width: int, times: int, index: int):
        self.width, self.times, self.index = int(width), int(times), int(index)
        if not (0 <= self.index < self.times):
            raise ValueError("pass_marker: the pass's number must lie below the number of passes")
        self.needs_embedding_output = self.index > 0
        self.row = None

    def weight_specs(self):
        return [WeightSpec("step", (self.times, self.width), "vector", ("normal", 0.1))]

    def bind(self, tensors, rt):
        self.row = tensors["step"].float()[self.index].contiguous()

    def forward(self, x, x0, rt):
        rt.launches += 1
        ops.add_rows(x, x0 if self.index > 0 else None, self.row)


class _HyperPreNorm(Arrangement):
    """A pre-norm layer over a residual stream kept in several copies (``ModelSpec.streams``): each sublayer reads
    the copies through its connection and its norm, adds its result into a cleared float32 buffer y, and the
    connection puts y into every copy (and clears it).  The mixer's write and the feed-forward's read are one pass
    over the copies.  y is kept from layer to layer of a pass."""

    def _buffer(self, xs, rt):
        carry = getattr(rt, "_hyper_carry", None)
        key = (rt.pass_id, xs.data_ptr(), tuple(xs.shape))
        if carry is not None and carry[0] == key:
            return carry[1]
        y = rt.arena.alloc(tuple(xs.shape[1:]), xs.dtype)
        y.zero_()
        rt._hyper_carry = (key, y)
        return y

    def run(self, layer, xs, batch, cache, rt):
        if xs.dim() != 3:
            raise ValueError("this arrangement runs on a stream kept in copies (ModelSpec.streams > 0)")
        y = self._buffer(xs, rt)
        mark = rt.arena.mark()
        h = layer.mixer_connection.read(xs, layer.mixer_norm, rt)
        layer.mixer.forward(h, y, batch, cache, rt)
        rt.arena.reset(mark)
        ff = getattr(layer, "feed_forward", None)
        if ff is None:
            layer.mixer_connection.write(xs, y, rt)
            return
        h = layer.mixer_connection.write(xs, y, rt, then=(layer.feed_forward_connection, layer.feed_forward_norm))
        ff.forward(h, y, batch, rt)
        layer.feed_forward_connection.write(xs, y, rt)
        rt.arena.reset(mark)


@register_part("arrangement", "hyper_pre_norm")
class HyperPreNorm(_HyperPreNorm):
    roles = {"mixer_connection": "connection", "mixer_norm": "norm", "mixer": "mixer",
             "feed_forward_connection": "connection", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self):
        pass


@register_part("arrangement", "hyper_pre_norm_mixer_only")
class HyperPreNormMixerOnly(_HyperPreNorm):
    """The same layer without a feed-forward."""
    roles = {"mixer_connection": "connection", "mixer_norm": "norm", "mixer": "mixer"}

    def __init__(self):
        pass


@register_part("arrangement", "pre_norm_mixer_only")
class PreNormMixerOnly(Arrangement):
    """x += mixer(norm(x)): the pre-norm block without a feed-forward."""
    roles = {"mixer_norm": "norm", "mixer": "mixer"}

    def __init__(self):
        pass

    def run(self, layer, x, batch, cache, rt):
        mark = rt.arena.mark()
        h = layer.mixer_norm.forward(x, rt)
        layer.mixer.forward(h, x, batch, cache, rt)
        rt.arena.reset(mark)
