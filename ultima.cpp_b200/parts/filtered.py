"""A pre-norm layer whose sublayers read their input through a filter over time and whose results are scaled
channel by channel on their way into the stream, with something done to the stream behind the sublayers:

    h = filter1(norm1(x));  x += gate1 * mixer(h);  h = filter2(norm2(x));  x += gate2 * feed_forward(h);  tail(x)

The pieces are parts of families of their own, so that another design can take one without the others:
``residual_gate`` "layer_scale" (and "plain"), ``input_filter`` "causal_conv_residual" (and "none"), ``tail``
"token_side" (and "none").
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import Arrangement, InputFilter, ResidualGate, StateNeed, Tail, register_part


def _next_mode(then):
    """How the joining kernel writes what the next reader wants: (mode, weight, eps), or None if it cannot."""
    if then is None:
        return ops.NEXT_NONE, None, 0.0
    if then == "plain":
        return ops.NEXT_PLAIN, None, 0.0
    kind = getattr(then, "kind", None)
    if kind == "layer":
        return ops.NEXT_LAYER, then.weight, then.eps
    if kind == "rms":
        return ops.NEXT_RMS, then.weight, then.eps
    return None


class _ChannelGate(ResidualGate):
    """x += s * y with one constant a channel (or 1), y cleared; the same kernel writes what comes next: ``then`` is
    None, "plain" (the new x in the activation type) or a norm of kind "layer" / "rms" (its output); any other norm is
    run behind the join.  Returns that output (None for ``then`` None)."""

    scale = None

    def kernel_needs(self, run_dtype):
        return [("rowwise.cu", ())]

    def join(self, h, y, x, rt, sums=None, then=None):
        how = _next_mode(then)
        rt.launches += 1
        if how is None:
            ops.scale_add_norm(y, self.scale, x)
            return then.forward(x, rt)
        mode, w, eps = how
        if mode == ops.NEXT_PLAIN and rt.dtype == x.dtype:
            ops.scale_add_norm(y, self.scale, x)
            return x                                   # a 32-bit run reads the stream itself
        out = rt.arena.alloc(tuple(x.shape), rt.dtype) if mode != ops.NEXT_NONE else None
        ops.scale_add_norm(y, self.scale, x, mode, w, eps, out)
        return out


@register_part("residual_gate", "layer_scale")
class LayerScale(_ChannelGate):
    """A sublayer's result is multiplied element by element by a learned vector (tensor ``scale`` [width]) before the
    sum; the product and the sum are float32."""

    def __init__(self, width: int):
        self.width = int(width)

    def weight_specs(self):
        return [WeightSpec("scale", (self.width,), "vector", ("normal", 0.3))]

    def bind(self, tensors, rt):
        self.scale = tensors["scale"].float().contiguous()


@register_part("residual_gate", "plain")
class PlainSum(_ChannelGate):
    """x += y."""

    def __init__(self):
        pass


@register_part("input_filter", "none")
class NoFilter(InputFilter):
    def __init__(self):
        pass

    def forward(self, h, batch, cache, rt):
        return h


@register_part("input_filter", "causal_conv_residual")
class CausalConvResidual(InputFilter):
    """h_t <- h_t + sum_j w[:, j] h_(t - taps + 1 + j): a causal convolution over time on every channel (tensor ``weight``
    [width, taps], no bias, zeros before a sequence's start), added to its own input.  The last taps - 1 inputs are
    per-sequence state (float32).  The sums are float32."""

    def __init__(self, width: int, taps: int):
        self.width, self.taps = int(width), int(taps)
        if not (1 <= self.taps <= 16):
            raise ValueError(f"causal_conv_residual: {self.taps} taps is not what the kernel takes (1 to 16)")

    def weight_specs(self):
        return [WeightSpec("weight", (self.width, self.taps), "vector", ("normal", 0.2))]

    def cache_need(self):
        return StateNeed((self.taps - 1, self.width), "float32") if self.taps > 1 else None

    def kernel_needs(self, run_dtype):
        return [("rowwise.cu", ())]

    def bind(self, tensors, rt):
        self.w = tensors["weight"].float().contiguous()

    def forward(self, h, batch, cache, rt):
        out = rt.arena.alloc(tuple(h.shape), h.dtype)
        state = cache.states[0] if self.taps > 1 else None
        one_each = batch.max_new == 1 and batch.n_seqs == h.shape[0]      # one token a sequence: the kernel moves the state on itself
        rt.launches += 1
        ops.causal_conv(h, self.w, state, batch, out, add_input=True, update_state=one_each)
        if self.taps > 1 and not one_each:
            rt.launches += 1
            ops.causal_conv_state(h, state, batch)
        return out


@register_part("tail", "none")
class NoTail(Tail):
    needs_activations = False

    def __init__(self):
        pass

    def forward(self, x, xa, batch, rt):
        pass


@register_part("tail", "token_side")
class TokenSide(Tail):
    """A per-layer input from the token itself: with e the columns [index * dim, (index + 1) * dim) of the token's row
    of a second embedding table (tensor ``embed`` [vocab, tables * dim], shared by the layers),

        g = gelu_tanh(W_gate x) * e;   y = W_proj g;   x += y / sqrt(mean(y^2) + eps) * norm

    (``gate`` [dim, width], ``proj`` [width, dim], ``norm`` [width], a plain RMS-norm weight).  The two products read
    the activation type; the GELU, the norm and the sum are float32."""
    needs_activations = True

    def __init__(self, width: int, vocab_size: int, dim: int, index: int, tables: int, eps: float):
        self.width, self.vocab, self.dim = int(width), int(vocab_size), int(dim)
        self.index, self.tables, self.eps = int(index), int(tables), float(eps)
        if not (0 <= self.index < self.tables) or self.dim < 1:
            raise ValueError("token_side: the layer's columns must lie inside the table")
        self.dim_pad = -(-self.dim // 8) * 8

    def weight_specs(self):
        return [WeightSpec("embed", (self.vocab, self.tables * self.dim)),
                WeightSpec("gate", (self.dim, self.width)),
                WeightSpec("proj", (self.width, self.dim)),
                WeightSpec("norm", (self.width,), "vector", ("one_plus_normal", 0.05))]

    def kernel_needs(self, run_dtype):
        return [("rowwise.cu", ())]

    def bind(self, tensors, rt):
        # one copy of the table for all layers
        t = tensors["embed"]
        self.table = rt.shared(("token_side_table", t.data_ptr()), lambda: t.contiguous())
        self.w_gate = tensors["gate"].contiguous()
        p = tensors["proj"]
        if self.dim_pad != self.dim:                   # an aligned operand: columns of zeros
            wp = torch.zeros((self.width, self.dim_pad), dtype=p.dtype, device=p.device)
            wp[:, :self.dim] = p
            p = wp
        self.w_proj = p.contiguous()
        self.norm_w = tensors["norm"].float().contiguous()

    def forward(self, x, xa, batch, rt):
        T = x.shape[0]
        s = rt.arena.alloc((T, self.dim), torch.float32)
        rt.matmul(xa, self.w_gate, s)
        g = rt.arena.alloc((T, self.dim_pad), rt.dtype)
        rt.launches += 1
        ops.side_gate(s, self.table, self.index * self.dim, batch.tok_ids, g, self.dim)
        y = rt.arena.alloc((T, self.width), torch.float32)
        rt.matmul(g, self.w_proj, y)
        rt.launches += 1
        ops.rmsnorm_add(y, self.norm_w, x, self.eps)


class _PreNormFiltered(Arrangement):
    """See the module's text.  Sublayers add into a cleared float32 buffer y that lives from layer to layer of a pass; a
    gate's kernel folds y into x, clears it, and writes the next norm's output in the same pass over the row.  The
    filters' state and the mixer's cache are shares of the run's cache."""
    shares_cache = True

    def _buffer(self, x, rt):
        carry = getattr(rt, "_filtered_carry", None)
        key = (rt.pass_id, x.data_ptr(), tuple(x.shape))
        if carry is not None and carry[0] == key:
            return carry[1]
        y = rt.arena.alloc(tuple(x.shape), x.dtype)
        y.zero_()
        rt._filtered_carry = (key, y)
        return y

    def run(self, layer, x, batch, cache, rt):
        y = self._buffer(x, rt)
        mark = rt.arena.mark()
        ff = getattr(layer, "feed_forward", None)
        tail = layer.tail
        after = "plain" if getattr(tail, "needs_activations", False) else None
        h = layer.mixer_norm.forward(x, rt)
        h = layer.mixer_filter.forward(h, batch, layer.cache_of("mixer_filter", cache), rt)
        layer.mixer.forward(h, y, batch, layer.cache_of("mixer", cache), rt)
        rt.arena.reset(mark)
        if ff is None:
            xa = layer.mixer_gate.join(None, y, x, rt, then=after)
        else:
            h = layer.mixer_gate.join(None, y, x, rt, then=layer.feed_forward_norm)
            h = layer.feed_forward_filter.forward(h, batch, layer.cache_of("feed_forward_filter", cache), rt)
            ff.forward(h, y, batch, rt)
            rt.arena.reset(mark)
            xa = layer.feed_forward_gate.join(None, y, x, rt, then=after)
        tail.forward(x, xa, batch, rt)
        rt.arena.reset(mark)


@register_part("arrangement", "pre_norm_filtered")
class PreNormFiltered(_PreNormFiltered):
    roles = {"mixer_norm": "norm", "mixer_filter": "input_filter", "mixer": "mixer", "mixer_gate": "residual_gate",
             "feed_forward_norm": "norm", "feed_forward_filter": "input_filter", "feed_forward": "feed_forward",
             "feed_forward_gate": "residual_gate", "tail": "tail"}

    def __init__(self):
        pass


@register_part("arrangement", "pre_norm_filtered_mixer_only")
class PreNormFilteredMixerOnly(_PreNormFiltered):
    """The same layer without a feed-forward."""
    roles = {"mixer_norm": "norm", "mixer_filter": "input_filter", "mixer": "mixer", "mixer_gate": "residual_gate",
             "tail": "tail"}

    def __init__(self):
        pass
