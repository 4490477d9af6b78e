"""The attention mixer: grouped-query attention over the cache, with optional per-head norm
of queries and keys, an optional position encoding (any part of the "position" family) and an
optional window."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import Mixer, KVNeed, PartSpec, StateNeed, build_part, register_part


@register_part("mixer", "attention")
class Attention(Mixer):
    """q, k, v projections (no bias), per-head RMSNorm of q and k before the rotation when
    ``qk_norm`` (one weight of head size for all heads, the layer's eps), rotation, write of
    k and v into the cache before reading so a token sees itself, softmax(q k / sqrt(d)) v
    with query head h on KV head h // (heads / kv heads), output projection added to the
    residual stream.  Reference: src/model/qwen_block.cpp:682-690, :713-727, :732-751,
    :775-783, :94-135.

    The three projections are held as one matrix [q | k | v] and run as one product.

    Further parameters, each off by default:
      v_head_dim  the values' head size where it is not the keys'
      block       a token at position p sees j <= p only with j // block == p // block (blocks are
                  counted from the sequence's start, whatever a step brings)
      head_gate   one more projection of the mixer's input, one number a head; a head's output is
                  multiplied by its sigmoid before the output projection
      own_kv      False: the layer has no key and value tensors; its run reads another run's cache
                  (``Run.cache_from``) with its own queries
      norm_whole  the q/k norm runs over all of a token's query heads at once (and over all its key heads),
                  with one weight a column of the projection, instead of head by head
      window + keep_first   behind a window of ``window`` positions the sequence's first ``keep_first``
                  positions stay visible (the cache then holds every position)
      distance_slope   a: head h (of H) takes 2^(-a (h + 1) / H) * (distance to the key) off every score
      sink        the softmax's sum has one more term exp(0), which brings no value
      values_are_keys   no value projection: a position's value is its key as projected, before norm and
                  rotation (the cache holds both forms)
      wide_gate   one more projection of the mixer's input, one number an output element; the heads' outputs
                  are multiplied by its sigmoid before the output projection
      out_scale   a constant on the mixer's output (applied to the heads' outputs, in float32)
      softcap     c: a scaled score s becomes c * tanh(s / c)
      distance_buckets   (B, D): a learned bias by distance, tensor ``rel`` [B, heads]; the key at distance n adds
                  rel[bucket(n), h] to the score (behind scale and cap): bucket(n) = n below B // 2, beyond that
                  min(B - 1, B // 2 + floor(ln(n / (B // 2)) / ln(D / (B // 2)) * (B - B // 2))), equal steps of ln(n) up to D
      learned_sink   the sink's term is exp(sink[h]) with a learned number a head (tensor ``sink`` [heads]) instead of exp(0)
      in_bias     the q, k and v projections have biases (tensors ``q_proj.bias`` ...), added to the projection's sums
      conv        taps of a short causal convolution over time on every channel of q, k and v (tensors ``q_conv.weight``
                  [channels, taps] ..., no bias, the last tap on the current token, zeros before the sequence), directly behind
                  the projection and its bias, before norm and rotation; the last taps - 1 projected rows are per-sequence
                  state (float32), so the layer then asks the cache for keys, values AND a state
      value_mix   "source": the layer's values (behind the convolution) are also handed to the later layers of the pass that
                  say "blend"; those replace their own by (1 - lam) * own + lam * the source's values of the same token (tensor
                  ``vmix``, a scalar) before they are cached.  ``value_mix_key`` tells groups of such layers apart.  Both
                  layers' value rows must have the same width.
    The last three run as one kernel between the projection and the placement (csrc/rowwise.cu).
    With any of them the layer runs on the general kernels (csrc/attn_simple.cu: placement of q, k, v from
    one fused projection row [q | k | v | gate], attention with the mask and the gate inside); a block
    mask alone, with equal head sizes, still takes the tensor-core attention kernels.
    """

    @property
    def graph_safe(self) -> bool:
        """Launches kernels only, no host work that depends on the data; a position encoding it holds
        has to say the same of itself."""
        return self.position is None or bool(getattr(self.position, "graph_safe", False))

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, qk_norm: bool,
                 eps: float, position: PartSpec | None, window: int | None = None,
                 scale: float | None = None, v_head_dim: int | None = None, block: int | None = None,
                 head_gate: bool = False, own_kv: bool = True, norm_whole: bool = False, keep_first: int = 0,
                 distance_slope: float | None = None, sink: bool = False, values_are_keys: bool = False,
                 wide_gate: bool = False, out_scale: float = 1.0, softcap: float | None = None,
                 distance_buckets: tuple | None = None, learned_sink: bool = False, in_bias: bool = False, conv: int = 0,
                 value_mix: str | None = None, value_mix_key: str = ""):
        if n_heads % n_kv_heads:
            raise ValueError("heads must be a multiple of kv heads")
        self.width, self.nh, self.nkv, self.hd = int(width), int(n_heads), int(n_kv_heads), int(head_dim)
        self.qk_norm, self.eps, self.window = bool(qk_norm), float(eps), window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(self.hd)
        self.position = build_part("position", position) if position is not None else None
        self.q_width, self.kv_width = self.nh * self.hd, self.nkv * self.hd
        self.hdv = int(v_head_dim) if v_head_dim is not None else self.hd
        self.block = int(block) if block else None
        self.head_gate, self.own_kv = bool(head_gate), bool(own_kv)
        if self.block is not None and self.block < 1:
            raise ValueError("attention: a block mask needs a positive block size")
        self.o_width, self.v_width = self.nh * self.hdv, self.nkv * self.hdv
        self.norm_whole, self.keep_first, self.sink = bool(norm_whole) and self.qk_norm, int(keep_first or 0), bool(sink)
        self.distance_slope = float(distance_slope) if distance_slope is not None else None
        self.values_are_keys, self.wide_gate, self.out_scale = bool(values_are_keys), bool(wide_gate), float(out_scale)
        self.softcap = float(softcap) if softcap else None
        self.distance_buckets = (int(distance_buckets[0]), float(distance_buckets[1])) if distance_buckets else None
        self.learned_sink = bool(learned_sink)
        if self.learned_sink:
            self.sink = True
        if self.distance_buckets is not None and (self.distance_buckets[0] < 2 or self.distance_buckets[1] <= self.distance_buckets[0] // 2):
            raise ValueError("attention: a bias by distance needs at least two buckets and a largest distance beyond the "
                             "buckets that hold one distance each")
        if self.softcap is not None and self.softcap <= 0:
            raise ValueError("attention: the score cap must be positive")
        if self.values_are_keys and (self.hdv != self.hd or not self.own_kv):
            raise ValueError("attention: values that are the keys have the keys' head size and belong to the layer itself")
        if self.wide_gate and self.head_gate:
            raise ValueError("attention: one gate a head or one an element, not both")
        if self.keep_first and (self.window is None or self.block is not None):
            raise ValueError("attention: kept first positions go with a window (and not with a block mask)")
        if self.keep_first < 0:
            raise ValueError("attention: keep_first must not be negative")
        # what only the row-wise placement and the any-shape attention kernel take
        interleaved = self.position is not None and bool(getattr(self.position, "interleaved", False))
        self.extended = (self.norm_whole or self.keep_first > 0 or self.distance_slope is not None or self.sink
                         or self.values_are_keys or self.wide_gate or self.out_scale != 1.0 or self.softcap is not None
                         or self.distance_buckets is not None)
        self._table_options = self.softcap is not None or self.distance_buckets is not None or self.learned_sink
        self.in_bias, self.conv = bool(in_bias), int(conv or 0)
        self.value_mix, self.value_mix_key = value_mix, str(value_mix_key)
        if value_mix not in (None, "source", "blend"):
            raise ValueError("attention: value_mix is 'source', 'blend' or None")
        if not (0 <= self.conv <= 16):
            raise ValueError(f"attention: a convolution of {self.conv} taps is not one the kernel takes (at most 16)")
        # projections that are reshaped (bias, convolution, blended values) before they are placed
        self.shaped = self.in_bias or self.conv > 0 or self.value_mix is not None
        if self.shaped and (self.head_gate or self.wide_gate or self.values_are_keys or not self.own_kv):
            raise ValueError("attention: biases, a convolution and blended values go with plain q, k and v projections of the "
                             "layer's own")
        self.place_rows = (self.norm_whole or self.values_are_keys or self.wide_gate or (self.extended and interleaved)
                           or self.shaped)
        self.general = (self.hdv != self.hd or self.block is not None or self.head_gate or not self.own_kv
                        or self.extended or self.shaped)
        self.wqkv = self.wo = self.q_norm = self.k_norm = None

    def weight_specs(self):
        s = [WeightSpec("q_proj.weight", (self.q_width, self.width))]
        if self.own_kv:
            s.append(WeightSpec("k_proj.weight", (self.kv_width, self.width)))
            if not self.values_are_keys:
                s.append(WeightSpec("v_proj.weight", (self.v_width, self.width)))
        s.append(WeightSpec("o_proj.weight", (self.width, self.o_width)))
        if self.qk_norm:
            s.append(WeightSpec("q_norm.weight", (self.q_width if self.norm_whole else self.hd,), "vector",
                                ("one_plus_normal", 0.05)))
            if self.own_kv:
                s.append(WeightSpec("k_norm.weight", (self.kv_width if self.norm_whole else self.hd,), "vector",
                                    ("one_plus_normal", 0.05)))
        if self.head_gate:
            s.append(WeightSpec("gate_proj.weight", (self.nh, self.width)))
        if self.wide_gate:
            s.append(WeightSpec("gate_proj.weight", (self.o_width, self.width)))
        if self.distance_buckets is not None:
            s.append(WeightSpec("rel", (self.distance_buckets[0], self.nh), "vector", ("normal", 0.5)))
        if self.learned_sink:
            s.append(WeightSpec("sink", (self.nh,), "vector", ("normal", 1.0)))
        for n, rows in (("q", self.q_width), ("k", self.kv_width), ("v", self.v_width)):
            if self.in_bias:
                s.append(WeightSpec(f"{n}_proj.bias", (rows,), "vector", ("normal", 0.1)))
            if self.conv > 0:
                s.append(WeightSpec(f"{n}_conv.weight", (rows, self.conv), "vector", ("normal", 0.4)))
        if self.value_mix is not None:
            s.append(WeightSpec("vmix", (), "vector", ("normal", 0.5)))
        return s

    def cache_need(self):
        # kept first positions lie outside any ring of the window's size: the cache then holds all positions
        kv = KVNeed(self.nkv, self.hd, None if self.keep_first else self.window, self.hdv if self.hdv != self.hd else None)
        if self.conv > 1:
            return (kv, StateNeed((self.conv - 1, self.q_width + self.kv_width + self.v_width), "float32"))
        return kv

    def kernel_needs(self, run_dtype):
        from ..kernels import attn_tc, catalog
        shaping = [("rowwise.cu", ())] if self.shaped else []
        if run_dtype != torch.bfloat16:
            return [("attn_simple.cu", ())] + shaping
        if self.general:
            out = [("attn_simple.cu", ())] + shaping
            if self.extended:
                if self._fast_extended() and attn_tc.EXTENDED:
                    out.append(attn_tc.target(self.hd))
                    if self.hd in catalog.TC_HEAD_DIMS and not self.window and self.distance_slope is None:
                        out.append(attn_tc.tc_target(self.hd))
                return out
            if self._fast_attention() and attn_tc.BLOCK_MASK:
                out.append(attn_tc.target(self.hd))
                if self.hd in catalog.TC_HEAD_DIMS:
                    out.append(attn_tc.tc_target(self.hd))
            return out
        if self.hd % 16 == 0 and 16 <= self.hd <= 256:
            out = [attn_tc.target(self.hd)]
            if self.hd in catalog.TC_HEAD_DIMS:
                out.append(attn_tc.tc_target(self.hd))
            return out
        return [("attn_simple.cu", ())]

    def _fast_attention(self) -> bool:
        """Whether a general layer's attention itself can still go to the tensor-core kernels: equal head
        sizes of a kind they take; the block mask they know, the gate is applied behind them."""
        return self.hdv == self.hd and self.hd % 16 == 0 and 16 <= self.hd <= 256 and not self.extended

    def _fast_extended(self) -> bool:
        """Whether a layer with the further options can go to the tensor-core kernels that know them (mma.sync):
        equal head sizes of a kind they take, no block mask, no gate a head."""
        return (self.extended and self.hdv == self.hd and self.hd % 16 == 0 and 16 <= self.hd <= 256
                and self.block is None and not self.head_gate and self.own_kv)

    def bind(self, tensors, rt):
        if (self.hd % 2 and not self.general) or self.hd > ops.MAX_HEAD_DIM or self.hdv > ops.MAX_HEAD_DIM:
            raise ValueError(f"attention: head size {self.hd} is not one the kernels take (even, at most "
                             f"{ops.MAX_HEAD_DIM})")
        ws = [tensors["q_proj.weight"]]
        if self.own_kv:
            ws.append(tensors["k_proj.weight"])
            if not self.values_are_keys:
                ws.append(tensors["v_proj.weight"])
        if self.head_gate or self.wide_gate:
            ws.append(tensors["gate_proj.weight"])
        if len({w.dtype for w in ws}) != 1:
            raise ValueError("q, k and v projections must share one element type")
        self.wqkv = torch.cat(ws, dim=0).contiguous()
        self.wo = tensors["o_proj.weight"].contiguous()
        if self.qk_norm:
            self.q_norm = tensors["q_norm.weight"].float().contiguous()
            if self.own_kv:
                self.k_norm = tensors["k_norm.weight"].float().contiguous()
        if self.position is not None:
            self.position.bind({}, rt)
            if self.general and self.position.rotation() is None:
                raise ValueError("attention: with a block mask, a gate, unequal head sizes or shared keys the "
                                 "position encoding must be a rotation of pairs")
            if self.general and self.position.rotation().interleaved and not self.place_rows:
                raise ValueError("attention: the head-wise placement kernel rotates pairs (j, j + rotary_dim / 2) only")
        names = ("q", "k", "v")
        self.bias_qkv = torch.cat([tensors[f"{n}_proj.bias"].float() for n in names]).contiguous() if self.in_bias else None
        self.conv_w = torch.cat([tensors[f"{n}_conv.weight"].float() for n in names], dim=0).contiguous() if self.conv > 0 else None
        self.lam = tensors["vmix"].float().reshape(1).contiguous() if self.value_mix is not None else None
        self.sink_vals = tensors["sink"].float().contiguous() if self.learned_sink else None
        self.dist_bias = None
        if self.distance_buckets is not None:
            # the table by distance itself: row n is the bucket's row of ``rel``; beyond D every distance has the last bucket
            B, D = self.distance_buckets
            half = B // 2
            reach = int(math.ceil(D)) + 1
            if self.window:
                reach = min(reach, int(self.window))
            bucket = [n if n < half else min(B - 1, half + int(math.floor(math.log(n / half) / math.log(D / half) * (B - half))))
                      for n in range(reach)]
            rel = tensors["rel"].float()
            self.dist_bias = rel[torch.tensor(bucket, dtype=torch.long, device=rel.device)].contiguous()
        self.slopes = self.slopes_log2 = None
        if self.distance_slope is not None:
            h = torch.arange(1, self.nh + 1, dtype=torch.float64)
            slopes = torch.pow(torch.tensor(2.0, dtype=torch.float64), -self.distance_slope * h / self.nh)
            self.slopes = slopes.float().contiguous().to(rt.device)
            self.slopes_log2 = (slopes * math.log2(math.e)).float().contiguous().to(rt.device)   # for kernels that work in powers of two

    def input_weight(self):
        """The stacked [q | k | v | gate] matrix of a layer on the general kernels, which take its float32 sums."""
        return self.wqkv if self.general else None

    def adopt_input_weight(self, w):
        self.wqkv = w

    def _forward_general(self, h, residual, batch, cache, rt, projected=None):
        """One product [q | k | v | gate] in float32, placement (norm, rotation, cache write), attention
        with the block mask, the gate, the output projection."""
        T = h.shape[0]
        kv = cache.kv
        if kv.owner != self.own_kv:
            raise ValueError("attention: a layer without keys and values of its own must read another run's "
                             "cache, and one with them must own its cache")
        rot = self.position.rotation() if self.position is not None else None
        x = projected if projected is not None else rt.matmul_parts(h, self.wqkv)    # few tokens: K in slices, summed by the placement kernel
        if x is None:
            x = rt.arena.alloc((T, self.wqkv.shape[0]), torch.float32)
            rt.matmul(h, self.wqkv, x)
        if self.shaped:
            x = self._shape_projections(x, T, batch, cache, rt)
        q = rt.arena.alloc((T, self.q_width), rt.dtype)
        k_off = self.q_width if self.own_kv else None
        v_off = (k_off if self.values_are_keys else self.q_width + self.kv_width) if self.own_kv else None
        g_off = self.q_width + ((self.kv_width + (0 if self.values_are_keys else self.v_width)) if self.own_kv else 0)
        gate = rt.arena.alloc((T, self.nh), torch.float32) if self.head_gate else None
        if self.wide_gate:
            gate = rt.arena.alloc((T, self.o_width), torch.float32)
        rt.launches += 1
        if self.place_rows:
            ops.qkv_place_rows(x, 0, k_off, v_off, q, self.q_norm, self.k_norm, self.norm_whole, rot.cos if rot else None,
                               rot.sin if rot else None, rot.dim if rot else 0, bool(rot.interleaved) if rot else False,
                               batch.tok_pos, batch.tok_seq, kv.k, kv.v, kv.table, kv.ring, kv.page, self.nh, self.nkv,
                               self.hd, self.hdv, self.eps, g_off, gate)
        else:
            ops.qkv_place(x, 0, k_off, v_off, q, self.q_norm, self.k_norm, rot.cos if rot else None,
                          rot.sin if rot else None, rot.dim if rot else 0, batch.tok_pos, batch.tok_seq, kv.k, kv.v,
                          kv.table, kv.ring, kv.page, self.nh, self.nkv, self.hd, self.hdv, self.eps, g_off, gate)
        o = rt.arena.alloc((T, self.o_width), rt.dtype)
        if self._fast_extended() and rt.attention_ext(q, kv, o, batch, self.nh, self.nkv, self.hd, self.scale, window=self.window,
                                                      keep_first=self.keep_first, sink=self.sink, slopes_log2=self.slopes_log2,
                                                      out_scale=self.out_scale, gate=gate, softcap=self.softcap,
                                                      dist_bias=self.dist_bias, sink_vals=self.sink_vals):
            pass
        elif self._fast_attention() and rt.attention_fast(q, kv, o, batch, self.nh, self.nkv, self.hd, self.scale,
                                                          self.block):
            if gate is not None:
                rt.launches += 1
                ops.head_gate(o, gate, self.nh, self.hdv)
        else:
            rt.launches += 1
            ops.attn_simple(q, kv.k, kv.v, o, batch.tok_pos, batch.tok_seq, kv.table, kv.ring, kv.page, self.nh,
                            self.nkv, self.hd, self.window, self.scale, v_head_dim=self.hdv, block=self.block, gate=gate,
                            keep_first=self.keep_first, slopes=self.slopes, sink=self.sink, out_scale=self.out_scale,
                            softcap=self.softcap, dist_bias=self.dist_bias, sink_vals=self.sink_vals)
        rt.matmul(o, self.wo, residual, ops.EPI_ADD)

    def _shape_projections(self, x, T, batch, cache, rt):
        """Bias, the short convolution over time and the blending of values, in one kernel: the float32 sums of the
        [q | k | v] product (whole or in K slices) become the rows that are normed, rotated and cached."""
        C = self.q_width + self.kv_width + self.v_width
        out = rt.arena.alloc((T, C), torch.float32)
        mix = None
        if self.value_mix is not None:
            first = rt.carry(("value_mix", self.value_mix_key), T, self.v_width, torch.float32)
            mix = (1 if self.value_mix == "source" else 2, self.q_width + self.kv_width, C, self.lam, first)
        state = cache.states[0] if self.conv > 1 else None
        one_each = batch.max_new == 1 and batch.n_seqs == T           # one token a sequence: the kernel moves the state on itself
        rt.launches += 1
        ops.causal_conv(x, self.conv_w, state, batch, out, bias=self.bias_qkv, mix=mix, update_state=one_each)
        if self.conv > 1 and not one_each:
            rt.launches += 1
            ops.causal_conv_state(x, state, batch, bias=self.bias_qkv)
        return out

    def forward(self, h, residual, batch, cache, rt, projected=None):
        if self.general:
            return self._forward_general(h, residual, batch, cache, rt, projected)
        T = h.shape[0]
        kv = cache.kv
        # A position encoding that describes itself as a rotation of pairs is applied by the kernels
        # that norm and write the cache; any other is called between the norm and the cache write.
        rot = self.position.rotation() if self.position is not None else None
        apart = self.position is not None and rot is None
        cos, sin = (rot.cos, rot.sin) if rot is not None else (None, None)
        whole = rot is None or (rot.dim == self.hd and not rot.interleaved)
        o = rt.arena.alloc((T, self.q_width), rt.dtype)
        parts = rt.matmul_parts(h, self.wqkv)        # few tokens: K in slices, summed by the next kernel
        if parts is not None:
            # one token a sequence: the attention kernel can take the slices as they are
            if not apart and whole and rt.attention_from_qkv(parts, self.q_norm, self.k_norm, cos, sin, self.eps, kv,
                                                             o, batch, self.nh, self.nkv, self.hd, self.scale):
                rt.matmul(o, self.wo, residual, ops.EPI_ADD)
                return
            qkv = parts
            q = rt.arena.alloc((T, self.q_width), rt.dtype)
        else:
            qkv = rt.arena.alloc((T, self.q_width + 2 * self.kv_width), rt.dtype)
            rt.matmul(h, self.wqkv, qkv)
            q = qkv[:, :self.q_width]
        rt.launches += 1
        if apart:
            kbuf = rt.arena.alloc((2, T, self.kv_width), q.dtype)
            ops.qk_prepare(qkv, self.q_norm, self.k_norm, None, None, batch.tok_pos, batch.tok_seq,
                           kv.k, kv.v, kv.table, kv.ring, kv.page, self.nh, self.nkv, self.hd, self.eps,
                           write_kv=kv.owner, q_out=q, kv_out=(kbuf[0], kbuf[1]))
            self.position.forward(q.view(T, self.nh, self.hd), kbuf[0].view(T, self.nkv, self.hd), batch.tok_pos, rt)
            if kv.owner:
                rt.launches += 1
                ops.kv_write(kbuf[0], kbuf[1], batch.tok_pos, batch.tok_seq, kv.k, kv.v, kv.table, kv.ring, kv.page,
                             self.nkv, self.hd)
        else:
            ops.qk_prepare(qkv, self.q_norm, self.k_norm, cos, sin, batch.tok_pos, batch.tok_seq,
                           kv.k, kv.v, kv.table, kv.ring, kv.page, self.nh, self.nkv, self.hd, self.eps,
                           write_kv=kv.owner, q_out=q, rotary_dim=rot.dim if rot is not None else None,
                           interleaved=bool(rot.interleaved) if rot is not None else False)
        rt.attention(q, kv, o, batch, self.nh, self.nkv, self.hd, self.scale)
        rt.matmul(o, self.wo, residual, ops.EPI_ADD)
