"""Token embedding and the output head."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import Part, StateNeed, register_part


@register_part("embedding", "token_table")
class TokenTable(Part):
    """x_t = E[id_t, :], no scaling (reference: src/model/qwen_model.cpp:145-157).  A token id
    outside the vocabulary is refused on the host before the launch; the kernel checks again
    and raises a flag."""

    def __init__(self, vocab_size: int, width: int, norm: str | None = None, eps: float = 0.0):
        """``norm``: "layer" or "rms": the gathered rows pass a norm with a weight of its own (tensor ``norm.weight``) and
        ``eps`` before they enter the stream (float32 in and out)."""
        self.vocab_size, self.width = int(vocab_size), int(width)
        if norm not in (None, "layer", "rms"):
            raise ValueError("token_table: norm is 'layer', 'rms' or None")
        self.norm, self.eps = norm, float(eps)
        self.table = self.norm_w = None

    def weight_specs(self):
        s = [WeightSpec("weight", (self.vocab_size, self.width))]
        if self.norm:
            s.append(WeightSpec("norm.weight", (self.width,), "vector", ("one_plus_normal", 0.05)))
        return s

    def kernel_needs(self, run_dtype):
        return [("rowwise.cu", ())] if self.norm == "layer" else []

    def bind(self, tensors, rt):
        self.table = tensors["weight"].contiguous()
        self.status = rt.status[0:1]
        if self.norm:
            self.norm_w = tensors["norm.weight"].float().contiguous()

    def forward(self, ids, rt):
        x = rt.arena.alloc((ids.numel(), self.width), torch.float32)
        rt.launches += 1
        ops.embed(self.table, ids, x, self.status)
        if self.norm:
            out = rt.arena.alloc((ids.numel(), self.width), torch.float32)
            rt.launches += 1
            (ops.layernorm if self.norm == "layer" else ops.rmsnorm)(x, self.norm_w, out, self.eps)
            return out
        return x


@register_part("embedding", "token_table_hashed_pairs")
class TokenTableHashedPairs(Part):
    """x_t = scale * E[id_t, :] + P[r_t, :] with a second table P of ``buckets`` + 1 rows:
    r_t = (id_{t-1} * mul_prev + id_t * mul_cur) mod buckets, and r = buckets for a sequence's first token.
    The token before a step's first one is state of the sequence: one int32 a slot (the id plus one; zero
    means none yet), which the kernel reads and moves on, so a decode step that takes its ids from the
    device needs nothing of the host."""

    def __init__(self, vocab_size: int, width: int, scale: float, buckets: int, mul_prev: int, mul_cur: int):
        self.vocab_size, self.width, self.scale = int(vocab_size), int(width), float(scale)
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        if self.buckets < 1:
            raise ValueError("token_table_hashed_pairs: at least one bucket is needed")
        self.table = self.pairs = None

    def weight_specs(self):
        return [WeightSpec("weight", (self.vocab_size, self.width)),
                WeightSpec("pairs", (self.buckets + 1, self.width))]

    def cache_need(self):
        return StateNeed((1,), "int32")

    def bind(self, tensors, rt):
        self.table = tensors["weight"].contiguous()
        self.pairs = tensors["pairs"].to(self.table.dtype).contiguous()
        self.status = rt.status[0:1]

    def forward_step(self, batch, cache, rt):
        x = rt.arena.alloc((batch.tok_ids.numel(), self.width), torch.float32)
        rt.launches += 1
        ops.embed_pairs(self.table, self.pairs, batch.tok_ids, batch, cache.state, x, self.status, self.scale, self.buckets,
                        self.mul_prev, self.mul_cur)
        return x


@register_part("head", "linear")
class LinearHead(Part):
    """logits = W h, float32 out, no bias; ``tied`` takes the embedding table as W
    (reference: src/model/qwen_model.cpp:189-202, src/model/qwen_tensor_slots.cpp:150-158)."""

    def __init__(self, vocab_size: int, width: int, tied: bool):
        self.vocab_size, self.width, self.tied = int(vocab_size), int(width), bool(tied)
        self.weight = None

    def weight_specs(self):
        return [] if self.tied else [WeightSpec("weight", (self.vocab_size, self.width))]

    def bind(self, tensors, rt):
        self.weight = tensors["weight"].contiguous()

    def forward(self, h, rt):
        logits = torch.empty((h.shape[0], self.vocab_size), dtype=torch.float32, device=rt.device)
        rt.matmul(h, self.weight, logits)
        return logits
