"""The routed feed-forward: a mixture of small gated feed-forwards of which a token uses a few."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..kernels import ops
from ..weights.spec import WeightSpec
from .base import FeedForward, build_part, part, register_part


@dataclass
class RoutePlan:
    """Where a step's (token, choice) rows lie once they are sorted by expert, all on the device: ``tiles`` int32
    [max_tiles, 4] (expert, first sorted row, rows, -), ``n_tiles`` int32 [1], ``src_rows`` int32 [rows]: the token
    behind a sorted row.  ``gather``: the product reads its rows through ``src_rows`` (else they were copied)."""
    tiles: torch.Tensor
    n_tiles: torch.Tensor
    src_rows: torch.Tensor
    max_tiles: int
    n_rows: int
    gather: bool = True
    tile: int = ops.ROUTE_TILE           # the most rows a tile has


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    """``n_experts`` feed-forwards down(silu(gate h) * (up h)) of inner size ``inner`` (no biases), of which a token uses
    ``top``.  The router: z = W_r h in float32 over n_experts + ``n_identity`` outputs, s = softmax(z); the choice
    scores are s + correction (a stored vector); with ``groups`` = (count, keep) the outputs form ``count`` equal
    groups of neighbours, a group's score is its largest choice score, and only outputs of the ``keep`` best groups can
    be chosen (the others count as -inf); the ``top`` largest choice scores are chosen and weighted with their s, not
    renormalised.  The last ``n_identity`` outputs are identity experts: they hand the input on, scaled by the choice's weight, and
    have no tensors.  ``shared_inner``: one more gated feed-forward that every token uses, added unweighted.

    Other routers and experts of the same family, each a parameter:
      score="sigmoid"        s = sigmoid(z), every output on its own, instead of the softmax
      group_score="top2_sum" a group's score is the sum of its two largest choice scores instead of the largest
      normalise=True         the chosen outputs' weights are divided by their sum (+ 1e-20)
      weight_scale           a constant on the weights (behind the normalisation)
      expert="relu_squared"  an expert (and the shared one) is down(max(up h, 0)^2): no gate matrix

    On the GPU: the router's product with float32 sums (CUDA cores and float32 weights; in a bfloat16 run the stored
    bfloat16 weights on the tensor cores, whose products of two bfloat16 numbers are exact); one kernel picks and counts, one lays
    out the experts' segments and tiles, one hands every (token, choice) its sorted row; the experts' gate/up and
    down products are two grouped products over the sorted rows (stacked weights [experts, 2 inner, width] and
    [experts, width, inner]); one kernel adds the weighted rows into the stream in the order of the choices.  In
    bfloat16 the grouped products run on the tensor cores (tcgen05, tiles of 16 to 128 rows by the rows an expert
    gets on average), for which one more kernel copies the tokens' rows into the sorted order; in float32, and with
    sizes the tensor maps do not take, on the CUDA cores, which read the rows through the list.  Nothing is read on
    the host, so a step can be captured."""

    graph_safe = True

    def __init__(self, width: int, inner: int, n_experts: int, top: int, n_identity: int = 0, groups: tuple | None = None,
                 shared_inner: int | None = None, correction: bool = True, score: str = "softmax", group_score: str = "max",
                 normalise: bool = False, weight_scale: float = 1.0, expert: str = "gated_silu"):
        self.width, self.inner, self.ne, self.top = int(width), int(inner), int(n_experts), int(top)
        self.ni = int(n_identity or 0)
        self.n_out = self.ne + self.ni
        self.groups = (int(groups[0]), int(groups[1])) if groups else (1, 1)
        self.correction = bool(correction)
        if self.top > self.n_out or self.n_out % self.groups[0] or not (1 <= self.groups[1] <= self.groups[0]):
            raise ValueError("routed_experts: top must not exceed the router's outputs, which divide into equal groups")
        if self.n_out > 1024 or self.ne < 1:
            raise ValueError("routed_experts: the router kernel takes up to 1,024 outputs, at least one of them an expert")
        if score not in ("softmax", "sigmoid") or group_score not in ("max", "top2_sum") or expert not in ("gated_silu", "relu_squared"):
            raise ValueError("routed_experts: score is 'softmax' or 'sigmoid', group_score 'max' or 'top2_sum', expert "
                             "'gated_silu' or 'relu_squared'")
        self.mode = ((ops.ROUTE_SIGMOID if score == "sigmoid" else 0) | (ops.ROUTE_GROUP_TOP2 if group_score == "top2_sum" else 0)
                     | (ops.ROUTE_NORMALISE if normalise else 0))
        self.weight_scale, self.gated = float(weight_scale), expert == "gated_silu"
        if not self.gated and self.ni:
            raise ValueError("routed_experts: identity experts go with gated experts")
        shared = part("gated_silu", width=self.width, inner=int(shared_inner or 0)) if self.gated else \
            part("plain_mlp", width=self.width, inner=int(shared_inner or 0), activation="relu_squared")
        self.shared = build_part("feed_forward", shared) if shared_inner else None

    def weight_specs(self):
        W = WeightSpec
        s = [W("router.weight", (self.n_out, self.width), "matrix", ("normal", 0.3))]
        if self.correction:
            s.append(W("correction", (self.n_out,), "vector", ("normal", 0.05)))
        for e in range(self.ne):
            if self.gated:
                s.append(W(f"experts.{e}.gate_proj.weight", (self.inner, self.width)))
            s += [W(f"experts.{e}.up_proj.weight", (self.inner, self.width)),
                  W(f"experts.{e}.down_proj.weight", (self.width, self.inner))]
        if self.shared is not None:
            s += [W("shared." + w.name, w.shape, w.kind, w.init) for w in self.shared.weight_specs()]
        return s

    def kernel_needs(self, run_dtype):
        out = [("routed.cu", ())]
        if not self.gated:
            out.append(("rowwise.cu", ()))
        if run_dtype == torch.bfloat16:
            out.append(("gemm_tcgen05.cu", ()))
        return out

    def bind(self, tensors, rt):
        # the router's sums are 32-bit.  Stored bfloat16 weights against the bfloat16 rounding of the input give exact
        # products, so that pair may go to the tensor cores, which add them up in float32; anything else runs on the
        # CUDA cores with float32 weights
        wr = tensors["router.weight"]
        self.w_router = wr.contiguous() if (wr.dtype == torch.bfloat16 and rt.dtype == torch.bfloat16 and self.width % 8 == 0) \
            else wr.float().contiguous()
        self.corr = tensors["correction"].float().contiguous() if self.correction else None
        g0 = tensors["experts.0.up_proj.weight"]
        rows = 2 * self.inner if self.gated else self.inner          # [gate ; up] or up alone
        self.w_gu = torch.empty((self.ne, rows, self.width), dtype=g0.dtype, device=g0.device)
        self.w_down = torch.empty((self.ne, self.width, self.inner), dtype=g0.dtype, device=g0.device)
        for e in range(self.ne):
            if self.gated:
                self.w_gu[e, :self.inner] = tensors[f"experts.{e}.gate_proj.weight"]
            self.w_gu[e, rows - self.inner:] = tensors[f"experts.{e}.up_proj.weight"]
            self.w_down[e] = tensors[f"experts.{e}.down_proj.weight"]
        if self.shared is not None:
            self.shared.bind({w.name: tensors["shared." + w.name] for w in self.shared.weight_specs()}, rt)
        # the one-block routing kernel keeps sixteen warps' work space and the experts' counters in 48 KB of shared memory
        self._small_fits = 16 * (2 * self.n_out + self.groups[0]) * 4 + (4 * self.ne + 1) * 4 <= 48 * 1024
        # counters of the routing kernels, shared by the model's routed layers (one runs at a time): rows of every
        # expert, hand-out cursors, first sorted row of every expert, number of tiles
        self.ws = rt.shared(("routed_counters", self.ne), lambda: torch.zeros(3 * self.ne + 4, dtype=torch.int32, device=rt.device))

    def forward(self, h, residual, batch, rt):
        T, ne, top = h.shape[0], self.ne, self.top
        i32, f32 = torch.int32, torch.float32
        z = rt.matmul_parts(h, self.w_router)          # few tokens: K in slices, summed by the routing kernel
        if z is None:
            z = rt.arena.alloc((T, self.n_out), f32)
            rt.matmul(h, self.w_router, z)
        idx = rt.arena.alloc((T, top), i32)
        wts = rt.arena.alloc((T, top), f32)
        row_pos = rt.arena.alloc((T, top), i32)
        src_rows = rt.arena.alloc((T * top,), i32)
        act = rt.arena.alloc((T * top, self.inner), rt.dtype)
        y = rt.arena.alloc((T * top, self.width), f32)
        if self.gated:
            w_gate, w_up = self.w_gu[:, :self.inner], self.w_gu[:, self.inner:]
            first = (w_gate, act, ops.EPI_SWIGLU, w_up)
        else:
            first = (self.w_gu, act, ops.EPI_STORE, None)          # the squared rectifier in the up product's epilogue
        unary = 0 if self.gated else ops.UNARY_RELU_SQUARED
        # the tensor-core products take both or neither: their tiles are cut to the rows an expert gets on average
        fast = (rt.grouped_on_tensor_cores(h, first[0], first[1], first[2], first[3])
                and rt.grouped_on_tensor_cores(act, self.w_down, y))
        tile = ops.ROUTE_TILE
        if fast:
            from ..kernels import gemm_tc
            tile = gemm_tc.row_tile(T * top, ne)
        max_tiles = min(T * top, -(-T * top // tile) + ne)
        tiles = rt.arena.alloc((max_tiles, 4), i32)
        counts, cursor, seg_start, n_tiles = self.ws[:ne], self.ws[ne:2 * ne], self.ws[2 * ne:3 * ne], self.ws[3 * ne:3 * ne + 1]
        if T <= ops.ROUTE_SMALL_TOKENS and self._small_fits:
            rt.launches += 1                  # few tokens: the three steps as one launch of one block
            ops.route_small(z, self.corr, ne, top, self.groups[0], self.groups[1], idx, wts, tiles, n_tiles, row_pos, src_rows, tile,
                            mode=self.mode, wscale=self.weight_scale)
        else:
            rt.launches += 3
            ops.route(z, self.corr, ne, top, self.groups[0], self.groups[1], idx, wts, counts, mode=self.mode, wscale=self.weight_scale)
            ops.route_plan(counts, cursor, seg_start, tiles, n_tiles, ne, tile)
            ops.route_scatter(idx, seg_start, cursor, row_pos, src_rows, ne)
        plan = RoutePlan(tiles, n_tiles, src_rows, max_tiles, T * top, tile=tile)
        if fast:
            rows = rt.arena.alloc((T * top, self.width), rt.dtype)
            rt.launches += 1
            ops.route_gather(h, row_pos, rows)
            plan.gather = False
            rt.matmul_grouped(rows, first[0], first[1], plan, first[2], w2=first[3], unary=unary)
        else:
            rt.matmul_grouped(h, first[0], first[1], plan, first[2], w2=first[3], unary=unary)
        plan.gather = False
        rt.matmul_grouped(act, self.w_down, y, plan)
        rt.launches += 1
        ops.route_combine(y, h, row_pos, wts, residual)
        if self.shared is not None:
            self.shared.forward(h, residual, batch, rt)
