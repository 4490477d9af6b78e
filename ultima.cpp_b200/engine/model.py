"""A model built from its description: parts made, weights bound, and the forward pass of
one step over the run list."""
from __future__ import annotations

import os
import sys

import torch

# ULTIMA_TRACE=1: a line for every run of a layer with the sum of the residual stream behind it, in
# the form of the reference's trace ("name-layer = {n} sum = ...", src/model/qwen_block.cpp:29-42),
# so that two runs (32-bit and bfloat16, or two ways of cutting a prompt) can be compared line by line.
TRACE = os.environ.get("ULTIMA_TRACE", "") not in ("", "0")


def _trace(name: str, index: int, x: torch.Tensor) -> None:
    print(f"{name}-{index} = {{{x.numel()}}} sum = {x.double().sum().item():.6f}", file=sys.stderr, flush=True)

from ..parts.base import KVNeed, ModelSpec, StateNeed, build_part


class BuiltLayer:
    """A layer's arrangement and its parts, built and bound; a part is reached by its role
    (``layer.mixer``, ``layer.parts["mixer"]``)."""

    def __init__(self, arrangement, parts: dict):
        self.arrangement, self.parts = arrangement, dict(parts)
        for role, p in parts.items():
            setattr(self, role, p)
        holders = [(role, p) for role, p in parts.items()
                   if getattr(p, "cache_need", None) is not None and p.cache_need() is not None]
        if len(holders) > 1 and not getattr(arrangement, "shares_cache", False):
            raise ValueError("a layer of this arrangement may hold one part that keeps a cache; this one has "
                             + ", ".join(f"{p.family} '{p.kind}'" for _, p in holders))
        self.cache_holder = holders[0][1] if holders else None
        # several holders (an arrangement that says ``shares_cache``): the run's need is all of theirs in the order of the
        # roles, and ``cache_of`` hands a part its share
        self._needs = {role: (n if isinstance(n, tuple) else (n,)) for role, p in holders for n in (p.cache_need(),)}
        if sum(isinstance(n, KVNeed) for ns in self._needs.values() for n in ns) > 1:
            raise ValueError("a layer may keep one set of keys and values")

    def cache_need(self):
        if len(self._needs) <= 1:
            return self.cache_holder.cache_need() if self.cache_holder is not None else None
        return tuple(n for ns in self._needs.values() for n in ns)

    def cache_of(self, role: str, cache):
        """The part of the run's cache that belongs to the part in ``role`` (None if it keeps nothing)."""
        mine = self._needs.get(role)
        if cache is None or mine is None:
            return None
        if len(self._needs) == 1:
            return cache
        before = 0
        for r, ns in self._needs.items():
            if r == role:
                break
            before += sum(isinstance(n, StateNeed) for n in ns)
        states = tuple(cache.states[before:before + sum(isinstance(n, StateNeed) for n in mine)])
        kv = cache.kv if any(isinstance(n, KVNeed) for n in mine) else None
        return type(cache)(kv=kv, state=states[0] if states else None, owner=cache.owner, states=states)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts.values())


class Model:
    def __init__(self, spec: ModelSpec, tensors: dict, rt):
        """tensors: full tensor name -> tensor on the runtime's device, already in their
        storage types."""
        self.spec, self.rt = spec, rt

        def bound(family, ps, prefix):
            p = build_part(family, ps)
            p.bind({s.name: tensors[spec.stored_name(prefix + s.name)] for s in p.weight_specs()}, rt)
            return p

        self.embedding = bound("embedding", spec.embedding, spec.embedding_name)
        self.layers = []
        for L in spec.layers:
            arrangement = build_part("arrangement", L.arrangement)
            parts = {role: bound(family, L.part(role), L.name_of(role)) for role, family in L.roles().items()}
            self.layers.append(BuiltLayer(arrangement, parts))
        self.entries = [bound("entry", ps, prefix) for ps, prefix in spec.entries]
        self.final_norm = bound("norm", spec.final_norm, spec.final_norm_name)
        self.head = build_part("head", spec.head)
        if spec.head.get("tied"):
            self.head.bind({"weight": self.embedding.table}, rt)
        else:
            self.head.bind({s.name: tensors[spec.stored_name(spec.head_name + s.name)]
                            for s in self.head.weight_specs()}, rt)
        for r in spec.runs:
            if not (0 <= r.layer < len(self.layers)):
                raise ValueError(f"run list names layer {r.layer}; the model has {len(self.layers)}")
            if r.entry is not None and not (0 <= r.entry < len(self.entries)):
                raise ValueError(f"run list names entry {r.entry}; the model has {len(self.entries)}")
        self._keeps_embedding = any(self.entries[r.entry].needs_embedding_output for r in spec.runs if r.entry is not None)
        # an embedding that keeps per-sequence state gets a place in the cache behind the runs'
        need = getattr(self.embedding, "cache_need", None)
        self._embedding_need = need() if need is not None else None
        self._stack = None            # see _stack_plan
        self.tap = None               # a callable (run index, residual stream): called behind every run (for comparisons)

    def all_parts(self) -> list:
        return [self.embedding, self.final_norm, self.head] + self.entries + [p for L in self.layers for p in L.parts.values()]

    @property
    def graph_safe(self) -> bool:
        return all(L.graph_safe for L in self.layers) and all(e.graph_safe for e in self.entries)

    def cache_needs(self):
        """For each run of the run list, what its layer asks of the cache; behind them, what the embedding
        asks (an embedding with state of its own: the entry with index ``len(runs)``)."""
        needs = [self.layers[r.layer].cache_need() for r in self.spec.runs]
        if self._embedding_need is not None:
            needs.append(self._embedding_need)
        return needs

    def cache_sources(self):
        return [r.cache_from for r in self.spec.runs] + ([None] if self._embedding_need is not None else [])

    def _stack_plan(self, cache):
        """The plan that runs all layers of a decode step as one resident kernel, if this model's layers
        are of the kinds that kernel takes (kernels/decode_stack.py); None otherwise."""
        if self._stack is None:
            from ..kernels import decode_stack
            self._stack = decode_stack.StackPlan(self, self.rt, cache) if not TRACE and \
                decode_stack.StackPlan.fits(self, self.rt, cache) else False
        return self._stack or None

    def forward(self, batch, cache) -> torch.Tensor:
        """Logits (float32 [wanted rows, vocabulary]) of one step; the cache is read and
        extended in place."""
        rt = self.rt
        rt.arena.reset(0)
        rt.pass_id += 1
        if self._embedding_need is not None:
            x = self.embedding.forward_step(batch, cache.run_cache(len(self.spec.runs), batch.tables), rt)
        else:
            x = self.embedding.forward(batch.tok_ids, rt)
        if TRACE:
            _trace("embd", 0, x)
        S = int(self.spec.streams or 0)
        if S > 0:
            # the stream in S copies, all equal to the embedding's output; layers take [S, T, width]
            from ..kernels import ops
            copies = rt.arena.alloc((S,) + tuple(x.shape), x.dtype)
            rt.launches += 1
            ops.streams_fill(x, copies)
            x = copies
        x0 = None
        if self._keeps_embedding:
            x0 = rt.arena.alloc(tuple(x.shape), x.dtype)
            x0.copy_(x)
        plan = self._stack_plan(cache) if (batch.max_new == 1 and batch.n_tokens <= 64 and S == 0) else None
        if plan is not None:
            plan.run(x, batch)                    # one token a sequence: the whole stack in one kernel
        else:
            for i, r in enumerate(self.spec.runs):
                layer = self.layers[r.layer]
                if r.entry is not None:
                    self.entries[r.entry].forward(x, x0, rt)
                layer.arrangement.run(layer, x, batch, cache.run_cache(i, batch.tables), rt)
                if TRACE:
                    _trace("l_out", i, x)
                if self.tap is not None:
                    self.tap(i, x if S == 0 else x.sum(0))
        if batch.want_rows.numel() == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=rt.device)
        if S > 0:
            # the copies are summed where the final norm reads them, at the wanted rows only
            from ..kernels import ops
            h = rt.arena.alloc((batch.want_rows.numel(), self.spec.width), rt.dtype)
            rt.launches += 1
            ops.streams_pass(x, read=(None, self.final_norm.weight, self.final_norm.eps), out=h, rows=batch.want_rows)
            return self.head.forward(h, rt)
        h = self.final_norm.forward(x, rt, rows=batch.want_rows)
        return self.head.forward(h, rt)
