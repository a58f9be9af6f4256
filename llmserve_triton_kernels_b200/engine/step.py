"""The step function: one batch of (request, its next tokens) through the model, from the cache.

It runs only the tokens it is given, as one batch — portions of prompts beside single decoded
tokens, cut anywhere — and returns the logits at the wanted places.  The reference's
counterpart is ``ContinuousBatchingEngine._forward`` (src/llmserve/scheduler/engine.py:236-246)
over ``PagedKVCache.build_batch`` (src/llmserve/kvcache/paged.py:174-218), which advances the
lengths before the forward pass; here pages are reserved first and lengths advance only after
the pass has been issued.
"""

from __future__ import annotations

import torch

from ..cache import CacheManager
from ..models.model import Model
from .batch import StepContext, StepEntry, pack_step
from .graph import StepGraph


class StepFunction:
    # Shapes other than decode steps are captured the second time they are seen; so many of them are kept.
    MAX_SHAPE_GRAPHS = 24
    # A step of more tokens than this is not captured: its kernels are long, the host keeps ahead of them anyway.
    MAX_GRAPH_TOKENS = 8192

    def __init__(self, model: Model, cache: CacheManager, use_graphs: bool | None = None):
        """``use_graphs``: replay steps whose shape has been seen before as CUDA graphs (default: on a CUDA
        device, when every part of the model says it can be captured)."""
        self.model = model
        self.cache = cache
        self.h2d_bytes = 0  # bytes of the last step's descriptor copy
        self.last_context: StepContext | None = None
        if use_graphs is None:
            use_graphs = cache.device.type == "cuda" and model.graph_safe
        self.use_graphs = bool(use_graphs)
        self.graphs: dict[int, StepGraph] = {}  # decode steps, by their number of requests
        self.shape_graphs: dict[tuple, StepGraph] = {}  # other shapes, least recently used first
        self._seen_shapes: dict[tuple, int] = {}
        self.graph_pool = None  # the memory pool that this step function's graphs share (that of the first one captured)
        self.last_was_graph = False  # the last step replayed a graph

    def __call__(self, entries: list[StepEntry]) -> torch.Tensor:
        """Returns 32-bit logits ``[wanted places, vocab]`` on the device, in the order of the
        entries and of each entry's ``want``.  The tensor may be a buffer that the next call
        overwrites: read or copy it before stepping again."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        cache, limit = self.cache, self.model.plan.max_positions
        vocab = self.model.plan.vocab_size
        pairs = []
        for e in entries:
            if not cache.has_request(e.request):
                cache.add_request(e.request)
            if not e.tokens:
                raise ValueError(f"request {e.request!r} brings no tokens")
            if cache.lengths[e.request] + len(e.tokens) > limit:
                raise ValueError(
                    f"request {e.request!r} would hold {cache.lengths[e.request] + len(e.tokens)} tokens, "
                    f"beyond the model's {limit} positions"
                )
            if min(e.tokens) < 0 or max(e.tokens) >= vocab:
                raise ValueError(f"request {e.request!r} has a token id outside [0, {vocab})")
            pairs.append((e.request, len(e.tokens)))
        cache.reserve(pairs)
        group_arrays, state_slots = cache.step_tables(pairs)
        lengths = [cache.lengths[req] for req, _ in pairs]
        self.last_was_graph = False
        if self.use_graphs:
            graph = self._graph_for(entries)
            if graph is not None:
                tokens = [t for e in entries for t in e.tokens]
                return self._replay(graph, pairs, tokens, lengths, state_slots, group_arrays)
        ctx, group_tensors, self.h2d_bytes = pack_step(entries, lengths, state_slots, group_arrays, cache.device)
        views = cache.views(group_tensors, ctx.state_slots, ctx.host_state_slots)
        logits = self.model.forward(ctx, views)
        cache.commit(pairs)
        self.last_context = ctx
        return logits

    def _decode_graph(self, requests: int) -> StepGraph:
        graph = self.graphs.get(requests)
        if graph is None:
            graph = self.graphs[requests] = StepGraph(self.model, self.cache, (1,) * requests, ((0,),) * requests, owner=self)
        return graph

    def _graph_for(self, entries: list[StepEntry]) -> StepGraph | None:
        """The graph of this step's shape, or None if the step runs kernel by kernel (a shape seen for the first
        time, or too large to be worth it)."""
        if all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            return self._decode_graph(len(entries))
        if sum(len(e.tokens) for e in entries) > self.MAX_GRAPH_TOKENS:
            return None
        shape = tuple((len(e.tokens), tuple(e.want)) for e in entries)
        graph = self.shape_graphs.pop(shape, None)
        if graph is None:
            seen = self._seen_shapes[shape] = self._seen_shapes.get(shape, 0) + 1
            if len(self._seen_shapes) > 4096:
                self._seen_shapes.clear()
            if seen < 2:
                return None
            graph = StepGraph(self.model, self.cache, tuple(n for n, _ in shape), tuple(w for _, w in shape), owner=self)
            while len(self.shape_graphs) >= self.MAX_SHAPE_GRAPHS:
                self.shape_graphs.pop(next(iter(self.shape_graphs)))
        self.shape_graphs[shape] = graph  # most recently used last
        return graph

    def _replay(self, graph: StepGraph, pairs, tokens, lengths, state_slots, group_arrays) -> torch.Tensor:
        cache = self.cache
        graph.fill(tokens, lengths, state_slots, group_arrays)
        logits = graph.run()
        cache.commit(pairs)
        self.h2d_bytes, self.last_context, self.last_was_graph = graph.h2d_bytes, graph.ctx, True
        return logits

    def decode_ahead(self, requests: list, device_tokens: torch.Tensor) -> torch.Tensor:
        """One decode step (one token per request, its logits wanted) whose token ids are not on the host yet:
        ``device_tokens`` (int32 ``[len(requests)]``, in the order of ``requests``) holds what the step before chose.
        The requests must be live and have room for one more token.  Where decode steps replay a graph the host
        never reads the tokens here; elsewhere this is an ordinary step on tokens read from the tensor."""
        if not self.use_graphs:  # no graphs (a model that cannot be captured, or the CPU under test): the plain way
            return self([StepEntry(r, [int(t)], [0]) for r, t in zip(requests, device_tokens.tolist())])
        cache, limit = self.cache, self.model.plan.max_positions
        for r in requests:
            if cache.lengths[r] + 1 > limit:
                raise ValueError(f"request {r!r} would hold {cache.lengths[r] + 1} tokens, beyond the model's {limit} positions")
        pairs = [(r, 1) for r in requests]
        cache.reserve(pairs)
        group_arrays, state_slots = cache.step_tables(pairs)
        lengths = [cache.lengths[r] for r in requests]
        return self._replay(self._decode_graph(len(pairs)), pairs, device_tokens, lengths, state_slots, group_arrays)
