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
from .graph import DecodeGraph


class StepFunction:
    def __init__(self, model: Model, cache: CacheManager, use_graphs: bool | None = None):
        """``use_graphs``: replay decode-only steps as CUDA graphs (default: on a CUDA device,
        when every part of the model says it can be captured)."""
        self.model = model
        self.cache = cache
        self.h2d_bytes = 0  # bytes of the last step's descriptor copy
        self.last_context: StepContext | None = None
        if use_graphs is None:
            use_graphs = cache.device.type == "cuda" and model.graph_safe
        self.use_graphs = bool(use_graphs)
        self.graphs: dict[int, DecodeGraph] = {}
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
        if self.use_graphs and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            return self._replay(pairs, [e.tokens[0] for e in entries], lengths, state_slots, group_arrays)
        ctx, group_tensors, self.h2d_bytes = pack_step(entries, lengths, state_slots, group_arrays, cache.device)
        views = cache.views(group_tensors, ctx.state_slots, ctx.host_state_slots)
        logits = self.model.forward(ctx, views)
        cache.commit(pairs)
        self.last_context = ctx
        return logits

    def _replay(self, pairs, tokens, lengths, state_slots, group_arrays) -> torch.Tensor:
        cache = self.cache
        graph = self.graphs.get(len(pairs))
        if graph is None:
            graph = self.graphs[len(pairs)] = DecodeGraph(self.model, cache, len(pairs))
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
        return self._replay(pairs, device_tokens, lengths, state_slots, group_arrays)
