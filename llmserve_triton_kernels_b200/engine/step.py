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


class StepFunction:
    def __init__(self, model: Model, cache: CacheManager):
        self.model = model
        self.cache = cache
        self.h2d_bytes = 0  # bytes of the last step's descriptor copy
        self.last_context: StepContext | None = None

    def __call__(self, entries: list[StepEntry]) -> torch.Tensor:
        """Returns 32-bit logits ``[wanted places, vocab]`` on the device, in the order of the
        entries and of each entry's ``want``."""
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
        ctx, group_tensors, self.h2d_bytes = pack_step(entries, lengths, state_slots, group_arrays, cache.device)
        views = cache.views(group_tensors, ctx.state_slots, ctx.host_state_slots)
        logits = self.model.forward(ctx, views)
        cache.commit(pairs)
        self.last_context = ctx
        return logits
