"""The arrangement of a layer's parts around the residual stream.

Parity: src/llmserve/model/llama.py:131-135 — ``x += mixer(norm(x)); x += ff(norm(x))``.
The residual stream is a 32-bit tensor that the norms update in place: each part returns its
contribution, and the next norm adds it before normalising (one pass over the row instead of
three).  In bfloat16 the last product of a part adds into the stream itself (see ``ops.ResidualSink``): a
small step's product also hands the stream on already normalised for the next norm, so a decode step has
no norm launches of its own; a large step's product leaves a norm kernel that only reads the stream.
"""

from __future__ import annotations

from .. import ops
from .base import Block, FeedForward, Mixer, Norm, register_part


class PreNormBlock(Block):
    roles = {"mixer_norm": "norm", "mixer": "mixer", "ff_norm": "norm", "feed_forward": "feed_forward"}

    def __init__(self, mixer_norm: Norm, mixer: Mixer, ff_norm: Norm, feed_forward: FeedForward):
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.ff_norm = ff_norm
        self.feed_forward = feed_forward

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward))

    def forward(self, resid, pending, ctx, cache, next_norm=None):
        x = self._normed(self.mixer_norm, resid, pending, self.mixer)
        sink = self._sink(self.mixer, self.ff_norm, resid, ctx)
        pending = self.mixer.forward(x, ctx, cache, sink=sink) if sink else self.mixer.forward(x, ctx, cache)
        x = self._normed(self.ff_norm, resid, pending, self.feed_forward)
        sink = self._sink(self.feed_forward, next_norm, resid, ctx)
        return self.feed_forward.forward(x, ctx, sink=sink) if sink else self.feed_forward.forward(x, ctx)

    @staticmethod
    def _normed(norm, resid, pending, consumer):
        """``pending`` is a contribution still to be added, or the stream already summed and
        normalised for ``norm`` by the part before (a fused decode kernel did both).  A consumer
        that does not say it takes the factored form gets a plain tensor."""
        if isinstance(pending, ops.NormedInput):
            if pending.norm is not norm:
                raise RuntimeError("a part handed the residual stream on normalised for another norm")
            return pending if getattr(consumer, "accepts_sink", False) else pending.materialize()
        if pending is ops.ADDED:  # the part's last product added its result to the stream itself
            pending = None
        return norm.add_forward(resid, pending)

    @staticmethod
    def _sink(part, norm, resid, ctx):
        """A sink for the part's last product, if the part takes one and another norm follows (the last part of the
        last layer keeps its contribution: only the rows whose logits are wanted are summed).  Where that norm is an
        RMS norm its weight goes along, so that a small step's product can hand the stream on normalised."""
        if norm is None or not getattr(part, "accepts_sink", False):
            return None
        if not ops.ResidualSink.usable(ctx.num_tokens, getattr(norm, "out_dtype", None)):
            return None
        fused = getattr(norm, "fused_params", None)
        weight, eps = fused() if fused is not None else (None, 0.0)
        return ops.ResidualSink(resid, weight, eps, norm)


register_part("block", "pre_norm", PreNormBlock)
