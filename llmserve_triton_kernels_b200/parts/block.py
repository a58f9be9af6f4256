"""The arrangement of a layer's parts around the residual stream.

Parity: src/llmserve/model/llama.py:131-135 — ``x += mixer(norm(x)); x += ff(norm(x))``.
The residual stream is a 32-bit tensor that the norms update in place: each part returns its
contribution, and the next norm adds it before normalising (one pass over the row instead of
three).
"""

from __future__ import annotations

from .base import Block, FeedForward, Mixer, Norm, register_part


class PreNormBlock(Block):
    def __init__(self, mixer_norm: Norm, mixer: Mixer, ff_norm: Norm, feed_forward: FeedForward):
        self.mixer_norm = mixer_norm
        self.mixer = mixer
        self.ff_norm = ff_norm
        self.feed_forward = feed_forward

    @property
    def graph_safe(self) -> bool:
        return all(p.graph_safe for p in (self.mixer_norm, self.mixer, self.ff_norm, self.feed_forward))

    def forward(self, resid, pending, ctx, cache):
        x = self.mixer_norm.add_forward(resid, pending)
        pending = self.mixer.forward(x, ctx, cache)
        x = self.ff_norm.add_forward(resid, pending)
        return self.feed_forward.forward(x, ctx)


register_part("block", "pre_norm", PreNormBlock)
