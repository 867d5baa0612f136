"""Block arrangements.  'pre_norm' is the reference's (runtime/src/text_model.cpp:146-168):
    x += mixer(norm(x));  x += feed_forward(norm(x))
The residual stream is float32.  A block hands the feed-forward's output on as a pending
delta, which the next norm adds in its own pass."""
from __future__ import annotations

from .base import Block
from .registry import build_part, register_part


class PreNormBlock(Block):
    def __init__(self, spec, source, rt):
        self.mixer_norm = build_part("norm", spec.mixer_norm, source, rt)
        self.mixer = build_part("mixer", spec.mixer, source, rt)
        self.ffn_norm = build_part("norm", spec.ffn_norm, source, rt)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, source, rt)

    def forward(self, residual, pending, ctx, cache):
        if self.mixer is not None:
            h = self.mixer_norm.add_norm(residual, pending)
            pending = self.mixer.forward(h, ctx, cache)
        if self.feed_forward is not None:
            h = self.ffn_norm.add_norm(residual, pending)
            pending = self.feed_forward.forward(h, ctx)
        return residual, pending


register_part("block", "pre_norm", PreNormBlock)
