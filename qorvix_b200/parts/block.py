"""Block arrangements.  'pre_norm' is the reference's (runtime/src/text_model.cpp:146-168):
    x += mixer(norm(x));  x += feed_forward(norm(x))
The residual stream is float32.  A block hands the feed-forward's output on as a pending
delta, which the next norm adds in its own pass."""
from __future__ import annotations

from ..csrc import ops
from .base import Block, PreNormed
from .registry import build_part, register_part


class PreNormBlock(Block):
    def __init__(self, spec, source, rt):
        self.mixer_norm = build_part("norm", spec.mixer_norm, source, rt)
        self.mixer = build_part("mixer", spec.mixer, source, rt)
        self.ffn_norm = build_part("norm", spec.ffn_norm, source, rt)
        self.feed_forward = build_part("feed_forward", spec.feed_forward, source, rt)

    def forward(self, residual, pending, ctx, cache):
        # Few tokens: a part that folds norms (folds_norms) is told which norm (one that folds into products) reads the stream
        # after it; it may then add its output to the stream in its last product's epilogue and hand
        # on that norm's half-done input (a PreNormed) instead of a delta, and the part after the norm
        # finishes the norm in its first product.  Anything else takes the norm kernel.
        fold = ops.folded_norm_enabled(residual.shape[0])
        after = getattr(ctx, "next_norm", None)            # the norm the block after this one starts with
        if self.mixer is not None:
            x = self._normed(self.mixer_norm, self.mixer, residual, pending)
            if fold and getattr(self.mixer, "folds_norms", False):
                nxt = self.ffn_norm if self.feed_forward is not None else after
                pending = self.mixer.forward(x, ctx, cache, residual=residual, next_norm=nxt if _folds(nxt) else None)
            else:
                pending = self.mixer.forward(x, ctx, cache)
        if self.feed_forward is not None:
            x = self._normed(self.ffn_norm, self.feed_forward, residual, pending)
            if fold and getattr(self.feed_forward, "folds_norms", False):
                pending = self.feed_forward.forward(x, ctx, residual=residual, next_norm=after if _folds(after) else None)
            else:
                pending = self.feed_forward.forward(x, ctx)
        return residual, pending

    @staticmethod
    def _normed(norm, part, residual, pending):
        """The input of `part`: the PreNormed as it is when it was made for this norm and the part takes
        one, else the normed rows."""
        if isinstance(pending, PreNormed) and pending.norm is norm and getattr(part, "folds_norms", False):
            return pending
        return norm.add_norm(residual, pending)

    def first_norm(self):
        """The norm this block reads the stream with first (what the block ahead may prepare for)."""
        if self.mixer is not None:
            return self.mixer_norm
        return self.ffn_norm if self.feed_forward is not None else None


def _folds(norm) -> bool:
    """Whether a norm lets the products around it take over its passes (see parts/base.py)."""
    return norm is not None and getattr(norm, "folds_into_products", False)


register_part("block", "pre_norm", PreNormBlock)
