"""A decoder assembled from a ModelSpec: embedding, blocks in the spec's order, final norm,
output head.  It knows nothing of any one architecture; the counterpart of the
reference's TextModel::forwardFromState (runtime/src/text_model.cpp:133-176) for a batch of
tokens from several requests.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..csrc import ops
from ..parts.base import Runtime
from ..parts.linear import Linear
from ..parts.registry import build_part


class TextModel:
    def __init__(self, spec, source, rt: Runtime):
        self.spec = spec
        self.rt = rt
        source.check(spec.expected_shapes(), optional=spec.optional_tensors, ignored=getattr(spec, "ignored_tensors", ()))
        self.embedding = source.get(spec.embedding)
        self.blocks = [build_part("block", _BlockView(layer), source, rt) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, source, rt)
        self.lm_head = Linear(source.get(spec.lm_head)) if spec.lm_head is not None else Linear(self.embedding)
        self.order: List[int] = list(spec.order)
        self._native = None            # the native executor of this model over a cache, made on first use (False: not applicable)

    def cache_needs(self):
        """What each RUN of the execution order wants of the cache manager: (cache spec or None, index
        of the run whose cache it reads or None).  A layer that the order names twice keeps a cache per
        run: in a later step its first run must find the keys its first run wrote, not its second's.
        A mixer that reads another layer's cache reads that layer's latest run before its own."""
        needs = []
        last_run_of = {}
        for run, li in enumerate(self.order):
            m = getattr(self.blocks[li], "mixer", None)
            spec = m.cache_spec() if m is not None else None
            src = m.reads_cache_of() if m is not None else None
            src_run = None
            if src is not None:
                if src not in last_run_of:
                    raise ValueError(f"layer {li} reads the cache of layer {src}, which has not run before it")
                src_run = last_run_of[src]
            needs.append((spec, src_run))
            last_run_of[li] = run
        return needs

    def forward(self, ctx, cache) -> Optional[torch.Tensor]:
        """Runs the tokens of `ctx`; returns float32 logits [wanted rows, vocab] (None if none wanted)."""
        T = ctx.num_tokens
        if self._native is None:
            from ..engine.native_executor import NativeExecutor
            self._native = NativeExecutor.try_build(self, cache) or False
        if self._native:
            # every block is one the native executor knows: the whole step in one call
            return self._native.forward(ctx)
        residual = torch.empty((T, self.spec.hidden_size), device=self.rt.device, dtype=torch.float32)
        ops.embed(residual, self.embedding, ctx.token_ids)
        pending = None
        for run, li in enumerate(self.order):
            # which norm reads the stream after this block (a block that can prepares that norm's input);
            # none after the last block: the final norm gathers the wanted rows
            nxt = self.blocks[self.order[run + 1]] if run + 1 < len(self.order) else None
            ctx.next_norm = nxt.first_norm() if hasattr(nxt, "first_norm") else None
            residual, pending = self.blocks[li].forward(residual, pending, ctx, cache.layer_view(run))
        if ctx.num_wanted == 0:
            return None
        h = self.final_norm.add_norm(residual, pending, rows=ctx.want_rows)
        return self.lm_head(h, out_dtype=torch.float32)


class _BlockView:
    """Lets a LayerSpec be built through the block registry: its `kind` is the arrangement."""

    def __init__(self, layer):
        self.kind = layer.block
        self.mixer, self.feed_forward = layer.mixer, layer.feed_forward
        self.mixer_norm, self.ffn_norm = layer.mixer_norm, layer.ffn_norm
