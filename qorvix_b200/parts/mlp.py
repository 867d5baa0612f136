"""SwiGLU feed-forward: down(silu(gate x) * up x), dense, no bias
(reference: runtime/src/text_model.cpp:162-168, runtime/src/ops.cpp:96-100).  gate and up
are one fused projection."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, PreNormed
from .linear import Linear
from .registry import register_part


class SwiGLU(FeedForward):
    def __init__(self, spec, source, rt):
        self.rt = rt
        self.f = int(spec.intermediate_size)
        g, u = source.get(spec.gate_proj), source.get(spec.up_proj)
        dt = torch.float32 if (g.dtype == torch.float32 or u.dtype == torch.float32) else g.dtype
        # When the width allows, gate and up rows are interleaved in groups of 16 (16 gate rows, the 16
        # up rows of the same features, ...), so that one tile of the product holds both halves of a
        # feature and the activation is applied in the product's epilogue.
        self.interleaved = self.f % 16 == 0
        if self.interleaved:
            k = g.shape[1]
            fused = torch.stack([g.to(dt).view(self.f // 16, 16, k), u.to(dt).view(self.f // 16, 16, k)], dim=1)
            self.gate_up = Linear(fused.reshape(2 * self.f, k))
            del fused
        else:
            self.gate_up = Linear(torch.cat([g.to(dt), u.to(dt)], dim=0))
        del g, u
        self.down = Linear(source.get(spec.down_proj))

    folds_norms = True             # forward() takes a PreNormed x, residual= and next_norm=

    def forward(self, x, ctx, residual=None, next_norm=None):
        """x: the normed rows [T, d], or a PreNormed (few tokens: the norm's scale is then applied to the
        gate/up sums before the activation).  With residual and next_norm the down projection adds the
        output to the stream itself and the PreNormed input of next_norm is returned instead."""
        act = None
        if isinstance(x, PreNormed):
            act = torch.empty((x.scaled.shape[0], self.f), device=x.scaled.device, dtype=self.rt.dtype)
            if not (self.interleaved and self.gate_up.forward_prenormed(x, act, swiglu=True)):
                act, x = None, x.materialise()
        if act is None:
            act = torch.empty((x.shape[0], self.f), device=x.device, dtype=self.rt.dtype)
            if self.interleaved:
                ops.gemm_swiglu(act, x, self.gate_up.weight, self.gate_up.packed, self.gate_up.out_features)
            else:
                gu = self.gate_up(x, out_dtype=self.rt.dtype)
                ops.swiglu(act, gu)
        if residual is not None and next_norm is not None:
            pre = self.down.forward_to_stream(act, residual, next_norm)
            if pre is not None:
                return pre
        return self.down(act, out_dtype=self.rt.dtype)


register_part("feed_forward", "swiglu", SwiGLU)
