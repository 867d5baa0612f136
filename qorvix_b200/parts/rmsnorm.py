"""RMSNorm: out = (x * 1/sqrt(mean(x^2) + eps)) * w, no bias, no 1+w
(reference: runtime/src/ops.cpp:8-13).  The residual sum that precedes it is fused in: the
residual stream is float32 and the delta is added in float32 in the same pass."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Norm, PreNormed
from .registry import register_part


class RMSNorm(Norm):
    def __init__(self, spec, source, rt):
        self.eps = float(spec.eps)
        self.size = int(spec.size)
        self.weight = source.get(spec.weight, dtype=torch.float32)   # tiny; always read as float32
        self.rt = rt

    folds_into_products = True         # x * rsqrt(mean(x^2) + eps) * weight

    def scale_weight(self):
        return self.weight

    def add_norm(self, residual, delta, rows=None):
        """residual[T,d] float32 (+= delta in place when rows is None).  rows: int32 row
        indices; then only those rows are normed and the residual is left as it is."""
        if isinstance(delta, PreNormed):
            delta = None                    # the product is in the stream already
        n = residual.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), device=residual.device, dtype=self.rt.dtype)
        ops.add_rmsnorm(out, residual, delta, self.weight, self.eps, row_idx=rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)
