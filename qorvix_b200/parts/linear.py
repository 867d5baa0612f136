"""y = x W^T, the one matrix product every projection uses.  The kernel is chosen by the
weight's dtype and the shape: float32 weights run on the CUDA cores in true float32;
bfloat16 weights run on the tensor-core kernels where the shape allows, else on the same
CUDA-core kernel with float32 accumulation.  All of them are kernels of this package.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import PreNormed


class Linear:
    def __init__(self, weight: torch.Tensor, keep_rows: bool = False):
        assert weight.dim() == 2
        self.weight = weight.contiguous()
        self.out_features, self.in_features = weight.shape
        # A bfloat16 matrix is stored as the 16 KB tiles the MMA consumes (128 rows x 64 k in its
        # swizzled shared-memory layout), which HBM and an SM's copy engine deliver faster than
        # rows; the rows are then dropped (keep_rows, or QORVIX_KEEP_ROWS=1, keeps them, for tests
        # that compare the two layouts).
        self.packed = None
        if (self.weight.is_cuda and self.weight.dtype == torch.bfloat16 and self.in_features % 8 == 0
                and ops.packed_weights_enabled()):
            try:
                self.packed = ops.pack_weight(self.weight)
            except torch.cuda.OutOfMemoryError:
                self.packed = None          # no room for the tiles beside the rows: the rows serve
            if self.packed is not None and not (keep_rows or _keep_rows()):
                self.weight = None

    def forward(self, x: torch.Tensor, out: torch.Tensor = None, out_dtype: torch.dtype = None) -> torch.Tensor:
        M = x.shape[0]
        if out is None:
            out = torch.empty((M, self.out_features), device=x.device, dtype=out_dtype or x.dtype)
        if M == 0:
            return out
        ops.gemm(out, x, self.weight, self.packed, self.out_features)
        return out

    __call__ = forward

    def forward_prenormed(self, pre, out: torch.Tensor, swiglu: bool = False) -> bool:
        """out = rmsnorm(stream) W^T from a PreNormed (the root mean square applied to the product's
        sums); False, nothing written, when the kernel does not take the product."""
        if self.packed is None:
            return False
        return ops.gemm_bf16_norm(out, pre.scaled, self.packed, self.out_features, swiglu=swiglu, ssq_in=pre.stats,
                                  stream_width=pre.norm.size, eps=pre.norm.eps)

    def forward_to_stream(self, x: torch.Tensor, residual: torch.Tensor, norm):
        """residual += x W^T in the product's epilogue; returns the PreNormed input of `norm` (one that
        declares folds_into_products), or None, nothing written, when the kernel does not take the product."""
        M, N = x.shape[0], self.out_features
        if (self.packed is None or M > 64 or x.dtype != torch.bfloat16 or residual.dtype != torch.float32
                or tuple(residual.shape) != (M, N) or residual.stride(1) != 1 or norm.size != N):
            return None
        scaled = torch.empty((M, N), device=x.device, dtype=x.dtype)
        stats = ops.new_norm_stats(N, x.device)
        if not ops.gemm_bf16_norm(scaled, x, self.packed, N, residual=residual, norm_weight=norm.scale_weight(), ssq_out=stats):
            return None
        return PreNormed(scaled=scaled, stats=stats, norm=norm, residual=residual)


def _keep_rows() -> bool:
    import os
    return os.environ.get("QORVIX_KEEP_ROWS", "0") == "1"
