"""All layers of a decode step as one persistent kernel (csrc/decode_fused.cu).

A fusion above the parts, like the captured graph: it recognises a model whose every layer in
the execution order is the pre-norm arrangement of RMS norm, rotary grouped-query attention
over its own pages and an interleaved SwiGLU feed-forward in bfloat16, and runs those layers
as one launch that streams every weight once and never lets HBM idle between operations (the
reference's decode is ~10 launches per layer, cuda/src/cuda_backend.cu:1380-1440).  Any other
model, size or step takes the parts' own path; `try_build` then returns None.  The fusion is
opt-in (QORVIX_FUSED_DECODE=1): at the sizes measured so far the parts' path, whose kernels
overlap through programmatic dependent launch, is the faster one.

The plan belongs to one captured decode step: it holds pointers to that step's positions,
slots and block tables, and workspaces sized for its rows.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_double, c_longlong, c_void_p
from typing import Optional

import numpy as np
import torch

from ..csrc import ops
from ..csrc.build import load_library
from ..parts.attention import Attention
from ..parts.block import PreNormBlock
from ..parts.mlp import SwiGLU
from ..parts.rmsnorm import RMSNorm
from ..parts.rotary import RotaryEmbedding


class _HostLayer(ctypes.Structure):
    _fields_ = [("w", c_void_p * 4), ("n", c_longlong * 4), ("k", c_longlong * 4), ("norm1", c_void_p),
                ("norm2", c_void_p), ("cache", c_void_p), ("block_table", c_void_p), ("rope", c_void_p),
                ("eps1", c_double), ("eps2", c_double), ("scale", c_double), ("window", c_longlong),
                ("rot", c_longlong), ("rope_rows", c_longlong), ("interleaved", c_longlong)]


class _HostArgs(ctypes.Structure):
    _fields_ = [("layers", c_void_p), ("final_norm", c_void_p), ("resid", c_void_p),
                ("x_norm", c_void_p), ("q_buf", c_void_p), ("attn_out", c_void_p), ("act", c_void_p),
                ("ws", c_void_p * 4), ("attn_partial", c_void_p), ("ssq", c_void_p), ("tok_pos", c_void_p), ("tok_seg", c_void_p),
                ("barrier", c_void_p), ("err", c_void_p),
                ("num_layers", c_longlong), ("M", c_longlong), ("BN", c_longlong), ("d", c_longlong),
                ("H", c_longlong), ("Hkv", c_longlong), ("hd", c_longlong), ("f", c_longlong), ("page", c_longlong),
                ("max_blocks", c_longlong), ("splits", c_longlong), ("final_eps", c_double)]


def _lib():
    L = load_library("decode_fused")
    if not getattr(L, "_qv_typed", False):
        L.qv_fused_workspace_floats.restype = c_longlong
        L.qv_fused_workspace_floats.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.qv_fused_fill_layer.argtypes = [c_void_p, ctypes.POINTER(_HostLayer)]
        L.qv_fused_decode.argtypes = [ctypes.POINTER(_HostArgs), c_void_p]
        L._qv_typed = True
    return L


def enabled() -> bool:
    return os.environ.get("QORVIX_FUSED_DECODE", "0") == "1"


class FusedDecode:
    @staticmethod
    def try_build(model, cache, ctx, rows: int) -> Optional["FusedDecode"]:
        """A plan for `rows` tokens (one per request) of the captured step `ctx`, or None when the
        model, its sizes or the step are not what the kernel takes."""
        if not enabled() or rows > 64 or model.rt.dtype != torch.bfloat16:
            return None
        runs = []
        for run, li in enumerate(model.order):
            b = model.blocks[li]
            if type(b) is not PreNormBlock or type(b.mixer) is not Attention or type(b.feed_forward) is not SwiGLU:
                return None
            if type(b.mixer_norm) is not RMSNorm or type(b.ffn_norm) is not RMSNorm or type(model.final_norm) is not RMSNorm:
                return None
            a, ff = b.mixer, b.feed_forward
            if a.spec.kv_from is not None:
                return None
            if a.position is not None and type(a.position) is not RotaryEmbedding:
                return None
            mats = (a.qkv_proj.weight, a.o_proj.weight, ff.gate_up.weight, ff.down.weight)
            if any(m is None or m.dtype != torch.bfloat16 or m.shape[1] % 8 for m in mats):     # needs the rows
                return None
            view = cache.layer_view(run)
            if view.kind != "paged" or view.tensor is None or view.tensor.dtype != torch.bfloat16:
                return None
            runs.append((b, view))
        if not runs:
            return None
        a0, f0 = runs[0][0].mixer, runs[0][0].feed_forward
        d = model.spec.hidden_size
        for b, _ in runs:
            a, ff = b.mixer, b.feed_forward
            if (a.H, a.Hkv, a.hd, ff.f) != (a0.H, a0.Hkv, a0.hd, f0.f) or a.qkv_proj.in_features != d:
                return None
        if a0.hd % 16 or not 16 <= a0.hd <= 128 or a0.H // a0.Hkv > 16 or d % 8 or f0.f % 8:
            return None
        try:
            return FusedDecode(model, cache, ctx, rows, runs)
        except ops.KernelError:
            return None

    def __init__(self, model, cache, ctx, rows, runs):
        self.lib = _lib()
        dev = model.rt.device
        a0, f0 = runs[0][0].mixer, runs[0][0].feed_forward
        self.M, self.BN = rows, 16 if rows <= 16 else (32 if rows <= 32 else 64)
        self.d, self.H, self.Hkv, self.hd, self.f = model.spec.hidden_size, a0.H, a0.Hkv, a0.hd, f0.f
        self.page = cache.page_size
        BN, bf = self.BN, torch.bfloat16
        self.x_norm = torch.zeros((BN, self.d), device=dev, dtype=bf)
        self.q_buf = torch.zeros((rows, self.H * self.hd), device=dev, dtype=bf)
        self.attn_out = torch.zeros((BN, self.H * self.hd), device=dev, dtype=bf)
        self.act = torch.zeros((BN, self.f), device=dev, dtype=bf)
        grid = self.lib.qv_fused_grid()
        self.splits = max(1, min(32, (grid * 8) // (rows * self.Hkv)))
        self.attn_partial = torch.zeros(rows * self.H * self.splits * (self.hd + 2), device=dev, dtype=torch.float32)
        self.ssq = torch.zeros(rows * (-(-self.d // 128)), device=dev, dtype=torch.float32)
        self.barrier = torch.zeros(1, device=dev, dtype=torch.int32)
        self.err = ops._tc_buffers(dev)["err"]
        # one record per run of the execution order
        rec = self.lib.qv_fused_layer_bytes()
        host = np.zeros(len(runs) * rec, dtype=np.uint8)
        ws_floats = [0, 0, 0, 0]
        self._keep = []
        for i, (b, view) in enumerate(runs):
            a, ff = b.mixer, b.feed_forward
            mats = (a.qkv_proj.weight, a.o_proj.weight, ff.gate_up.weight, ff.down.weight)
            table = a.position.table() if a.position is not None else None
            bt = ctx.block_tables[view.group]
            self.max_blocks = bt.shape[-1]
            h = _HostLayer()
            for j, m in enumerate(mats):
                h.w[j], h.n[j], h.k[j] = m.data_ptr(), m.shape[0], m.shape[1]
                ws_floats[j] = max(ws_floats[j], self.lib.qv_fused_workspace_floats(m.shape[0], m.shape[1], BN))
            h.norm1, h.norm2 = b.mixer_norm.weight.data_ptr(), b.ffn_norm.weight.data_ptr()
            h.cache, h.block_table = view.tensor.data_ptr(), bt.data_ptr()
            h.rope = table.data_ptr() if table is not None else None
            h.eps1, h.eps2, h.scale = b.mixer_norm.eps, b.ffn_norm.eps, a.scale
            h.window = a.window
            h.rot = table.shape[1] * 2 if table is not None else 0
            h.rope_rows = table.shape[0] if table is not None else 0
            h.interleaved = 1 if ff.interleaved else 0
            rc = self.lib.qv_fused_fill_layer(host[i * rec:].ctypes.data, ctypes.byref(h))
            if rc != 0:
                raise ops.KernelError(f"fused decode: layer record refused (code {rc})")
            self._keep.append((mats, table, bt, view.tensor))
        self.layers = torch.from_numpy(host).to(dev)
        self.ws = [torch.zeros(max(1, n), device=dev, dtype=torch.float32) for n in ws_floats]
        self.final_norm = model.final_norm
        args = _HostArgs()
        args.layers = self.layers.data_ptr()
        args.final_norm = self.final_norm.weight.data_ptr()
        args.x_norm, args.q_buf = self.x_norm.data_ptr(), self.q_buf.data_ptr()
        args.attn_out, args.act = self.attn_out.data_ptr(), self.act.data_ptr()
        for j in range(4):
            args.ws[j] = self.ws[j].data_ptr()
        args.attn_partial = self.attn_partial.data_ptr()
        args.ssq = self.ssq.data_ptr()
        args.tok_pos, args.tok_seg = ctx.tok_pos.data_ptr(), ctx.tok_seg.data_ptr()
        args.barrier, args.err = self.barrier.data_ptr(), self.err.data_ptr()
        args.num_layers, args.M, args.BN, args.d = len(runs), rows, BN, self.d
        args.H, args.Hkv, args.hd, args.f, args.page = self.H, self.Hkv, self.hd, self.f, self.page
        args.max_blocks, args.splits, args.final_eps = self.max_blocks, self.splits, self.final_norm.eps
        self.args = args
        self._ctx_keep = (ctx.tok_pos, ctx.tok_seg)

    def run(self, residual: torch.Tensor) -> torch.Tensor:
        """residual [rows, d] float32 holds the embedded tokens; on return it is the residual stream
        after the last layer.  Returns the final norm's output [rows, d] (a view of the plan's buffer)."""
        assert residual.dtype == torch.float32 and residual.is_contiguous() and tuple(residual.shape) == (self.M, self.d)
        self.args.resid = residual.data_ptr()
        rc = self.lib.qv_fused_decode(ctypes.byref(self.args), ops._stream())
        ops._check(rc, "fused_decode")
        return self.x_norm[: self.M]
