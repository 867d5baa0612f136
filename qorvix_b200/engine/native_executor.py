"""The native step executor behind the Python step function.

When every block of a model is a pre-norm block of RMS norm, rotary grouped-query attention over
its own paged cache and SwiGLU (the arrangement of the reference's decoder,
runtime/src/text_model.cpp:146-168), a step's whole forward pass is issued by C++
(csrc/host/executor.hpp): one call a step instead of a dozen a layer, with the same kernels and the
same choices the part objects make.  Anything else (another mixer, feed-forward, norm, position
encoding or arrangement, a layer run twice, a layer that reads another's cache) keeps the part-by-part
path: `try_build` returns None.  QORVIX_NATIVE_EXECUTOR=0 switches it off (for comparison and tests).
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_longlong, c_void_p
from typing import Optional

import torch

from ..csrc import ops
from ..csrc.build import load_library, write_manifest


class _Linear(Structure):
    _fields_ = [("rows", c_void_p), ("packed", c_void_p), ("N", c_int), ("K", c_int), ("dt", c_int), ("pad", c_int)]


class _Layer(Structure):
    _fields_ = [("norm1", c_void_p), ("norm2", c_void_p), ("qkv", _Linear), ("o", _Linear), ("gate_up", _Linear), ("down", _Linear),
                ("cache", c_void_p), ("cache_pages", c_longlong), ("interleaved", c_int), ("window", c_int)]


class _Model(Structure):
    _fields_ = [(n, c_int) for n in ("dt", "d", "H", "Hkv", "hd", "f", "V", "page", "rot", "table_rows", "sms", "emb_dt", "n_layers", "pad")] + [
        ("eps", c_float), ("scale", c_float), ("cos_sin", c_void_p), ("embedding", c_void_p), ("final_norm", c_void_p), ("head", _Linear),
        ("layers", POINTER(_Layer))]


class _Step(Structure):
    _fields_ = [(n, c_int) for n in ("T", "S", "R", "n1", "max_q_len", "max_ctx_len", "rest_max_q", "captured", "max_blocks", "portion_max_ctx")] + [
        (n, c_void_p) for n in ("token_ids", "tok_pos", "tok_seg", "seg_q_start", "seg_pos0", "block_table", "want_rows", "logits")]


ROUTES = ("attention_prefill_tc", "gemm_qkv_rope", "attention_decode_bf16", "attention_prefill_bf16", "attention_generic", "gemm_bf16_norm")
_lib = None


def lib():
    global _lib
    if _lib is None:
        L = load_library("executor")
        L.qvx_last_error.restype = c_char_p
        L.qvx_create.restype, L.qvx_create.argtypes = c_void_p, [c_char_p, POINTER(_Model), c_void_p]
        L.qvx_destroy.restype, L.qvx_destroy.argtypes = None, [c_void_p]
        L.qvx_workspace_bytes.restype, L.qvx_workspace_bytes.argtypes = c_longlong, [c_void_p, c_int, c_int, c_int]
        L.qvx_forward.restype, L.qvx_forward.argtypes = c_longlong, [c_void_p, POINTER(_Step), c_void_p, c_longlong, c_void_p]
        L.qvx_route_count.restype, L.qvx_route_count.argtypes = c_longlong, [c_int]
        _lib = L
    return _lib


def route_counts() -> dict:
    """How often the kernels that a step's shape chooses between have served steps of the native
    executor in this process (0 for all when it was never loaded)."""
    if _lib is None:
        return {n: 0 for n in ROUTES}
    return {n: int(_lib.qvx_route_count(i)) for i, n in enumerate(ROUTES)}


def enabled() -> bool:
    return os.environ.get("QORVIX_NATIVE_EXECUTOR", "1") != "0"


def _linear(lin) -> _Linear:
    w = lin.weight
    return _Linear(rows=w.data_ptr() if w is not None else None, packed=lin.packed.data_ptr() if lin.packed is not None else None,
                   N=lin.out_features, K=lin.in_features, dt=ops.dt_code(w.dtype) if w is not None else ops.BF16, pad=0)


class NativeExecutor:
    def __init__(self, handle, keep, rt, vocab, group):
        self._h, self._keep, self.rt, self.vocab, self.group = handle, keep, rt, vocab, group

    def __del__(self):
        if getattr(self, "_h", None) and _lib is not None:
            _lib.qvx_destroy(self._h)
            self._h = None

    @staticmethod
    def try_build(model, cache) -> Optional["NativeExecutor"]:
        """The executor for `model` (a models.text_model.TextModel) over `cache`, or None when the model
        is not made of the blocks it knows."""
        from ..parts.attention import Attention
        from ..parts.block import PreNormBlock
        from ..parts.mlp import SwiGLU
        from ..parts.rmsnorm import RMSNorm
        from ..parts.rotary import RotaryEmbedding
        if not enabled() or model.order != list(range(len(model.blocks))) or type(model.final_norm) is not RMSNorm:
            return None
        rt = model.rt
        layers, keep, group, table = [], [], None, None
        for run, b in enumerate(model.blocks):
            if type(b) is not PreNormBlock or type(b.mixer) is not Attention or type(b.feed_forward) is not SwiGLU:
                return None
            if type(b.mixer_norm) is not RMSNorm or type(b.ffn_norm) is not RMSNorm or type(b.mixer.position) is not RotaryEmbedding:
                return None
            m, f = b.mixer, b.feed_forward
            if m.spec.kv_from is not None or b.mixer_norm.eps != model.final_norm.eps or b.ffn_norm.eps != model.final_norm.eps:
                return None
            view = cache.layer_view(run)
            if view.kind != "paged" or (group is not None and view.group != group):
                return None
            group = view.group
            first = model.blocks[0].mixer
            if (m.H, m.Hkv, m.hd, m.scale) != (first.H, first.Hkv, first.hd, first.scale) or f.f != model.blocks[0].feed_forward.f:
                return None
            if table is None:
                table = m.position.cos_sin
            elif m.position.cos_sin.data_ptr() != table.data_ptr() and not torch.equal(m.position.cos_sin, table):
                return None
            layers.append(_Layer(norm1=b.mixer_norm.weight.data_ptr(), norm2=b.ffn_norm.weight.data_ptr(), qkv=_linear(m.qkv_proj),
                                 o=_linear(m.o_proj), gate_up=_linear(f.gate_up), down=_linear(f.down), cache=view.tensor.data_ptr(),
                                 cache_pages=view.tensor.shape[0], interleaved=1 if f.interleaved else 0, window=m.window))
            keep.append(view.tensor)
        if not layers:
            return None
        first = model.blocks[0].mixer
        arr = (_Layer * len(layers))(*layers)
        # the products' workspace is registered with their library here: whole steps never pass through ops' wrappers
        err = (ops._gemm_buffers if rt.dtype == torch.bfloat16 else ops._tc_buffers)(rt.device)["err"]
        desc = _Model(dt=ops.dt_code(rt.dtype), d=model.spec.hidden_size, H=first.H, Hkv=first.Hkv, hd=first.hd, f=model.blocks[0].feed_forward.f,
                      V=model.spec.vocab_size, page=cache.page_size, rot=first.position.rotary_dim, table_rows=table.shape[0], sms=ops.sm_count(),
                      emb_dt=ops.dt_code(model.embedding.dtype), n_layers=len(layers), pad=0, eps=model.final_norm.eps, scale=first.scale,
                      cos_sin=table.data_ptr(), embedding=model.embedding.data_ptr(), final_norm=model.final_norm.weight.data_ptr(),
                      head=_linear(model.lm_head), layers=arr)
        L = lib()
        # the decode kernel's bounded waits report into the same word as everything else
        alib = ops._lib("attention_bf16")
        if not getattr(alib, "_qv_err_set", False):
            alib.qv_attn_set_error_word(err.data_ptr())
            alib._qv_err_set = True
        h = L.qvx_create(str(write_manifest()).encode(), ctypes.byref(desc), err.data_ptr())
        if not h:
            raise ops.KernelError(f"the native executor could not be made: {L.qvx_last_error().decode()}")
        keep += [arr, table, err, model]
        return NativeExecutor(h, keep, rt, model.spec.vocab_size, group)

    def forward(self, ctx) -> Optional[torch.Tensor]:
        """Runs the tokens of `ctx`; float32 logits [wanted rows, vocab], or None when none is wanted."""
        T, S, R = ctx.num_tokens, ctx.num_segments, ctx.num_wanted
        n1 = 0
        while n1 < S and ctx.seg_len[n1] == 1:
            n1 += 1
        rest = max(ctx.seg_len[n1:], default=0)
        deep = max((p0 + n for p0, n in zip(ctx.seg_start_pos, ctx.seg_len) if n > 1), default=0)
        bt = ctx.block_tables[self.group]
        logits = torch.empty((R, self.vocab), device=self.rt.device, dtype=torch.float32) if R else None
        nbytes = _lib.qvx_workspace_bytes(self._h, T, R, n1)
        ws = torch.empty(nbytes, device=self.rt.device, dtype=torch.uint8)
        step = _Step(T=T, S=S, R=R, n1=n1, max_q_len=ctx.max_q_len, max_ctx_len=ctx.max_ctx_len, rest_max_q=rest,
                     captured=1 if ctx.captured else 0, max_blocks=bt.shape[-1], portion_max_ctx=deep, token_ids=ctx.token_ids.data_ptr(),
                     tok_pos=ctx.tok_pos.data_ptr(), tok_seg=ctx.tok_seg.data_ptr(), seg_q_start=ctx.seg_q_start.data_ptr(),
                     seg_pos0=ctx.seg_pos0.data_ptr(), block_table=bt.data_ptr(), want_rows=ctx.want_rows.data_ptr() if R else None,
                     logits=logits.data_ptr() if R else None)
        n = _lib.qvx_forward(self._h, ctypes.byref(step), ws.data_ptr(), nbytes, ops._stream())
        if n < 0:
            raise ops.KernelError(_lib.qvx_last_error().decode())
        ops.add_launches(int(n))
        return logits
