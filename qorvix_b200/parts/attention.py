"""Causal grouped-query attention over the paged cache (reference: runtime/src/text_model.cpp:78-116,
146-158).  q, k and v come from one fused projection; the rotation of q and k and the
write of k and v into the request's pages are one kernel; attention reads keys and values
from the pages only, so a prompt portion and a single decoded token take the same path.
"""
from __future__ import annotations

import torch

from ..cache.spec import PagedKVSpec
from ..csrc import ops
from .base import Mixer, PreNormed
from .linear import Linear
from .registry import build_part, register_part


class Attention(Mixer):
    def __init__(self, spec, source, rt):
        self.spec = spec
        self.rt = rt
        self.H, self.Hkv, self.hd = spec.num_heads, spec.num_kv_heads, spec.head_dim
        if self.H % self.Hkv:
            raise ValueError(f"num_heads {self.H} is not a multiple of num_kv_heads {self.Hkv}")
        mats = [source.get(spec.q_proj)]
        if spec.kv_from is None:
            mats += [source.get(spec.k_proj), source.get(spec.v_proj)]
        dt = torch.float32 if any(m.dtype == torch.float32 for m in mats) else mats[0].dtype
        self.qkv_proj = Linear(torch.cat([m.to(dt) for m in mats], dim=0))
        del mats
        self.o_proj = Linear(source.get(spec.o_proj))
        self.position = build_part("position", spec.position, source, rt)
        self.window = int(spec.window)
        self.scale = float(spec.scale)

    def cache_spec(self):
        if self.spec.kv_from is not None:
            return None
        return PagedKVSpec(self.Hkv, self.hd, self.window)

    def reads_cache_of(self):
        return self.spec.kv_from

    folds_norms = True             # forward() takes a PreNormed x, residual= and next_norm=

    def forward(self, x, ctx, cache, residual=None, next_norm=None):
        """x: the normed rows [T, d], or a PreNormed (few tokens: the norm's scale is then applied to the
        projection's sums).  With residual and next_norm the output projection adds the output to the
        stream itself and the PreNormed input of next_norm is returned instead of the output."""
        H, Hkv, hd = self.H, self.Hkv, self.hd
        own_kv = self.spec.kv_from is None
        table = self.position.table() if self.position is not None else None
        bt = ctx.block_tables[cache.group]
        qkv = None
        if isinstance(x, PreNormed):
            qkv = torch.empty((x.scaled.shape[0], self.qkv_proj.out_features), device=x.scaled.device, dtype=self.rt.dtype)
            if self.qkv_proj.forward_prenormed(x, qkv):
                self._rotate_and_write(qkv, ctx, cache, table, bt)
            else:
                qkv, x = None, x.materialise()
        if qkv is None:
            T = x.shape[0]
            if (own_kv and table is not None and self.rt.dtype == torch.bfloat16 and self.qkv_proj.packed is not None
                    and ops.fused_rope_enabled(T)):
                # rotation and cache write in the projection's epilogue, where the kernel takes the sizes
                qkv = torch.empty((T, (H + 2 * Hkv) * hd), device=x.device, dtype=self.rt.dtype)
                if not ops.gemm_qkv_rope(qkv, x, self.qkv_proj.packed, cache.tensor, table, ctx.tok_pos, ctx.tok_seg, bt,
                                         H, Hkv, hd, cache.page_size):
                    qkv = None
            if qkv is None:
                qkv = self.qkv_proj(x, out_dtype=self.rt.dtype)             # [T, (H+2Hkv)*hd] or [T, H*hd]
                self._rotate_and_write(qkv, ctx, cache, table, bt)
        out = torch.empty((qkv.shape[0], H * hd), device=qkv.device, dtype=self.rt.dtype)
        ops.attention(out, qkv[:, : H * hd], cache.tensor, ctx, bt, H, Hkv, hd, cache.page_size,
                      self.window, self.scale)
        if residual is not None and next_norm is not None:
            pre = self.o_proj.forward_to_stream(out, residual, next_norm)
            if pre is not None:
                return pre
        return self.o_proj(out, out_dtype=self.rt.dtype)

    def _rotate_and_write(self, qkv, ctx, cache, table, bt):
        """Rotates q and k in place and writes k and v into the request's pages (own cache), or rotates q only."""
        H, Hkv, hd = self.H, self.Hkv, self.hd
        if self.spec.kv_from is None:
            if table is not None:
                ops.rope_kv_write(qkv, cache.tensor, table, ctx.tok_pos, ctx.tok_seg, bt, H, Hkv, hd,
                                  table.shape[1] * 2, cache.page_size)
            else:
                if self.position is not None:
                    self.position.apply(qkv, ctx, H, Hkv, hd)
                ops.rope_kv_write(qkv, cache.tensor, None, ctx.tok_pos, ctx.tok_seg, bt,
                                  H, Hkv, hd, 0, cache.page_size)
        elif self.position is not None:
            self.position.apply(qkv, ctx, H, 0, hd)


register_part("mixer", "attention", Attention)
