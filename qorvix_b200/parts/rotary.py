"""Rotary position encoding with optional llama3 frequency scaling.

Base frequencies f_i = theta^(-2i/rotary_dim) and the split-half pairing are the
reference's (runtime/src/ops.cpp:127-148).  The llama3 scaling is not in the reference (it
parses the keys for display only, gguf/src/gguf_file.cpp:233-243); it follows the published
rule: wavelengths shorter than orig/high keep f, longer than orig/low use f/factor, those
between blend linearly.  Angles pos*f are formed in float64 on the host and their cosine and
sine stored as a float32 table [positions, rotary_dim/2, 2], so the kernels do no
trigonometry and a position's rotation is the same in every step.
"""
from __future__ import annotations

import math

import torch

from ..csrc import ops
from .base import PositionEncoding
from .registry import register_part


def inverse_frequencies(rotary_dim: int, theta: float, scaling=None) -> torch.Tensor:
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    f = torch.exp(-(2.0 * i / rotary_dim) * math.log(theta))
    if scaling is None:
        return f
    orig = float(scaling.original_max_position_embeddings)
    low, high, factor = float(scaling.low_freq_factor), float(scaling.high_freq_factor), float(scaling.factor)
    wavelen = 2.0 * math.pi / f
    smooth = (orig / wavelen - low) / (high - low) if high != low else torch.ones_like(f)
    blended = (1.0 - smooth) * f / factor + smooth * f
    out = torch.where(wavelen < orig / high, f, torch.where(wavelen > orig / low, f / factor, blended))
    return out


class RotaryEmbedding(PositionEncoding):
    def __init__(self, spec, source, rt):
        self.rotary_dim = int(spec.rotary_dim)
        self.head_dim = int(spec.head_dim)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        self.inv_freq = inverse_frequencies(self.rotary_dim, float(spec.theta), spec.scaling)
        pos = torch.arange(rt.max_positions, dtype=torch.float64)
        ang = pos[:, None] * self.inv_freq[None, :]
        self.cos_sin = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).to(torch.float32).contiguous().to(rt.device)

    def table(self):
        return self.cos_sin

    def apply(self, qkv, ctx, num_heads, num_kv_heads, head_dim):
        ops.rope_kv_write(qkv, None, self.cos_sin, ctx.tok_pos, ctx.tok_seg, ctx.any_block_table(),
                          num_heads, num_kv_heads, head_dim, self.rotary_dim, 1)


register_part("position", "rotary", RotaryEmbedding)
