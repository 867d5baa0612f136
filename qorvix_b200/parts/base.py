"""The interfaces parts have, and the runtime they are built with.

Mixer         forward(x[T,d], ctx, cache) -> [T,d] in the compute dtype; cache_spec() says what
              it keeps per request (cache.spec.PagedKVSpec / FixedStateSpec / None);
              reads_cache_of() names another layer whose cache it reads instead.
FeedForward   forward(x[T,d], ctx) -> [T,d].
              A mixer or feed-forward with the attribute folds_norms = True also takes x as a
              PreNormed and the keywords residual=<float32 stream>, next_norm=<the RMS norm that reads
              the stream next>; it may then add its output to the stream itself and return a
              PreNormed for that norm (few tokens: the norm's two passes over the stream ride in the
              epilogues of the products around it).
Norm          add_norm(residual, delta, rows=None): residual (float32) += delta (delta may be None), returns
              the normed rows in the compute dtype; with rows (int32 row indices) only those rows of
              residual + delta are normed and the residual is left as it is.  The sum and the norm
              are computed in float32.
              A norm that is  x * rsqrt(mean(x^2) + eps) * w  for some per-feature w may declare
              folds_into_products = True and give size, eps and scale_weight() (w as float32): parts
              that fold norms then take its two passes over the stream into the epilogues of the
              products around it.  Nothing else about the norm is assumed.
Position      table() -> float32 [positions, rotary_dim/2, 2] of (cos, sin) if it is a rotation
              the attention kernels can fuse, else None; apply(qkv, ctx, H, Hkv, hd) rotates q and k
              in place for mixers that do not fuse it.
Block         forward(residual, pending, ctx, cache) -> (residual, pending): `pending` is a
              delta not yet added to the residual stream, so that the next norm adds it in
              the same pass.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class Runtime:
    """What parts need to know about where they run."""
    device: torch.device
    dtype: torch.dtype                 # compute dtype: torch.bfloat16 or torch.float32
    max_positions: int                 # rows of position tables
    page_size: int = 16

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, device=self.device, dtype=dtype or self.dtype)


@dataclass
class PreNormed:
    """The input of a folding norm as the product ahead of it left it: `scaled` is the float32 residual
    stream times the norm's weight (compute dtype, not yet divided by the root mean square) and
    `stats` what the producing kernel left of the stream's squares; only the kernels that produce and
    consume it (Linear.forward_to_stream / forward_prenormed) know its layout.  The residual stream
    already holds the product, so nothing is pending.  A consumer either hands it to a Linear, which
    scales the sums of its own product by rsqrt(mean of squares + eps), or calls materialise() for the
    normed rows."""
    scaled: torch.Tensor
    stats: object
    norm: object
    residual: torch.Tensor

    def materialise(self) -> torch.Tensor:
        return self.norm.add_norm(self.residual, None)


class Mixer:
    def cache_spec(self):
        return None

    def reads_cache_of(self) -> Optional[int]:
        return None

    def forward(self, x, ctx, cache):
        raise NotImplementedError


class FeedForward:
    def forward(self, x, ctx):
        raise NotImplementedError


class Norm:
    folds_into_products = False        # True: see the module's header; needs size, eps, scale_weight()

    def add_norm(self, residual, delta, rows=None):
        raise NotImplementedError

    def scale_weight(self):
        raise NotImplementedError


class PositionEncoding:
    def table(self):
        return None

    def apply(self, qkv, ctx, num_heads, num_kv_heads, head_dim):
        raise NotImplementedError


class Block:
    def forward(self, residual, pending, ctx, cache):
        raise NotImplementedError
