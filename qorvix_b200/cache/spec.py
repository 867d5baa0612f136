"""What a layer asks of the cache manager.  A mixer returns one of these (or None when it
keeps nothing, or reads another layer's cache); layers with equal needs share a group."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple


@dataclass(frozen=True)
class PagedKVSpec:
    """Keys and values of every token, in pages.  window > 0: only the last `window`
    positions are ever read again, so pages that lie wholly before them are given back."""
    num_kv_heads: int
    head_dim: int
    window: int = 0

    def elems_per_token(self) -> int:
        return 2 * self.num_kv_heads * self.head_dim


@dataclass(frozen=True)
class FixedStateSpec:
    """A state of fixed size per request (a recurrent state, a convolution tail, ...):
    one slot per live request, zeroed when the request is admitted."""
    shape: Tuple[int, ...]
    dtype: str = "float32"
