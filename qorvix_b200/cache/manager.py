"""The cache manager: pages of keys and values with a block table per request, one pool per
group of layers with the same needs, and slots of fixed-size state per request.

The reference's GlobalKvCache (memory/src/kv_cache.cpp) pages one layer at a time on the
CPU in float32 and its GPU model keeps a dense slab per session
(cuda/src/cuda_backend.cu:1329-1331).  Here a page id covers all layers of its group:
the group's tensor is [layers, pages + 1, 2, kv_heads, page_size, head_dim] (K then V; a
(page, kv head) tile of keys is contiguous), the extra last page being scratch that padded
rows of a captured step may write to.  Pages go back to the pool when a request ends and,
for a group with a window, as soon as the window has passed them; freed pages are handed
out again at once.  Reservation is all-or-nothing over all groups and happens before a step
is built, so running out of pages is the caller's decision to handle, never a fault inside
a step (the reference breaks out of its grow loop and then writes through a null slot,
runtime/src/text_model.cpp:138-140).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from .page_pool import PageError, PagePool
from .spec import FixedStateSpec, PagedKVSpec


class OutOfPages(RuntimeError):
    pass


class OutOfSlots(RuntimeError):
    pass


_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class LayerCacheView:
    """What a mixer gets for its layer: the layer's slice of its group's tensor."""
    kind: str                      # "paged" | "state" | "none"
    group: int = -1
    tensor: Optional[torch.Tensor] = None
    page_size: int = 0


@dataclass
class _Group:
    spec: object
    layers: List[int]
    pool: Optional[PagePool] = None
    tensor: Optional[torch.Tensor] = None


@dataclass
class _Request:
    slot: int
    length: int = 0
    tables: Dict[int, List[int]] = field(default_factory=dict)     # group -> page id per block (-1: given back)
    admitted_at: int = 0


class CacheManager:
    def __init__(self, needs: Sequence[Tuple[object, Optional[int]]], max_tokens: int, page_size: int,
                 max_requests: int, device="cuda", dtype=torch.bfloat16, allocate: bool = True):
        """needs[i] = (cache spec or None, index of the layer whose cache layer i reads or None).
        max_tokens: how many tokens (each request rounded up to whole pages) fit at once."""
        if page_size <= 0 or page_size % 16:
            raise ValueError(f"page_size {page_size} must be a positive multiple of 16")
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.num_pages = max(1, -(-int(max_tokens) // self.page_size))
        self.device = torch.device(device)
        self.dtype = dtype
        self.groups: List[_Group] = []
        self._layer_group: List[int] = [-1] * len(needs)
        self._layer_index: List[int] = [-1] * len(needs)
        by_spec: Dict[Hashable, int] = {}
        for li, (spec, _) in enumerate(needs):
            if spec is None:
                continue
            if spec not in by_spec:
                by_spec[spec] = len(self.groups)
                self.groups.append(_Group(spec=spec, layers=[]))
            g = by_spec[spec]
            self._layer_group[li] = g
            self._layer_index[li] = len(self.groups[g].layers)
            self.groups[g].layers.append(li)
        self._reads_from = [src for _, src in needs]
        for li, src in enumerate(self._reads_from):
            if src is not None and (not 0 <= src < len(needs) or needs[src][0] is None):
                raise ValueError(f"layer {li} reads the cache of layer {src}, which keeps none")
        for g in self.groups:
            if isinstance(g.spec, PagedKVSpec):
                g.pool = PagePool(self.num_pages)
                if allocate:
                    g.tensor = torch.zeros((len(g.layers), self.num_pages + 1, 2, g.spec.num_kv_heads,
                                            self.page_size, g.spec.head_dim), device=self.device, dtype=dtype)
            elif isinstance(g.spec, FixedStateSpec):
                if allocate:
                    # one more slot than requests: the last is scratch for padded rows of a captured step
                    g.tensor = torch.zeros((len(g.layers), self.max_requests + 1, *g.spec.shape),
                                           device=self.device, dtype=_DTYPES.get(g.spec.dtype, g.spec.dtype))
            else:
                raise TypeError(f"unknown cache spec {g.spec!r}")
        self._free_slots: List[int] = list(range(self.max_requests - 1, -1, -1))
        self._requests: Dict[Hashable, _Request] = {}
        self._clock = 0

    # ------------------------------------------------------------------ queries
    @property
    def scratch_page(self) -> int:
        return self.num_pages

    @property
    def scratch_slot(self) -> int:
        return self.max_requests

    def paged_groups(self) -> List[int]:
        return [i for i, g in enumerate(self.groups) if g.pool is not None]

    def free_pages(self, group: int = None) -> int:
        pools = [g.pool for g in self.groups if g.pool is not None] if group is None else [self.groups[group].pool]
        return min((p.num_free for p in pools), default=self.num_pages)

    def free_slots(self) -> int:
        return len(self._free_slots)

    def has(self, req_id) -> bool:
        return req_id in self._requests

    def length(self, req_id) -> int:
        return self._requests[req_id].length

    def slot(self, req_id) -> int:
        return self._requests[req_id].slot

    def epoch(self, req_id) -> int:
        """A number that differs between two admissions of the same request id."""
        return self._requests[req_id].admitted_at

    def live_requests(self) -> list:
        return list(self._requests)

    def block_table(self, req_id, group: int) -> List[int]:
        return self._requests[req_id].tables[group]

    def pages_needed(self, req_id, n_new: int) -> Dict[int, int]:
        """Pages each paged group must add so that `n_new` more tokens fit (req_id None: a new request)."""
        r = self._requests.get(req_id) if req_id is not None else None
        length = r.length if r else 0
        blocks = -(-(length + n_new) // self.page_size)
        out = {}
        for gi in self.paged_groups():
            have = len(r.tables[gi]) if r else 0
            out[gi] = max(0, blocks - have)
        return out

    def one_more_token_fits(self, req_ids: Sequence[Hashable]) -> int:
        """How many of the given live requests, taken in order, can each hold one more token with
        the pages that are free now.  One pass; the scheduler's check for a round of decoding."""
        free = {gi: self.groups[gi].pool.num_free for gi in self.paged_groups()}
        page = self.page_size
        for n, rid in enumerate(req_ids):
            r = self._requests[rid]
            blocks = r.length // page + 1
            for gi in free:
                if len(r.tables[gi]) < blocks:
                    if free[gi] == 0:
                        return n
                    free[gi] -= 1
        return len(req_ids)

    def can_reserve(self, wants: Sequence[Tuple[Hashable, int]]) -> bool:
        """Whether all (request or None, new tokens) of a step fit together."""
        total: Dict[int, int] = {}
        new_slots = 0
        for req_id, n in wants:
            if req_id is None or req_id not in self._requests:
                new_slots += 1
                req_id = None
            for gi, k in self.pages_needed(req_id, n).items():
                total[gi] = total.get(gi, 0) + k
        if new_slots > len(self._free_slots):
            return False
        return all(k <= self.groups[gi].pool.num_free for gi, k in total.items())

    # ------------------------------------------------------------------ life of a request
    def admit(self, req_id) -> int:
        """Gives the request a slot (its state slots are zeroed); no pages yet."""
        if req_id in self._requests:
            raise ValueError(f"request {req_id!r} is already live")
        if not self._free_slots:
            raise OutOfSlots(f"all {self.max_requests} request slots are taken")
        slot = self._free_slots.pop()
        self._clock += 1
        self._requests[req_id] = _Request(slot=slot, tables={gi: [] for gi in self.paged_groups()},
                                          admitted_at=self._clock)
        for g in self.groups:
            if g.pool is None and g.tensor is not None:
                g.tensor[:, slot].zero_()
        return slot

    def reserve(self, req_id, n_new: int) -> bool:
        """Pages for n_new more tokens in every paged group, or nothing at all."""
        r = self._requests[req_id]
        need = self.pages_needed(req_id, n_new)
        if any(k > self.groups[gi].pool.num_free for gi, k in need.items()):
            return False
        for gi, k in need.items():
            r.tables[gi].extend(self.groups[gi].pool.alloc(k))
        return True

    def commit(self, req_id, n_new: int) -> None:
        """The request now holds n_new more tokens; pages a window has passed are given back."""
        r = self._requests[req_id]
        r.length += n_new
        for gi in self.paged_groups():
            g = self.groups[gi]
            if len(r.tables[gi]) * self.page_size < r.length:
                raise PageError(f"request {req_id!r} holds {r.length} tokens but only {len(r.tables[gi])} pages in group {gi}")
            w = g.spec.window
            if w > 0:
                first_needed = max(0, r.length - w + 1)        # the oldest key a later query reads
                dead_blocks = first_needed // self.page_size
                table = r.tables[gi]
                gone = [p for p in table[:dead_blocks] if p >= 0]
                if gone:
                    g.pool.free(gone)
                    for b in range(dead_blocks):
                        table[b] = -1

    def release(self, req_id) -> None:
        """The request ends: everything it holds goes back."""
        r = self._requests.pop(req_id)
        for gi, table in r.tables.items():
            self.groups[gi].pool.free([p for p in table if p >= 0])
        self._free_slots.append(r.slot)

    def youngest(self, among=None):
        """The most recently admitted live request (the one to preempt first)."""
        ids = [i for i in (among if among is not None else self._requests) if i in self._requests]
        return max(ids, key=lambda i: self._requests[i].admitted_at) if ids else None

    # ------------------------------------------------------------------ what the model sees
    def layer_view(self, layer: int) -> LayerCacheView:
        src = self._reads_from[layer]
        li = src if src is not None else layer
        gi = self._layer_group[li]
        if gi < 0:
            return LayerCacheView(kind="none")
        g = self.groups[gi]
        t = g.tensor[self._layer_index[li]] if g.tensor is not None else None
        if g.pool is not None:
            return LayerCacheView(kind="paged", group=gi, tensor=t, page_size=self.page_size)
        return LayerCacheView(kind="state", group=gi, tensor=t)

    # ------------------------------------------------------------------ checks (tests)
    def check_invariants(self) -> None:
        """No page lost, none held twice, none both free and held."""
        for gi in self.paged_groups():
            pool = self.groups[gi].pool
            seen = {}
            for rid, r in self._requests.items():
                for p in r.tables[gi]:
                    if p < 0:
                        continue
                    if p in seen:
                        raise PageError(f"group {gi}: page {p} is held by {seen[p]!r} and {rid!r}")
                    if not pool.is_held(p):
                        raise PageError(f"group {gi}: page {p} of {rid!r} is on the free list")
                    seen[p] = rid
            if len(seen) != pool.num_held:
                raise PageError(f"group {gi}: {pool.num_held} pages are taken but requests hold {len(seen)}")
            if len(set(pool._free)) != len(pool._free):
                raise PageError(f"group {gi}: a page is on the free list twice")
        slots = [r.slot for r in self._requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise PageError("a request slot is held twice or is both free and held")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise PageError("a request slot was lost")
