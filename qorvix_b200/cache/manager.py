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

The bookkeeping (free lists, block tables, slots, reservation, window release, invariants)
is C++ (csrc/host_runtime.cpp); this class owns the device tensors and maps request ids of
any hashable type to the integers the C++ side uses.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from . import native
from .spec import FixedStateSpec, PagedKVSpec



class PageError(RuntimeError):
    """The bookkeeping of pages is inconsistent (a page lost, held twice or freed twice)."""

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


class _PoolView:
    """Read-only view of one paged group's pool in the native manager."""

    def __init__(self, manager, paged_index: int):
        self._m, self._g = manager, paged_index

    @property
    def num_pages(self) -> int:
        return self._m.num_pages

    @property
    def num_free(self) -> int:
        return self._m._lib.qvh_free_pages(self._m._h, self._g)

    @property
    def num_held(self) -> int:
        return self._m._lib.qvh_held_pages(self._m._h, self._g)


@dataclass
class _Group:
    spec: object
    layers: List[int]
    pool: Optional[_PoolView] = None
    tensor: Optional[torch.Tensor] = None


class CacheManager:
    def __init__(self, needs: Sequence[Tuple[object, Optional[int]]], max_tokens: int, page_size: int,
                 max_requests: int, device="cuda", dtype=torch.bfloat16, allocate: bool = True):
        """needs[i] = (cache spec or None, index of the run whose cache run i reads or None).
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
        # the native side knows only the paged groups, numbered in the order they appear here
        self._paged: List[int] = []
        windows: List[int] = []
        for gi, g in enumerate(self.groups):
            if isinstance(g.spec, PagedKVSpec):
                self._paged.append(gi)
                windows.append(int(g.spec.window))
            elif not isinstance(g.spec, FixedStateSpec):
                raise TypeError(f"unknown cache spec {g.spec!r}")
        self._native_index = {gi: k for k, gi in enumerate(self._paged)}
        self._lib = native.lib()
        self._h = self._lib.qvh_create(len(windows), native.ints(windows) if windows else None, self.num_pages,
                                       self.page_size, self.max_requests)
        if not self._h:
            raise ValueError("the cache manager could not be created with these sizes")
        for gi, g in enumerate(self.groups):
            if isinstance(g.spec, PagedKVSpec):
                g.pool = _PoolView(self, self._native_index[gi])
                if allocate:
                    g.tensor = torch.zeros((len(g.layers), self.num_pages + 1, 2, g.spec.num_kv_heads,
                                            self.page_size, g.spec.head_dim), device=self.device, dtype=dtype)
            elif allocate:
                # one more slot than requests: the last is scratch for padded rows of a captured step
                g.tensor = torch.zeros((len(g.layers), self.max_requests + 1, *g.spec.shape),
                                       device=self.device, dtype=_DTYPES.get(g.spec.dtype, g.spec.dtype))
        self._ids: Dict[Hashable, int] = {}          # request id -> the integer the native side knows it by
        self._next_id = 1

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.qvh_destroy(self._h)
            self._h = None

    # ------------------------------------------------------------------ queries
    @property
    def scratch_page(self) -> int:
        return self.num_pages

    @property
    def scratch_slot(self) -> int:
        return self.max_requests

    def paged_groups(self) -> List[int]:
        return list(self._paged)

    def free_pages(self, group: int = None) -> int:
        if not self._paged:
            return self.num_pages
        return self._lib.qvh_free_pages(self._h, -1 if group is None else self._native_index[group])

    def free_slots(self) -> int:
        return self._lib.qvh_free_slots(self._h)

    def has(self, req_id) -> bool:
        return req_id in self._ids

    def native_id(self, req_id) -> int:
        return self._ids[req_id]

    def length(self, req_id) -> int:
        return self._lib.qvh_length(self._h, self._ids[req_id])

    def slot(self, req_id) -> int:
        return self._lib.qvh_slot(self._h, self._ids[req_id])

    def epoch(self, req_id) -> int:
        """A number that differs between two admissions of the same request id."""
        return self._lib.qvh_epoch(self._h, self._ids[req_id])

    def live_requests(self) -> list:
        return list(self._ids)

    def block_table(self, req_id, group: int) -> List[int]:
        nid, g = self._ids[req_id], self._native_index[group]
        n = self._lib.qvh_table_len(self._h, nid, g)
        out = (ctypes.c_int * max(n, 1))()
        self._lib.qvh_table_copy(self._h, nid, g, out, n)
        return list(out[:n])

    def pages_needed(self, req_id, n_new: int) -> Dict[int, int]:
        """Pages each paged group must add so that `n_new` more tokens fit (req_id None: a new request)."""
        known = req_id is not None and req_id in self._ids
        nid = self._ids[req_id] if known else 0
        return {gi: self._lib.qvh_pages_needed(self._h, nid, 1 if known else 0, n_new, self._native_index[gi])
                for gi in self._paged}

    def can_reserve(self, wants: Sequence[Tuple[Hashable, int]]) -> bool:
        """Whether all (request or None, new tokens) of a step fit together."""
        n = len(wants)
        if n == 0:
            return True
        rids = [self._ids.get(r, 0) if r is not None else 0 for r, _ in wants]
        new = [0 if (r is not None and r in self._ids) else 1 for r, _ in wants]
        return bool(self._lib.qvh_can_reserve(self._h, n, native.longs(rids), native.ints(new),
                                              native.ints([k for _, k in wants])))

    def one_more_token_fits(self, req_ids: Sequence[Hashable]) -> int:
        """How many of the given live requests, taken in order, can each hold one more token with
        the pages that are free now.  One pass; the scheduler's check for a round of decoding."""
        n = len(req_ids)
        if n == 0:
            return 0
        return self._lib.qvh_one_more_token_fits(self._h, n, native.longs([self._ids[r] for r in req_ids]))

    # ------------------------------------------------------------------ life of a request
    def admit(self, req_id) -> int:
        """Gives the request a slot (its state slots are zeroed); no pages yet."""
        if req_id in self._ids:
            raise ValueError(f"request {req_id!r} is already live")
        nid = self._next_id
        slot = self._lib.qvh_admit(self._h, nid)
        if slot == -1:
            raise OutOfSlots(f"all {self.max_requests} request slots are taken")
        self._next_id += 1
        self._ids[req_id] = nid
        for g in self.groups:
            if g.pool is None and g.tensor is not None:
                g.tensor[:, slot].zero_()
        return slot

    def reserve(self, req_id, n_new: int) -> bool:
        """Pages for n_new more tokens in every paged group, or nothing at all."""
        return self._lib.qvh_reserve(self._h, self._ids[req_id], n_new) == 1

    def commit(self, req_id, n_new: int) -> None:
        """The request now holds n_new more tokens; pages a window has passed are given back."""
        rc = self._lib.qvh_commit(self._h, self._ids[req_id], n_new)
        if rc == -3:
            raise PageError(f"request {req_id!r} holds more tokens than its pages have room for")

    def release(self, req_id) -> None:
        """The request ends: everything it holds goes back."""
        nid = self._ids.pop(req_id)                  # KeyError for a request that is not live
        self._lib.qvh_release(self._h, nid)

    def youngest(self, among=None):
        """The most recently admitted live request (the one to preempt first)."""
        ids = [i for i in (among if among is not None else self._ids) if i in self._ids]
        if not ids:
            return None
        k = self._lib.qvh_youngest(self._h, len(ids), native.longs([self._ids[i] for i in ids]))
        return ids[k] if k >= 0 else None

    # ------------------------------------------------------------------ captured decode steps
    def fill_decode_rows(self, req_ids: Sequence[Hashable], tokens: Optional[Sequence[int]], rows: int, width: int,
                         host_ptr: int, row_epoch_ptr: int, row_len_ptr: int) -> None:
        """Writes positions, slots and block tables (and tokens, if given) of a decode-only step for
        the given live requests into the pinned buffer at host_ptr, padded to `rows` rows."""
        n = len(req_ids)
        rc = self._lib.qvh_fill_decode(self._h, n, native.longs([self._ids[r] for r in req_ids]),
                                       native.ints(list(tokens)) if tokens is not None else None, rows, width,
                                       self.scratch_page, self.scratch_slot, host_ptr, row_epoch_ptr, row_len_ptr)
        if rc != 0:
            raise KeyError("a request of the decode step is not live")

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
        """No page lost, none held twice, none both free and held; the same for request slots."""
        buf = ctypes.create_string_buffer(512)
        if self._lib.qvh_check(self._h, buf, 512) != 0:
            raise PageError(buf.value.decode())
        if self._lib.qvh_num_live(self._h) != len(self._ids):
            raise PageError("the request table and the native manager disagree on the live requests")
