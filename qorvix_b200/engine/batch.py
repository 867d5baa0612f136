"""One step's batch: requests with their next tokens, flattened for the kernels.

The reference's step is one token of one session (runtime/include/qorvix/runtime/inference_engine.hpp:13-17,
51); here a step is any mix of segments, a segment being the next n >= 1 tokens of one
request (n > 1: a portion of a prompt; n = 1: usually a decoded token).  All integer
arrays of a step travel to the device in one copy from one pinned buffer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    """The next `tokens` of request `req_id`; `want` are the places among these tokens whose
    logits are asked for (may be empty)."""
    req_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepContext:
    """What parts see of a step.  Device tensors are int32."""
    num_tokens: int
    num_segments: int
    num_wanted: int
    token_ids: torch.Tensor            # [T]
    tok_pos: torch.Tensor              # [T] absolute position of each token in its request
    tok_seg: torch.Tensor              # [T] segment of each token
    seg_q_start: torch.Tensor          # [S+1] first row of each segment
    seg_pos0: torch.Tensor             # [S] position of each segment's first token
    seg_slot: torch.Tensor             # [S] request slot (index into fixed-size state)
    want_rows: torch.Tensor            # [R] rows whose logits are wanted
    block_tables: Dict[int, torch.Tensor]      # cache group -> [S, max_blocks]
    # host copies, for decisions that must not wait for the device
    seg_len: List[int] = field(default_factory=list)
    seg_start_pos: List[int] = field(default_factory=list)
    seg_slots: List[int] = field(default_factory=list)
    seg_first: List[bool] = field(default_factory=list)     # the request's first portion
    max_q_len: int = 0
    max_ctx_len: int = 0
    captured: bool = False             # the step is being captured or replayed as a CUDA graph
    next_norm: object = None           # set by the model before each block: the norm the block after it starts with

    @property
    def decode_only(self) -> bool:
        return self.max_q_len == 1

    def any_block_table(self) -> torch.Tensor:
        for t in self.block_tables.values():
            return t
        return self.seg_pos0.reshape(-1, 1)


class BatchBuilder:
    """Packs the integer arrays of a step into one pinned host buffer and one device buffer."""

    def __init__(self, device, pin: bool = True):
        self.device = torch.device(device)
        self._pin = pin and self.device.type == "cuda"
        # The copy to the device is asynchronous, so a pinned buffer may be rewritten only after
        # its last copy has run: a small ring of buffers, each guarded by an event.
        self._ring: List[list] = [[None, None] for _ in range(4)]
        self._turn = 0
        self.h2d_bytes = 0                       # bytes copied to the device so far

    def _host_buffer(self, n: int):
        self._turn = (self._turn + 1) % len(self._ring)
        slot = self._ring[self._turn]
        if slot[1] is not None:
            slot[1].synchronize()
        if slot[0] is None or slot[0].numel() < n:
            cap = max(1024, 1 << (n - 1).bit_length())
            slot[0] = torch.empty(cap, dtype=torch.int32, pin_memory=self._pin)
        return slot[0][:n], slot

    def build(self, segs: List[dict], group_tables: Dict[int, List[List[int]]], scratch_page: int) -> StepContext:
        """segs: dicts with tokens, pos0, slot, want, first.  group_tables[g][s] = page ids of
        segment s in cache group g (-1 entries, given back to the pool, read as the scratch page)."""
        S = len(segs)
        lens = [len(s["tokens"]) for s in segs]
        T = sum(lens)
        R = sum(len(s["want"]) for s in segs)
        widths = {g: max(1, max((len(t) for t in tabs), default=1)) for g, tabs in group_tables.items()}
        total = 3 * T + (S + 1) + 2 * S + R + sum(S * w for w in widths.values())
        host, ring_slot = self._host_buffer(max(total, 1))
        h = host.numpy()                                          # the arrays are written in place, no lists of T ints
        qstart = np.zeros(S + 1, dtype=np.int64)
        np.cumsum(lens, out=qstart[1:])
        pos0 = np.fromiter((s["pos0"] for s in segs), dtype=np.int64, count=S)
        for si, s in enumerate(segs):
            a, b = int(qstart[si]), int(qstart[si + 1])
            h[a:b] = s["tokens"]
            h[T + a: T + b] = np.arange(s["pos0"], s["pos0"] + (b - a), dtype=np.int32)
            h[2 * T + a: 2 * T + b] = si
        o = 3 * T
        h[o: o + S + 1] = qstart; o += S + 1
        h[o: o + S] = pos0; o += S
        h[o: o + S] = [s["slot"] for s in segs]; o += S
        if R:
            h[o: o + R] = [int(qstart[si]) + w for si, s in enumerate(segs) for w in s["want"]]
        o += R
        offsets = {}
        for g, tabs in group_tables.items():
            offsets[g] = o
            w = widths[g]
            block = h[o: o + S * w].reshape(S, w)
            block[:] = scratch_page
            for si, t in enumerate(tabs):
                if len(t):
                    row = np.asarray(t, dtype=np.int32)
                    block[si, : len(t)] = np.where(row >= 0, row, scratch_page)
            o += S * w
        if self.device.type == "cuda":
            dev = host.to(self.device, non_blocking=True)
            self.h2d_bytes += host.numel() * 4
            if ring_slot[1] is None:
                ring_slot[1] = torch.cuda.Event()
            ring_slot[1].record()
        else:
            dev = host.clone()
        o = 0

        def take(n):
            nonlocal o
            v = dev[o:o + n]
            o += n
            return v

        token_ids, tok_pos, tok_seg = take(T), take(T), take(T)
        seg_q_start, seg_pos0, seg_slot, want_rows = take(S + 1), take(S), take(S), take(R)
        block_tables = {g: dev[offsets[g]: offsets[g] + S * widths[g]].view(S, widths[g]) for g in group_tables}
        return StepContext(
            num_tokens=T, num_segments=S, num_wanted=R, token_ids=token_ids, tok_pos=tok_pos,
            tok_seg=tok_seg, seg_q_start=seg_q_start, seg_pos0=seg_pos0, seg_slot=seg_slot,
            want_rows=want_rows, block_tables=block_tables, seg_len=lens,
            seg_start_pos=[s["pos0"] for s in segs], seg_slots=[s["slot"] for s in segs],
            seg_first=[s["first"] for s in segs], max_q_len=max(lens, default=0),
            max_ctx_len=max((s["pos0"] + len(s["tokens"]) for s in segs), default=0))
