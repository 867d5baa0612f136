"""Decode-only steps as captured CUDA graphs.

A step in which every request brings one token has the same kernels and launch shapes
whatever the requests are, once all per-request data (token ids, positions, block tables,
state slots) lives in device buffers the kernels read.  The reference captures one graph
per session because its cache pointer is baked into the launch
(cuda/src/cuda_backend.cu:1341-1360, 1456-1476); here a graph is keyed by the padded number
of requests only, and the integer buffer is refreshed by one copy before each replay.  Rows
beyond the live requests are padding: token 0 at position 0 of the scratch page and the
scratch state slot.

The graph ends with a greedy argmax whose result is also written into the token slots, so
that a decode loop can run with its tokens never leaving the device.
"""
from __future__ import annotations

import gc
import weakref
from typing import Optional

import numpy as np
import torch

from ..csrc import ops
from .batch import StepContext


def _bucket(n: int) -> int:
    b = 1
    while b < n:
        b *= 2
    return b


class DecodeGraph:
    def __init__(self, runner, capacity: int):
        self._runner = weakref.ref(runner)          # the runner owns its graphs; no reference cycle
        self.S = S = capacity
        cache = runner.cache
        self.groups = cache.paged_groups()
        self.width = -(-runner.max_model_len // runner.page_size)
        dev = runner.device
        # dynamic part first (one contiguous copy per step), constants after
        self.n_dyn = 4 * S + len(self.groups) * S * self.width
        total = self.n_dyn + 3 * S + 1
        self.dbuf = torch.zeros(total, dtype=torch.int32, device=dev)
        # One pinned mirror of the dynamic part.  Block-table rows are kept between steps and only
        # their new entries are written, since a request's table grows by one page every page_size steps.
        self.host = torch.zeros(self.n_dyn, dtype=torch.int32, pin_memory=True)
        self.host_np = self.host.numpy()
        self.host_np[3 * S:4 * S] = cache.scratch_slot          # padded rows: scratch slot, scratch page
        self.host_np[4 * S:] = cache.scratch_page
        self.event: Optional[torch.cuda.Event] = None
        # what each block-table row of the mirror holds: the admission it belongs to and how many
        # entries of it are written (0: padding)
        self.row_epoch = np.zeros(max(1, len(self.groups) * S), dtype=np.int64)
        self.row_len = np.zeros(max(1, len(self.groups) * S), dtype=np.int32)
        o = self.n_dyn
        self.dbuf[o:o + S] = torch.arange(S, dtype=torch.int32)                 # tok_seg
        self.dbuf[o + S:o + 2 * S + 1] = torch.arange(S + 1, dtype=torch.int32)   # seg_q_start
        self.dbuf[o + 2 * S + 1:o + 3 * S + 1] = torch.arange(S, dtype=torch.int32)  # want_rows
        tables = {}
        for k, g in enumerate(self.groups):
            b = 4 * S + k * S * self.width
            tables[g] = self.dbuf[b:b + S * self.width].view(S, self.width)
            tables[g].fill_(cache.scratch_page)
        self.dbuf[3 * S:4 * S] = cache.scratch_slot
        self.ctx = StepContext(
            num_tokens=S, num_segments=S, num_wanted=S, token_ids=self.dbuf[0:S], tok_pos=self.dbuf[S:2 * S],
            tok_seg=self.dbuf[o:o + S], seg_q_start=self.dbuf[o + S:o + 2 * S + 1], seg_pos0=self.dbuf[2 * S:3 * S],
            seg_slot=self.dbuf[3 * S:4 * S], want_rows=self.dbuf[o + 2 * S + 1:o + 3 * S + 1], block_tables=tables,
            seg_len=[1] * S, seg_start_pos=[0] * S, seg_slots=[cache.scratch_slot] * S, seg_first=[False] * S,
            max_q_len=1, max_ctx_len=runner.max_model_len)
        self.ctx.captured = True
        self.next_ids = torch.zeros(S, dtype=torch.int32, device=dev)
        self.logits = None
        self.graph = None
        self.kernels = 0
        self._capture()

    @property
    def runner(self):
        return self._runner()

    def _forward(self):
        logits = self.runner.model.forward(self.ctx, self.runner.cache)
        ops.argmax(self.next_ids, logits)
        self.dbuf[0:self.S].copy_(self.next_ids)
        return logits

    def _capture(self):
        side = torch.cuda.Stream(device=self.runner.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._forward()                                   # builds libraries, sets attributes, warms the allocator
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(self.runner.device)
        before = ops.launch_count()
        self.graph = torch.cuda.CUDAGraph()
        # No garbage collection while capturing: freeing a pinned buffer or an event of some
        # older object touches the default stream, which invalidates a capture in progress.
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph):
                self.logits = self._forward()
        finally:
            if gc_was_on:
                gc.enable()
        self.kernels = ops.launch_count() - before
        self.dbuf[0:self.S].zero_()

    def run(self, req_ids, tokens) -> None:
        """Refreshes the integer buffer for the given live requests, whose pages for one more token
        are reserved, and replays.  tokens None: the token slots keep what the last replay left."""
        S, n = self.S, len(req_ids)
        if n > S:
            raise ValueError(f"{n} requests in a captured step of {S}")
        if self.event is not None:
            self.event.synchronize()                          # the last copy has read the mirror
        # Block-table rows are kept between steps; the C++ side writes only what grew or changed.
        self.runner.cache.fill_decode_rows(req_ids, tokens, S, self.width, self.host.data_ptr(),
                                           self.row_epoch.ctypes.data, self.row_len.ctypes.data)
        lo = 0 if tokens is not None else S
        self.dbuf[lo:self.n_dyn].copy_(self.host[lo:], non_blocking=True)
        if self.event is None:
            self.event = torch.cuda.Event()
        self.event.record()
        self.runner._builder.h2d_bytes += (self.n_dyn - lo) * 4
        self.graph.replay()
        ops.add_launches(self.kernels)


class DecodeLoop:
    """Greedy decoding of a fixed set of live requests with the tokens kept on the device: each
    step feeds the previous step's argmax.  The host only reserves pages and refreshes
    positions and block tables."""

    def __init__(self, runner, req_ids):
        self.runner = runner
        self.req_ids = list(req_ids)
        self.graph = runner.decode_graph(len(self.req_ids))
        self.produced = 0

    def start(self, first_tokens) -> None:
        n = len(self.req_ids)
        self.graph.dbuf[0:n].copy_(torch.tensor(list(first_tokens), dtype=torch.int32))

    def step(self) -> None:
        r = self.runner
        for rid in self.req_ids:
            if not r.cache.reserve(rid, 1):
                raise RuntimeError("out of pages in a decode loop")
        self.graph.run(self.req_ids, None)
        for rid in self.req_ids:
            r.cache.commit(rid, 1)
        self.produced += 1

    def last_tokens(self) -> torch.Tensor:
        return self.graph.next_ids[: len(self.req_ids)]

    def finish(self) -> None:
        torch.cuda.synchronize(self.runner.device)
        ops.check_kernel_errors()                  # a kernel that gave up on a bounded wait makes the loop's tokens void
