"""The step function: a batch of (request, its next tokens) in, logits at the wanted places out.

It runs only the tokens it is given, as one batch, from the cache that earlier steps
left; prompt portions stand beside single decoded tokens, cut anywhere.  This is the seam the
reference calls IInferenceEngine::forward / forwardBatch
(runtime/include/qorvix/runtime/inference_engine.hpp:36-97), widened from one token of one
session to any mix of segments.  The scheduler, the generation entry point and the trace
replay tool all drive the model through this one class.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict, Hashable, Iterable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager, OutOfPages, OutOfSlots
from ..config import load_config, lookup_architecture
from ..csrc import ops
from ..models.text_model import TextModel
from ..parts.base import Runtime
from ..weights import Checkpoint, TensorSource
from .batch import BatchBuilder, StepContext, StepEntry

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"dtype must be bfloat16 or float32, not {dtype}")
        return dtype
    if str(dtype) not in _DTYPES:
        raise ValueError(f"dtype must be one of {', '.join(_DTYPES)}, not {dtype!r}")
    return _DTYPES[str(dtype)]


class ModelRunner:
    def __init__(self, model_dir=None, *, config=None, tensors=None, dtype="bfloat16", max_tokens: int = 4096,
                 page_size: int = 16, max_requests: int = 8, max_model_len: Optional[int] = None,
                 device="cuda", use_graphs: bool = True, max_graph_batch: int = 64):
        """model_dir: folder with config.json and model.safetensors; or config + tensors (a
        mapping name -> tensor) for a model held in memory.  max_tokens sizes the page pool."""
        self.device = torch.device(device)
        _require_cuda(self.device)
        self.dtype = parse_dtype(dtype)
        if model_dir is not None:
            self.config = load_config(model_dir)
            source = TensorSource(checkpoint=Checkpoint(model_dir), device=self.device,
                                  compute_dtype=self.dtype, where=str(Path(model_dir) / "model.safetensors"))
        else:
            if config is None or tensors is None:
                raise ValueError("give a model folder, or a configuration together with its tensors")
            self.config = config
            source = TensorSource(tensors=tensors, device=self.device, compute_dtype=self.dtype, where="tensors in memory")
        entry = lookup_architecture(self.config.architecture)
        self.spec = entry.build_spec(self.config)
        self.page_size = int(page_size)
        pool_tokens = -(-int(max_tokens) // self.page_size) * self.page_size
        limit = self.spec.max_position if self.spec.max_position else pool_tokens
        self.max_model_len = int(max_model_len) if max_model_len else min(limit, pool_tokens)
        self.rt = Runtime(device=self.device, dtype=self.dtype, max_positions=self.max_model_len,
                          page_size=self.page_size)
        if self.dtype == torch.bfloat16:
            ops.prepare_products(self.device)
        self.model = TextModel(self.spec, source, self.rt)
        self.cache = CacheManager(self.model.cache_needs(), max_tokens=pool_tokens, page_size=self.page_size,
                                  max_requests=max_requests, device=self.device, dtype=self.dtype)
        self.vocab_size = self.spec.vocab_size
        self._builder = BatchBuilder(self.device)
        self.use_graphs = bool(use_graphs)
        self.max_graph_batch = int(max_graph_batch)
        self._graphs: Dict[int, object] = {}
        self.steps_run = 0
        self.tokens_run = 0

    # ------------------------------------------------------------------ planning
    def can_run(self, entries: Sequence[StepEntry]) -> bool:
        """Whether slots and pages suffice for all entries together (nothing is taken)."""
        return self.cache.can_reserve([(e.req_id, len(e.tokens)) for e in entries])

    def length(self, req_id) -> int:
        return self.cache.length(req_id) if self.cache.has(req_id) else 0

    # ------------------------------------------------------------------ the step
    @property
    def h2d_bytes(self) -> int:
        return self._builder.h2d_bytes

    def decode_graph(self, n: int):
        """The captured decode step that holds n requests (captured on first use)."""
        from .decode_graph import DecodeGraph, _bucket
        cap = _bucket(n)
        if cap not in self._graphs:
            self._graphs[cap] = DecodeGraph(self, cap)
        return self._graphs[cap]

    def decoder(self, req_ids):
        """A greedy decode loop over live requests whose tokens stay on the device."""
        from .decode_graph import DecodeLoop
        return DecodeLoop(self, req_ids)

    def prepare(self, entries: Sequence[StepEntry], build: bool = True):
        """Admits new requests, reserves pages for every entry (all or nothing) and builds the
        step's context.  Raises OutOfPages / OutOfSlots with nothing changed."""
        seen = set()
        arrays = []
        for e in entries:
            if e.req_id in seen:
                raise ValueError(f"request {e.req_id!r} appears twice in one step")
            seen.add(e.req_id)
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.req_id!r} brings no tokens")
            if n == 1:                                  # a decoded token: no array for one id
                toks = [int(e.tokens[0])]
                bad = None if 0 <= toks[0] < self.vocab_size else toks[0]
            else:
                toks = np.asarray(e.tokens, dtype=np.int64)
                if toks.ndim != 1:
                    raise ValueError(f"request {e.req_id!r}: tokens must be a flat sequence of ids")
                bad = None
                if int(toks.min()) < 0 or int(toks.max()) >= self.vocab_size:
                    bad = int(toks[(toks < 0) | (toks >= self.vocab_size)][0])
            if bad is not None:
                raise ValueError(f"request {e.req_id!r}: token id {bad} is outside the vocabulary of {self.vocab_size}")
            arrays.append(toks)
            if any(not 0 <= int(w) < n for w in e.want):
                raise ValueError(f"request {e.req_id!r}: a wanted place is outside its {n} tokens")
            if self.length(e.req_id) + n > self.max_model_len:
                raise ValueError(f"request {e.req_id!r} would hold {self.length(e.req_id) + n} tokens, "
                                 f"more than the engine's limit of {self.max_model_len}")
        if not self.cache.can_reserve([(e.req_id, len(e.tokens)) for e in entries]):
            new = sum(1 for e in entries if not self.cache.has(e.req_id))
            if new > self.cache.free_slots():
                raise OutOfSlots(f"{new} new requests but only {self.cache.free_slots()} free request slots")
            raise OutOfPages(f"the step needs more pages than the {self.cache.free_pages()} that are free")
        segs = []
        for e, toks in zip(entries, arrays):
            first = not self.cache.has(e.req_id)
            if first:
                self.cache.admit(e.req_id)
            ok = self.cache.reserve(e.req_id, len(e.tokens))
            assert ok, "reservation was checked for the whole step"
            if not build:
                continue
            segs.append(dict(tokens=toks, pos0=self.cache.length(e.req_id),
                             slot=self.cache.slot(e.req_id), want=[int(w) for w in e.want], first=first,
                             rid=(e.req_id, self.cache.epoch(e.req_id))))
        if not build:
            return None
        tables = {g: [self.cache.block_table(e.req_id, g) for e in entries] for g in self.cache.paged_groups()}
        return self._builder.build(segs, tables, self.cache.scratch_page)

    step_views = True          # step() takes copy_logits and sets last_greedy_ids

    def step(self, entries: Sequence[StepEntry], end: Iterable[Hashable] = (), copy_logits: bool = True,
             device_tokens: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Runs one batch.  Returns float32 logits [number of wanted places, vocab] on the device,
        ordered by entry and then by `want`, or None when nothing is wanted.  Requests in `end`
        are finished after this step and what they hold is given back.  With copy_logits=False the
        result may be a view of a buffer that the next step overwrites (for a caller that consumes it
        at once).  After a captured decode step whose every row is wanted, last_greedy_ids holds
        the argmax of each row (computed inside the captured step), else it is None.
        device_tokens: int32 ids on the device, one per entry, to feed instead of the entries' own
        (placeholder) tokens; only for a decode-only step that runs as a captured graph, which lets
        a caller launch a step before it has read the ids the step before produced."""
        entries = list(entries)
        logits = None
        self.last_greedy_ids = None
        if entries and self.use_graphs and len(entries) <= self.max_graph_batch and all(len(e.tokens) == 1 for e in entries):
            # decode-only: replay the captured step
            self.prepare(entries, build=False)
            graph = self.decode_graph(len(entries))
            if device_tokens is not None:
                graph.dbuf[0: len(entries)].copy_(device_tokens[: len(entries)])
                graph.run([e.req_id for e in entries], None)
            else:
                graph.run([e.req_id for e in entries], [int(e.tokens[0]) for e in entries])
            rows = [i for i, e in enumerate(entries) if len(e.want)]
            if rows:
                if len(rows) == len(entries):
                    logits = graph.logits[: len(rows)]
                    if copy_logits:
                        logits = logits.clone()
                    self.last_greedy_ids = graph.next_ids[: len(rows)]
                else:
                    logits = graph.logits[torch.tensor(rows, device=self.device)]
            for e in entries:
                self.cache.commit(e.req_id, 1)
            self.steps_run += 1
            self.tokens_run += len(entries)
        elif entries:
            if device_tokens is not None:
                raise ValueError("device_tokens need a decode-only step that runs as a captured graph")
            # A mixed step runs its single-token entries first: the attention kernels then serve the
            # decoded tokens and the prompt portions each with the kernel made for them.  The logits
            # go back in the order the caller gave.
            order, back = single_token_entries_first(entries)
            entries = [entries[i] for i in order]
            ctx = self.prepare(entries)
            logits = self.model.forward(ctx, self.cache)
            if logits is not None and back is not None and back != list(range(len(back))):
                logits = logits[torch.tensor(back, device=self.device)]
            for e in entries:
                self.cache.commit(e.req_id, len(e.tokens))
            self.steps_run += 1
            self.tokens_run += ctx.num_tokens
        for req_id in end:
            self.release(req_id)
        return logits

    def release(self, req_id) -> None:
        if self.cache.has(req_id):
            self.cache.release(req_id)


def single_token_entries_first(entries: Sequence[StepEntry]):
    """The order in which a step's entries run (single-token entries first, otherwise as given) and,
    when that order differs from the caller's, for every wanted row in the caller's order its row in
    the step's output (else None)."""
    order = sorted(range(len(entries)), key=lambda i: len(entries[i].tokens) != 1)
    if order == list(range(len(entries))):
        return order, None
    first_row, row = {}, 0
    for i in order:
        first_row[i] = row
        row += len(entries[i].want)
    back = [first_row[i] + k for i, e in enumerate(entries) for k in range(len(e.want))]
    return order, back


def _require_cuda(device: torch.device) -> None:
    if device.type != "cuda":
        raise RuntimeError("qorvix_b200 runs on a CUDA device only (sm_100a); there is no CPU path")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available; qorvix_b200 has no CPU path")
