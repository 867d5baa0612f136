"""Turns the logits of a step into one token per row, on the device.

Order of operations is the reference's (runtime/src/sampler.cpp:43-101): penalties over the
recent tokens, greedy if temperature <= 0, temperature, softmax, top-k, top-p, min-p, draw.
The uniform numbers of the draws come from one generator per request, seeded with the
request's seed, so a request's tokens do not depend on what else is in the batch (the
reference seeds one mt19937_64 per request the same way, scheduler/src/scheduler.cpp:69).
"""
from __future__ import annotations

import random
from typing import List, Sequence

import torch

from ..csrc import ops
from .params import SamplingParams


class RequestSamplerState:
    """What sampling keeps per request: its parameters and its random stream."""

    def __init__(self, params: SamplingParams):
        self.params = params
        self._rng = random.Random(params.seed)

    def next_uniform(self) -> float:
        return self._rng.random()


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, states: Sequence[RequestSamplerState],
               histories: Sequence[Sequence[int]]) -> torch.Tensor:
        """logits float32 [rows, vocab] on the device (may be rewritten); states[r] and histories[r]
        (prompt + generated tokens so far) belong to row r.  Returns int32 ids [rows] on the device."""
        rows = logits.shape[0]
        out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if rows == 0:
            return out
        if all(s.params.greedy and not s.params.has_penalties for s in states):
            ops.argmax(out, logits)
            return out
        f, i = [], []
        width = max([min(len(h), s.params.penalty_last_n) for s, h in zip(states, histories)
                     if s.params.has_penalties] + [0])
        for s, h in zip(states, histories):
            p = s.params
            u = 0.0 if p.greedy else s.next_uniform()
            pen = p.has_penalties
            f.append([p.temperature, p.top_p, p.min_p, u,
                      p.repetition_penalty if pen else 1.0, p.frequency_penalty if pen else 0.0,
                      p.presence_penalty if pen else 0.0])
            recent = list(h[-p.penalty_last_n:]) if (pen and width) else []
            i.append([p.top_k] + recent + [-1] * (width - len(recent)))
        fl = torch.tensor(f, dtype=torch.float32).t().contiguous().to(self.device, non_blocking=True)   # [7, rows]
        it = torch.tensor(i, dtype=torch.int32)
        top_k = it[:, 0].contiguous().to(self.device, non_blocking=True)
        recent = it[:, 1:].contiguous().to(self.device, non_blocking=True) if width else None
        ops.sample(out, logits, fl[0], top_k, fl[1], fl[2], fl[3], recent,
                   fl[4] if width else None, fl[5] if width else None, fl[6] if width else None)
        return out
