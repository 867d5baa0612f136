"""The Python entry point: token ids in, token ids out.

`LLM(model_dir).generate(prompts, SamplingParams(...))` is what the reference's
`qorvix generate` does (core/src/main.cpp:384-445: prefill, sample, decode loop, stop on EOS
or --max) for one or many prompts at once, through the scheduler.  Tokenizers are out of
scope: prompts are lists of token ids.
"""
from __future__ import annotations

import time
from typing import List, Optional, Sequence, Union

import torch

from ..csrc import ops
from ..sampling import Sampler, SamplingParams
from .runner import ModelRunner
from .scheduler import RequestResult, Scheduler, SchedulerConfig


class LLM:
    def __init__(self, model=None, *, config=None, tensors=None, dtype="bfloat16", max_tokens: int = 8192,
                 page_size: int = 16, max_concurrent: int = 8, max_batch_tokens: int = 2048,
                 max_chunk: int = 0, max_model_len: Optional[int] = None, device="cuda", lookahead: bool = True):
        self.runner = ModelRunner(model, config=config, tensors=tensors, dtype=dtype, max_tokens=max_tokens,
                                  page_size=page_size, max_requests=max_concurrent,
                                  max_model_len=max_model_len, device=device)
        self.sampler = Sampler(self.runner.device)
        self.scheduler_config = SchedulerConfig(max_concurrent=max_concurrent, max_batch_tokens=max_batch_tokens,
                                                max_chunk=max_chunk, lookahead=lookahead)
        eos = getattr(self.runner.config, "eos_token_ids", ())
        self.eos_token_ids = tuple(eos)
        self.last_stats = {}

    def new_scheduler(self) -> Scheduler:
        return Scheduler(self.runner, self.sampler, self.scheduler_config, self.eos_token_ids)

    def generate(self, prompts: Sequence[Sequence[int]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 on_token=None) -> List[RequestResult]:
        """Generates for every prompt (a list of token ids); results come back in prompt order."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        sched = self.new_scheduler()
        t0 = time.perf_counter()
        ids = [sched.submit(p, sp, on_token=on_token) for p, sp in zip(prompts, params)]
        results = {r.id: r for r in sched.run_to_completion()}
        torch.cuda.synchronize(self.runner.device)
        dt = time.perf_counter() - t0
        ops.check_kernel_errors()
        self.last_stats = dict(sched.stats, seconds=dt,
                               generated=sum(len(r.tokens) for r in results.values()))
        return [results[i] for i in ids]
