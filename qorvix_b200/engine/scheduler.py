"""Continuous batching above the step function.

The reference's scheduler (scheduler/src/scheduler.cpp:94-188) admits up to maxConcurrent
requests by (priority, arrival), prefills each whole prompt token by token inside the admitting
step, then decodes one token per active request per step, and retires on EOS, maxNewTokens or
the sequence limit.  Kept: queue order, one decoded token per request per step, the three
ways to finish, results per request, streaming callback.  New: a token budget per step,
prompts cut into portions that run beside the decode tokens of other requests, admission only
when the pages of the whole prompt can be reserved, and a decided answer to running out of pages (the reference has
none: scheduler.cpp never looks at the pool):

  * a waiting request that does not fit stays queued (it is not rejected);
  * when a running request cannot get the page its next token needs, the most recently
    admitted running request is preempted: its pages go back, and it re-enters the front of
    the queue with prompt + generated tokens as its prompt (recomputed later);
  * a request that is alone and still does not fit finishes with reason "length".
"""
from __future__ import annotations

import heapq
import itertools
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence

from ..sampling import RequestSamplerState, SamplingParams
from .batch import StepEntry

WAITING, RUNNING, DONE = "waiting", "running", "done"


@dataclass
class SchedulerConfig:
    max_concurrent: int = 8          # requests running at once (reference default, scheduler.hpp:47)
    max_batch_tokens: int = 2048     # token budget of one step
    max_chunk: int = 0               # longest prompt portion; 0: the budget alone limits it
    lookahead: bool = False          # while all requests decode, launch a step before the last one's ids are read


@dataclass
class RequestResult:
    """The reference's RequestResult (scheduler.hpp:33-40) in token ids."""
    id: int
    tokens: List[int]
    prompt_tokens: int
    hit_eos: bool = False
    rejected: bool = False
    finish_reason: str = ""          # "eos" | "stop" | "max_new_tokens" | "length" | "rejected"
    preemptions: int = 0


@dataclass
class _Request:
    id: int
    prompt: List[int]                # what must be in the cache before decoding (grows on preemption)
    n_prompt: int                    # the user's prompt length
    params: SamplingParams
    priority: int
    seq: int
    sampler: RequestSamplerState
    on_token: Optional[Callable[[int, int], None]] = None
    state: str = WAITING
    generated: List[int] = field(default_factory=list)
    computed: int = 0                # tokens of prompt (+ fed generated tokens) in the cache
    pending: Optional[int] = None    # sampled, not yet fed
    hit_eos: bool = False
    finish_reason: str = ""
    preemptions: int = 0

    def history(self) -> List[int]:
        return self.prompt[: self.n_prompt] + self.generated


@dataclass
class StepPlan:
    """What one step will run: (request, number of its next tokens) in batch order, plus the
    decisions taken to get there."""
    decode: List[int] = field(default_factory=list)           # request ids fed one sampled token
    prefill: List[tuple] = field(default_factory=list)        # (request id, portion length)
    admitted: List[int] = field(default_factory=list)
    preempted: List[int] = field(default_factory=list)
    finished_for_length: List[int] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return len(self.decode) + sum(n for _, n in self.prefill)


@dataclass
class _InFlight:
    """A decode step that has been launched and whose sampled ids are still on the device."""
    requests: List[_Request]                 # one per row
    ids: object                              # device tensor [rows] of sampled ids (the next launch feeds them)
    host_ids: object = None                  # their copy to pinned host memory, requested right after the step ...
    copied: object = None                    # ... and the event that says it has arrived
    dead: set = field(default_factory=set)   # rows whose request ended in the step before: their id is dropped


class Scheduler:
    def __init__(self, runner, sampler, config: SchedulerConfig = None, eos_token_ids: Sequence[int] = ()):
        """runner: has .cache (CacheManager), .step(entries, end), .release(id), .max_model_len.
        sampler: has .sample(logits, states, histories) -> ids."""
        self.runner = runner
        self.sampler = sampler
        self.config = config or SchedulerConfig()
        self.eos = set(int(e) for e in eos_token_ids)
        self._ids = itertools.count(1)
        self._seq = itertools.count()
        self._front = itertools.count(-1, -1)      # preempted requests go before everything of their priority
        self._waiting: List[tuple] = []            # heap of (-priority, seq, id)
        self._requests: Dict[int, _Request] = {}
        self._running: List[int] = []              # in admission order
        self._early: List[RequestResult] = []
        self._ahead: Optional[_InFlight] = None      # lookahead: the decode step whose ids are not read yet
        self._pinned: list = []                      # host buffers the ids of launched steps are copied to
        self.stats = {"steps": 0, "tokens": 0, "preemptions": 0, "admitted": 0, "ahead_steps": 0}

    # ------------------------------------------------------------------ submitting
    def submit(self, prompt: Sequence[int], params: SamplingParams = None, priority: int = 0,
               on_token: Callable[[int, int], None] = None) -> int:
        """Queues a request and returns its id.  An empty prompt, or one that cannot fit the
        engine's sequence limit, is rejected: its result comes back from the next step()."""
        params = params or SamplingParams()
        rid = next(self._ids)
        prompt = [int(t) for t in prompt]
        if not prompt or len(prompt) >= self.runner.max_model_len:
            self._early.append(RequestResult(rid, [], len(prompt), rejected=True, finish_reason="rejected"))
            return rid
        req = _Request(id=rid, prompt=prompt, n_prompt=len(prompt), params=params, priority=int(priority),
                       seq=next(self._seq), sampler=RequestSamplerState(params), on_token=on_token)
        self._requests[rid] = req
        heapq.heappush(self._waiting, (-req.priority, req.seq, rid))
        return rid

    def idle(self) -> bool:
        return not self._waiting and not self._running and not self._early and self._ahead is None

    def waiting(self) -> int:
        return len(self._waiting)

    def active(self) -> int:
        return len(self._running)

    def decoding(self) -> bool:
        """Nothing waits and every running request has its whole prompt in the cache."""
        return not self._waiting and bool(self._running) and all(
            self._requests[rid].computed >= len(self._requests[rid].prompt) for rid in self._running)

    # ------------------------------------------------------------------ deciding
    def plan_step(self) -> StepPlan:
        """Decides what the next step runs.  Changes queue and running set (admission,
        preemption) but touches neither the model nor the pages of requests that stay."""
        cfg, cache = self.config, self.runner.cache
        plan = StepPlan()
        while True:
            budget = cfg.max_batch_tokens
            wants = []                                    # (request id, new tokens) so far
            plan.decode, plan.prefill = [], []
            fits = True
            # decode tokens first: one per running request that has a sampled token to feed
            ready = [rid for rid in self._running if self._requests[rid].pending is not None][:budget]
            n_fit = cache.one_more_token_fits(ready)
            if n_fit < len(ready):
                fits = False
            else:
                plan.decode = ready
                wants = [(rid, 1) for rid in ready]
                budget -= len(ready)
            if fits:
                for rid in self._running:                 # then portions of running prompts
                    r = self._requests[rid]
                    if r.pending is None and budget > 0:
                        n = min(len(r.prompt) - r.computed, budget, cfg.max_chunk or budget)
                        while n > 0 and not cache.can_reserve(wants + [(rid, n)]):
                            n = self._shrink(rid, n, wants)
                        if n <= 0:
                            if not plan.decode and not plan.prefill:
                                fits = False              # nothing at all can move
                            break
                        wants.append((rid, n))
                        plan.prefill.append((rid, n))
                        budget -= n
            if fits:
                break
            victim = self._running[-1]                     # most recently admitted
            if len(self._running) == 1:
                self._running.remove(victim)
                self._finish(self._requests[victim], "length")
                plan.finished_for_length.append(victim)
                return plan
            self._preempt(victim)
            plan.preempted.append(victim)
        # admission: by priority then arrival, while a slot, budget and pages for a first portion exist
        while self._waiting and len(self._running) < cfg.max_concurrent and budget > 0:
            _, _, rid = self._waiting[0]
            r = self._requests[rid]
            n = min(len(r.prompt) - r.computed, budget, cfg.max_chunk or budget)
            # admitted only when the pages of its whole prompt are free now, although the prompt
            # may be fed in portions: a request let in on its first portion alone would soon have
            # to be preempted again
            if not cache.can_reserve(wants + [(rid, len(r.prompt) - r.computed)]):
                n = 0
            if n <= 0:
                if not self._running and not wants:
                    heapq.heappop(self._waiting)           # alone and still too big for the pool
                    self._finish(r, "length")
                    plan.finished_for_length.append(rid)
                    continue
                break
            heapq.heappop(self._waiting)
            r.state = RUNNING
            self._running.append(rid)
            self.stats["admitted"] += 1
            plan.admitted.append(rid)
            wants.append((rid, n))
            plan.prefill.append((rid, n))
            budget -= n
        return plan

    def _shrink(self, rid, n: int, wants) -> int:
        """A shorter portion that ends on a page edge, or 0."""
        page = self.runner.cache.page_size
        have = self.runner.cache.length(rid) if self.runner.cache.has(rid) else 0
        shorter = ((have + n - 1) // page) * page - have
        return shorter if 0 < shorter < n else 0

    def _preempt(self, rid: int) -> None:
        r = self._requests[rid]
        self._running.remove(rid)
        self.runner.release(rid)
        if r.pending is not None:
            r.prompt = r.prompt[: r.n_prompt] + r.generated     # generated includes the pending token
            r.pending = None
        r.computed = 0
        r.state = WAITING
        r.preemptions += 1
        self.stats["preemptions"] += 1
        heapq.heappush(self._waiting, (-r.priority, next(self._front), rid))

    # ------------------------------------------------------------------ running
    def step(self) -> List[RequestResult]:
        """One round.  Returns the requests that finished in it."""
        if self.config.lookahead and getattr(self.runner, "step_views", False):
            return self._step_lookahead()
        return self._step_sync()

    # Lookahead: while every running request decodes and nothing waits, the next step is launched
    # before the ids of the one in flight are read, so that the device never waits for the host's
    # bookkeeping.  The tokens it feeds are the in-flight step's ids, taken on the device.  A request
    # that turns out to have ended in the step in flight (end of sequence, stop token) has then run
    # one token too far: that token is dropped, and its pages go back at once (the step that still
    # writes to them is ahead of any later use in stream order).  Limits that the host can foresee
    # (max_new_tokens, the sequence limit, pages, new arrivals) end the lookahead before they bite,
    # and the rounds in between run one at a time as without it.
    def _steady(self, reqs: List[_Request]) -> bool:
        if self._waiting or not reqs or len(reqs) > getattr(self.runner, "max_graph_batch", 0):
            return False
        if not getattr(self.runner, "use_graphs", False):
            return False
        for r in reqs:
            p = r.params
            if p.has_penalties or len(r.generated) + 1 >= p.max_new_tokens:
                return False
            if r.n_prompt + len(r.generated) + 1 >= self.runner.max_model_len:
                return False
        ids = [r.id for r in reqs]
        return self.runner.cache.one_more_token_fits(ids) == len(ids)

    def _launch(self, reqs: List[_Request], device_tokens=None) -> _InFlight:
        entries = [StepEntry(r.id, [0 if device_tokens is not None else r.pending], [0]) for r in reqs]
        logits = self.runner.step(entries, copy_logits=False, device_tokens=device_tokens)
        self.stats["steps"] += 1
        self.stats["tokens"] += len(reqs)
        for r in reqs:
            r.computed += 1
            r.pending = None
        greedy_ids = self.runner.last_greedy_ids
        if greedy_ids is not None and all(r.params.greedy for r in reqs):
            ids = greedy_ids.clone()                       # the next launch overwrites the step's own buffer
        else:
            ids = self.sampler.sample(logits, [r.sampler for r in reqs], [r.history() for r in reqs])
        t = _InFlight(requests=list(reqs), ids=ids)
        # The copy to the host is queued now, ahead of the next launch: queued after it, it would
        # wait for that whole step, and reading the ids would stall the host for a step.
        if hasattr(ids, "is_cuda") and ids.is_cuda:
            import torch
            if not self._pinned:
                self._pinned = [torch.empty(max(64, self.config.max_concurrent), dtype=torch.int32, pin_memory=True) for _ in range(3)]
            buf = self._pinned[self.stats["steps"] % 3][: len(reqs)]
            buf.copy_(ids, non_blocking=True)
            t.host_ids, t.copied = buf, torch.cuda.Event()
            t.copied.record()
        return t

    def _complete(self, t: _InFlight, fed: bool) -> List[RequestResult]:
        """Reads the ids of a launched step.  fed: the step after it is launched already and feeds
        these ids itself; a request that goes on then has nothing pending on the host."""
        finished = []
        if t.copied is not None:
            t.copied.synchronize()
            toks = t.host_ids.tolist()
        else:
            toks = t.ids.tolist()
        for r, tok in zip(t.requests, toks):
            if r.id in t.dead:
                continue
            self._accept(r, int(tok))
            if r.state == DONE:
                self._running.remove(r.id)
                self.runner.release(r.id)
                finished.append(self._result(self._requests.pop(r.id)))
            elif fed:
                r.pending = None
        return finished

    def _step_lookahead(self) -> List[RequestResult]:
        t = self._ahead
        if t is None:
            reqs = [self._requests[rid] for rid in self._running]
            if not self._steady(reqs) or any(r.pending is None for r in reqs):
                return self._step_sync()
            finished, self._early = self._early, []
            self._ahead = self._launch(reqs)               # left in flight; its ids are read in the next round
            return finished
        finished, self._early = self._early, []
        live = [r for r in t.requests if r.id not in t.dead]
        nxt = None
        if not t.dead and [r.id for r in live] == self._running and self._steady(live):
            nxt = self._launch(live, device_tokens=t.ids)
            self.stats["ahead_steps"] += 1
        finished += self._complete(t, fed=nxt is not None)
        if nxt is not None:
            nxt.dead = {r.id for r in nxt.requests if r.id not in self._requests}
        self._ahead = nxt
        return finished

    def _step_sync(self) -> List[RequestResult]:
        """One round: plan, run the batch, sample, finish and free."""
        finished: List[RequestResult] = self._early
        self._early = []
        plan = self.plan_step()
        for rid in plan.finished_for_length:
            finished.append(self._result(self._requests.pop(rid)))
        entries, samplers = [], []
        for rid in plan.decode:
            r = self._requests[rid]
            entries.append(StepEntry(rid, [r.pending], [0]))
            samplers.append(r)
        for rid, n in plan.prefill:
            r = self._requests[rid]
            last = r.computed + n == len(r.prompt)
            entries.append(StepEntry(rid, r.prompt[r.computed: r.computed + n], [n - 1] if last else []))
            if last:
                samplers.append(r)
        if not entries:
            return finished
        views = getattr(self.runner, "step_views", False)      # the logits are consumed before the next step
        logits = self.runner.step(entries, copy_logits=False) if views else self.runner.step(entries)
        self.stats["steps"] += 1
        self.stats["tokens"] += plan.num_tokens
        for rid in plan.decode:
            r = self._requests[rid]
            r.computed += 1
            r.pending = None
        for rid, n in plan.prefill:
            self._requests[rid].computed += n
        if samplers:
            greedy_ids = getattr(self.runner, "last_greedy_ids", None) if views else None
            if greedy_ids is not None and all(r.sampler.params.greedy and not r.sampler.params.has_penalties for r in samplers):
                ids = greedy_ids                              # the captured step has taken the argmax already
            else:
                ids = self.sampler.sample(logits, [r.sampler for r in samplers], [r.history() for r in samplers])
            ids = ids.tolist() if hasattr(ids, "tolist") else list(ids)
            for r, tok in zip(samplers, ids):
                self._accept(r, int(tok))
        for rid in list(self._running):
            r = self._requests[rid]
            if r.state == DONE:
                self._running.remove(rid)
                self.runner.release(rid)
                finished.append(self._result(self._requests.pop(rid)))
        return finished

    def _accept(self, r: _Request, tok: int) -> None:
        """A sampled token: EOS ends the request and is not emitted (scheduler.cpp:149-156); else it
        is emitted and becomes the next token to feed unless a limit is reached."""
        p = r.params
        if not p.ignore_eos and tok in self.eos:
            r.hit_eos = True
            return self._finish(r, "eos")
        if tok in p.stop_token_ids:
            return self._finish(r, "stop")
        r.generated.append(tok)
        if r.on_token:
            r.on_token(r.id, tok)
        if len(r.generated) >= p.max_new_tokens:
            return self._finish(r, "max_new_tokens")
        if r.n_prompt + len(r.generated) >= self.runner.max_model_len:
            return self._finish(r, "length")
        r.pending = tok

    def _finish(self, r: _Request, reason: str) -> None:
        r.state = DONE
        r.finish_reason = reason
        if r.id not in self._running and r.id in self._requests and reason == "length":
            self.runner.release(r.id)

    def _result(self, r: _Request) -> RequestResult:
        return RequestResult(r.id, list(r.generated), r.n_prompt, hit_eos=r.hit_eos,
                             finish_reason=r.finish_reason, preemptions=r.preemptions)

    def run_to_completion(self) -> List[RequestResult]:
        out: List[RequestResult] = []
        while not self.idle():
            out.extend(self.step())
        return out
