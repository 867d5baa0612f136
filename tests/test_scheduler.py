"""The scheduler's decisions (no GPU): a fake step function on top of the real cache manager."""
import pytest
import torch

from qorvix_b200.cache import CacheManager, PagedKVSpec
from qorvix_b200.engine.scheduler import Scheduler, SchedulerConfig
from qorvix_b200.sampling import SamplingParams

VOCAB = 50


class FakeRunner:
    """Keeps the real page bookkeeping; its 'logits' make the next token (last token + 1) % VOCAB,
    so generated tokens are a function of the sequence alone."""

    def __init__(self, tokens=256, max_requests=4, max_model_len=200):
        self.cache = CacheManager([(PagedKVSpec(1, 16), None)], max_tokens=tokens, page_size=16,
                                  max_requests=max_requests, device="cpu", allocate=False)
        self.max_model_len = max_model_len
        self.vocab_size = VOCAB
        self.batches = []

    def step(self, entries, end=()):
        rows = []
        self.batches.append([(e.req_id, len(e.tokens), self.cache.length(e.req_id) if self.cache.has(e.req_id) else 0)
                             for e in entries])
        for e in entries:
            if not self.cache.has(e.req_id):
                self.cache.admit(e.req_id)
            assert self.cache.reserve(e.req_id, len(e.tokens)), "the scheduler planned a step that does not fit"
            self.cache.commit(e.req_id, len(e.tokens))
            for w in e.want:
                row = torch.zeros(VOCAB)
                row[(e.tokens[w] + 1) % VOCAB] = 1.0
                rows.append(row)
        self.cache.check_invariants()
        return torch.stack(rows) if rows else None

    def release(self, rid):
        if self.cache.has(rid):
            self.cache.release(rid)


class ArgmaxSampler:
    def sample(self, logits, states, histories):
        return logits.argmax(-1).tolist()


def greedy(n, **kw):
    return SamplingParams.greedy_params(max_new_tokens=n, **kw)


def expect(prompt, n):
    out, t = [], prompt[-1]
    for _ in range(n):
        t = (t + 1) % VOCAB
        out.append(t)
    return out


def sched(runner, **cfg):
    return Scheduler(runner, ArgmaxSampler(), SchedulerConfig(**cfg), eos_token_ids=cfg.pop("eos", ()) if "eos" in cfg else ())


def test_two_requests_run_to_completion():
    r = FakeRunner()
    s = sched(r)
    a = s.submit([1, 2, 3], greedy(5))
    b = s.submit([7], greedy(3))
    res = {x.id: x for x in s.run_to_completion()}
    assert res[a].tokens == expect([1, 2, 3], 5) and res[b].tokens == expect([7], 3)
    assert res[a].finish_reason == "max_new_tokens" and res[a].prompt_tokens == 3
    assert r.cache.free_pages() == 16 and r.cache.free_slots() == 4 and s.idle()


def test_five_requests_through_two_slots_and_priority_order():
    r = FakeRunner()
    s = sched(r, max_concurrent=2)
    ids = [s.submit([i + 1], greedy(2), priority=p) for i, p in enumerate([0, 0, 5, 0, 1])]
    order = []
    while not s.idle():
        plan_before = s.active()
        s.step()
        assert s.active() <= 2
    first_steps = [rid for batch in r.batches for rid, _, at in batch if at == 0]
    assert first_steps == [ids[2], ids[4], ids[0], ids[1], ids[3]]       # priority first, then arrival


def test_token_budget_cuts_prompts_into_portions_beside_decodes():
    r = FakeRunner(tokens=512, max_model_len=400)
    s = sched(r, max_batch_tokens=32, max_concurrent=4)
    a = s.submit(list(range(1, 11)), greedy(40))
    s.step()                                            # a: whole prompt (10 tokens)
    b = s.submit([3] * 100, greedy(2))
    s.step()
    assert r.batches[-1] == [(a, 1, 10), (b, 31, 0)]    # decode first, the rest of the budget to b's prompt
    s.step()
    assert r.batches[-1] == [(a, 1, 11), (b, 31, 31)]
    while not s.idle():
        s.step()
        assert sum(n for _, n, _ in r.batches[-1]) <= 32
    portions = [n for batch in r.batches for rid, n, _ in batch if rid == b and n > 1]
    assert sum(portions) == 100


def test_max_chunk_limits_a_portion():
    r = FakeRunner(tokens=512, max_model_len=400)
    s = sched(r, max_batch_tokens=64, max_chunk=24)
    s.submit([2] * 50, greedy(1))
    s.run_to_completion()
    assert [n for batch in r.batches for _, n, _ in batch] == [24, 24, 2]


def test_eos_stop_and_length_finishes():
    r = FakeRunner(max_model_len=12)
    s = Scheduler(r, ArgmaxSampler(), SchedulerConfig(), eos_token_ids=[9])
    a = s.submit([5], greedy(20))                       # 6 7 8 then 9 = eos, not emitted
    b = s.submit([5], greedy(20, ignore_eos=True))      # runs into the sequence limit
    c = s.submit([20], greedy(20, stop_token_ids=(23,)))
    d = s.submit([], greedy(3))
    e = s.submit([1] * 12, greedy(3))
    res = {x.id: x for x in s.run_to_completion()}
    assert res[a].tokens == [6, 7, 8] and res[a].hit_eos and res[a].finish_reason == "eos"
    assert res[b].finish_reason == "length" and len(res[b].tokens) == 11 and not res[b].hit_eos
    assert res[c].tokens == [21, 22] and res[c].finish_reason == "stop"
    assert res[d].rejected and res[e].rejected


def test_waiting_request_stays_queued_until_pages_are_free():
    r = FakeRunner(tokens=64)                           # 4 pages
    s = sched(r)
    a = s.submit([1] * 40, greedy(8))                   # 3 pages
    b = s.submit([2] * 30, greedy(2))                   # 2 pages: does not fit beside a
    s.step()
    assert s.active() == 1 and s.waiting() == 1
    res = {x.id: x for x in s.run_to_completion()}
    assert not res[b].rejected and res[b].tokens == expect([2], 2) and res[b].preemptions == 0
    assert res[a].tokens == expect([1], 8)


def test_out_of_pages_preempts_the_youngest_and_recomputes():
    r = FakeRunner(tokens=64)                           # 4 pages of 16
    s = sched(r)
    a = s.submit([1] * 15, greedy(40))                  # grows to 55 tokens: 4 pages on its own
    b = s.submit([2] * 15, greedy(40))
    res = {x.id: x for x in s.run_to_completion()}
    assert s.stats["preemptions"] >= 1
    assert res[b].preemptions >= 1 and res[a].preemptions == 0       # the youngest gives way
    assert res[a].tokens == expect([1], 40) and res[b].tokens == expect([2], 40)
    assert r.cache.free_pages() == 4
    # after preemption b re-enters with prompt + generated tokens as its prompt
    refill = [n for batch in r.batches for rid, n, at in batch if rid == b and at == 0]
    assert len(refill) >= 2 and refill[-1] > 15


def test_a_lone_request_that_cannot_fit_finishes_with_length():
    r = FakeRunner(tokens=32, max_model_len=200)        # 2 pages
    s = sched(r)
    a = s.submit([1] * 10, greedy(100))
    res = s.run_to_completion()
    assert res[0].finish_reason == "length" and 20 <= len(res[0].tokens) <= 23
    assert r.cache.free_pages() == 2
    b = s.submit([1] * 40, greedy(2))                   # the prompt alone is larger than the pool
    res = s.run_to_completion()
    assert res[0].finish_reason == "length" and res[0].tokens == []


def test_streaming_callback_sees_every_token_in_order():
    r = FakeRunner()
    s = sched(r)
    seen = []
    a = s.submit([4], greedy(4), on_token=lambda rid, tok: seen.append((rid, tok)))
    s.run_to_completion()
    assert seen == [(a, t) for t in expect([4], 4)]


class LookaheadRunner(FakeRunner):
    """A fake runner that can be fed the ids of the step before as a tensor, like the real one."""
    step_views = True
    use_graphs = True
    max_graph_batch = 64

    def __init__(self, **kw):
        super().__init__(**kw)
        self.last_greedy_ids = None
        self.fed_from_device = 0

    def step(self, entries, end=(), copy_logits=True, device_tokens=None):
        if device_tokens is not None:
            self.fed_from_device += 1
            fed = [int(t) for t in device_tokens[: len(entries)]]
            entries = [type(e)(e.req_id, [fed[i]], e.want) for i, e in enumerate(entries)]
        logits = super().step(entries, end)
        decode_only = all(len(e.tokens) == 1 and len(e.want) == 1 for e in entries)
        self.last_greedy_ids = logits.argmax(-1).to(torch.int32) if (logits is not None and decode_only) else None
        return logits


@pytest.mark.parametrize("eos", [(), (9, 23, 31)])
def test_lookahead_gives_the_same_results_as_one_round_at_a_time(eos):
    """Requests that end by length, by a stop token and by end of sequence at different times:
    launching a round before the ids of the one before are read changes nothing in what comes out,
    gives every page back, and is what runs while all requests decode."""
    prompts = [[1, 2, 3], [7], [20, 21, 22, 23, 24, 25], [40, 41], [5] * 30]
    params = [greedy(12), greedy(30), greedy(25, stop_token_ids=(45,)), greedy(3), greedy(40)]
    results = {}
    for look in (False, True):
        r = LookaheadRunner(tokens=512, max_requests=4)
        s = Scheduler(r, ArgmaxSampler(), SchedulerConfig(max_concurrent=4, lookahead=look), eos_token_ids=eos)
        ids = [s.submit(p, sp) for p, sp in zip(prompts, params)]
        got = {x.id: x for x in s.run_to_completion()}
        results[look] = [(got[i].tokens, got[i].finish_reason, got[i].hit_eos) for i in ids]
        r.cache.check_invariants()
        assert r.cache.free_pages() == r.cache.num_pages and r.cache.free_slots() == 4
        if look:
            assert r.fed_from_device > (10 if not eos else 0) and s.stats["ahead_steps"] == r.fed_from_device
        else:
            assert r.fed_from_device == 0
    assert results[True] == results[False]
