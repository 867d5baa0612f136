"""Generation through the Python entry point, the scheduler on the real engine, the command
line and bin/trace_run."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import TINY, PlainModel, assert_close_logits, assert_greedy_follows_plain, make_model_dir, random_tokens
from qorvix_b200 import LLM, SamplingParams

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def model_b():
    d = make_model_dir(TINY["B"], seed=3, sharpen=6.0)
    return d, PlainModel(d)


@pytest.fixture(scope="module")
def model_a():
    d = make_model_dir(TINY["A"], seed=4, sharpen=10.0)
    return d, PlainModel(d)


def test_greedy_generation_matches_plain_float32(model_b, model_a):
    for (d, pm), name in ((model_b, "B"), (model_a, "A")):
        llm = LLM(d, dtype="float32", max_tokens=512, max_concurrent=4, max_batch_tokens=48)
        prompts = [random_tokens(TINY[name].vocab_size, n, 60 + n) for n in (1, 5, 33, 70)]
        res = llm.generate(prompts, SamplingParams.greedy_params(max_new_tokens=12))
        for p, r in zip(prompts, res):
            assert r.tokens == pm.greedy(p, 12) and r.finish_reason == "max_new_tokens"
        assert llm.runner.cache.free_pages() == 512 // 16


@pytest.mark.parametrize("name,seed,sharpen,prompts", [("E", 5, 6.0, ((70, 1),)), ("C", 6, 6.0, ((70, 3), (9, 3)))])
def test_greedy_generation_bfloat16_follows_plain(name, seed, sharpen, prompts):
    """Untied models whose greedy continuations wander over the vocabulary (a constant continuation
    could not tell a cache that works from one that is ignored): the bfloat16 engine's tokens equal the
    plain implementation's, token for token, up to the first place where the plain top-2 gap is under
    5 % of the largest logit; the prompts are chosen so that at least five tokens come before it."""
    cfg = TINY[name]
    d = make_model_dir(cfg, seed=seed, sharpen=sharpen)
    pm = PlainModel(d)
    llm = LLM(d, dtype="bfloat16", max_tokens=512, max_concurrent=4)
    ps = [random_tokens(cfg.vocab_size, n, sd) for n, sd in prompts]
    res = llm.generate(ps, SamplingParams.greedy_params(max_new_tokens=10))
    for p, r in zip(ps, res):
        assert len(r.tokens) == 10
        assert len(set(pm.greedy(p, 10))) >= 4
        assert_greedy_follows_plain(pm, p, r.tokens, f"{name} prompt of {len(p)}", at_least=5)


def test_preemption_recomputes_to_the_same_tokens(model_b):
    d, pm = model_b
    prompts = [random_tokens(TINY["B"].vocab_size, 20, 90 + i) for i in range(3)]
    roomy = LLM(d, dtype="float32", max_tokens=1024, max_concurrent=3)
    want = [r.tokens for r in roomy.generate(prompts, SamplingParams.greedy_params(max_new_tokens=40))]
    tight = LLM(d, dtype="float32", max_tokens=128, max_concurrent=3)       # 8 pages for 3 x 60 tokens
    res = tight.generate(prompts, SamplingParams.greedy_params(max_new_tokens=40))
    assert tight.last_stats["preemptions"] >= 1
    assert [r.tokens for r in res] == want
    assert want[0] == pm.greedy(prompts[0], 40)
    assert tight.runner.cache.free_pages() == 8


def test_sampling_is_reproducible_and_independent_of_the_batch(model_b):
    d, _ = model_b
    llm = LLM(d, dtype="float32", max_tokens=512, max_concurrent=4)
    p1, p2 = random_tokens(384, 12, 1), random_tokens(384, 30, 2)
    sp = SamplingParams(temperature=0.9, top_k=20, top_p=0.9, min_p=0.02, seed=7, max_new_tokens=16)
    alone = llm.generate([p1], sp)[0].tokens
    again = llm.generate([p1], sp)[0].tokens
    both = llm.generate([p2, p1], [SamplingParams(seed=9, max_new_tokens=5), sp])[1].tokens
    other = llm.generate([p1], SamplingParams(temperature=0.9, top_k=20, top_p=0.9, min_p=0.02, seed=8, max_new_tokens=16))[0].tokens
    assert alone == again == both and len(alone) == 16
    assert other != alone


def test_eos_from_config_stops_generation(model_a):
    d, pm = model_a
    prompt = random_tokens(256, 10, 5)
    free_run = pm.greedy(prompt, 8)
    eos = free_run[3]
    llm = LLM(d, dtype="float32", max_tokens=256)
    llm.eos_token_ids = (eos,)
    r = llm.generate([prompt], SamplingParams.greedy_params(max_new_tokens=8))[0]
    cut = free_run.index(eos)
    assert r.tokens == free_run[:cut] and r.hit_eos and r.finish_reason == "eos"


def _run_trace(model_dir, dtype, steps, out_dir, max_tokens):
    env = dict(os.environ)
    p = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype, "--out", str(out_dir),
                        "--max-tokens", str(max_tokens)], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, env=env, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    return p.stdout.split("\n")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(model_b, tmp_path, dtype):
    d, pm = model_b
    a, b = random_tokens(384, 70, 11), random_tokens(384, 40, 12)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:50], "want": [0, 49]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[50:52], "want": []}, {"id": "b", "tokens": b[:33], "want": [32]}], "end": []},
        {"step": 2, "entries": [{"id": "b", "tokens": b[33:], "want": [6]}], "end": ["b"]},
        {"step": 3, "entries": [{"id": "a", "tokens": a[52:], "want": list(range(18))}], "end": ["a"]},
        {"step": 4, "entries": [{"id": "c", "tokens": b, "want": [39]}], "end": ["c"]},
    ]
    lines = _run_trace(d, dtype, steps, tmp_path, 128)
    assert [l for l in lines if l.startswith("done")] == [f"done {i}" for i in range(5)]
    V = 384
    get = lambda i: torch.from_numpy(np.fromfile(tmp_path / f"{i}.f32", dtype="<f4").reshape(-1, V))
    assert_close_logits(get(0), pm.logits(a)[[0, 49]], dtype, "step 0", sharp=True)
    assert_close_logits(get(1), pm.logits(b)[[32]], dtype, "step 1", sharp=True)
    assert_close_logits(get(2), pm.logits(b)[[39]], dtype, "step 2", sharp=True)
    assert_close_logits(get(3), pm.logits(a)[52:], dtype, "step 3", sharp=True)
    assert_close_logits(get(4), pm.logits(b)[[39]], dtype, "step 4", sharp=True)


def _four_mode_trace(reqs, pool):
    """Steps for bin/trace_run: every request (1) alone and whole, (2) most of it in one step and the
    last 32 tokens one by one, (3) in portions of changing size down to two tokens, (4) mixed, up to
    four live at a time, portions of some beside decoded tokens of others, admitted only while the
    live requests (each rounded up to 64 tokens) fit the pool, so that pages are used again.
    Returns (steps, [(step number, request, first position, count)]) with all logits wanted."""
    steps, where = [], []

    def add(entries, end):
        n = len(steps)
        steps.append({"step": n, "entries": [{"id": k, "tokens": reqs[k][a:a + c], "want": list(range(c))} for k, a, c in entries],
                      "end": list(end)})
        where.extend((n, k, a, c) for k, a, c in entries)

    for k, t in reqs.items():                                             # 1
        add([(k, 0, len(t))], [k])
    for k, t in reqs.items():                                             # 2
        head = max(1, len(t) - 32)
        add([(k, 0, head)], [])
        for i in range(head, len(t)):
            add([(k, i, 1)], [k] if i == len(t) - 1 else [])
    sizes = (7, 2, 19, 3, 2, 70, 1, 31, 2, 17, 66, 11)
    for k, t in reqs.items():                                             # 3
        i = j = 0
        while i < len(t):
            c = min(sizes[j % len(sizes)], len(t) - i)
            add([(k, i, c)], [k] if i + c == len(t) else [])
            i += c; j += 1
    waiting, live, cursor, j = list(reqs), [], {k: 0 for k in reqs}, 0    # 4
    rounded = lambda k: -(-len(reqs[k]) // 64) * 64
    while waiting or live:
        while waiting and len(live) < 4 and sum(map(rounded, live)) + rounded(waiting[0]) <= pool:
            live.append(waiting.pop(0))
        entries = []
        for x, k in enumerate(live):
            left = len(reqs[k]) - cursor[k]
            c = 1 if left <= 10 else min((13, 2, 70, 5, 36, 3)[(j + x) % 6], left - 10)
            if (j + x) % 5 == 4 and len(live) > 1:
                continue                                                  # sits this step out
            entries.append((k, cursor[k], c))
        j += 1
        if not entries:
            continue
        done = [k for k, a, c in entries if a + c == len(reqs[k])]
        add(entries, done)
        for k, a, c in entries:
            cursor[k] += c
        live = [k for k in live if k not in done]
    return steps, where


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program_in_all_four_modes(tmp_path, dtype):
    """The four ways of cutting, through the program itself (one process, the pool so small that
    pages are used again), at head size 64, against the plain implementation."""
    cfg = TINY["D"]
    d = make_model_dir(cfg, seed=17, sharpen=8.0)
    pm = PlainModel(d)
    reqs = {f"r{i}": random_tokens(cfg.vocab_size, n, 700 + i) for i, n in enumerate((170, 45, 120, 33, 90, 64))}
    steps, where = _four_mode_trace(reqs, 448)
    assert max(len(s["entries"]) for s in steps) == 4
    lines = _run_trace(d, dtype, steps, tmp_path, 448)
    assert [l for l in lines if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    V = cfg.vocab_size
    by_step = {}
    for n, k, a, c in where:
        by_step.setdefault(n, []).append((k, a, c))
    for n, parts in by_step.items():
        got = torch.from_numpy(np.fromfile(tmp_path / f"{n}.f32", dtype="<f4").reshape(-1, V))
        ref = torch.cat([pm.logits(reqs[k])[a:a + c] for k, a, c in parts])
        assert_close_logits(got, ref, dtype, f"step {n} {parts}", sharp=True)


def test_command_line_generate_and_info(model_a):
    d, pm = model_a
    prompt = random_tokens(256, 6, 8)
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "qorvix"), "generate", str(d), "--tokens", ",".join(map(str, prompt)),
                        "--max", "5", "--temp", "0", "--dtype", "float32"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = p.stdout.strip().split("\n")
    assert [int(t) for t in lines[1].split()] == pm.greedy(prompt, 5)
    assert "6 prompt tokens, 5 generated" in p.stdout
    q = subprocess.run([sys.executable, str(ROOT / "bin" / "qorvix"), "model-info", str(d)], capture_output=True, text=True, timeout=120)
    assert json.loads(q.stdout)["hidden_size"] == 64


def test_lookahead_gives_the_same_tokens_as_one_step_at_a_time():
    """With lookahead the scheduler launches a decode step before it has read the ids of the one in
    flight; requests that end on a stop token, on max_new_tokens or on the sequence limit at different
    times, greedy and sampled, must come out token for token as without it."""
    cfg = TINY["B"]
    d = make_model_dir(cfg, seed=91)
    prompts = [random_tokens(cfg.vocab_size, n, 200 + n) for n in (5, 23, 40, 64, 9, 31)]
    params = [SamplingParams.greedy_params(max_new_tokens=60),
              SamplingParams.greedy_params(max_new_tokens=17),
              SamplingParams(temperature=0.9, top_k=20, top_p=0.9, seed=4, max_new_tokens=45, repetition_penalty=1.0),
              SamplingParams(temperature=1.3, seed=5, max_new_tokens=33, repetition_penalty=1.0,
                             stop_token_ids=tuple(range(0, cfg.vocab_size, 7))),
              SamplingParams.greedy_params(max_new_tokens=80, stop_token_ids=tuple(range(3, cfg.vocab_size, 11))),
              SamplingParams(temperature=0.7, min_p=0.05, seed=6, max_new_tokens=70, repetition_penalty=1.0)]
    out = {}
    for look in (False, True):
        llm = LLM(d, dtype="bfloat16", max_tokens=2048, max_concurrent=4, lookahead=look, max_model_len=120)
        res = llm.generate(prompts, params)
        out[look] = [(r.tokens, r.finish_reason) for r in res]
        llm.runner.cache.check_invariants()
        assert llm.runner.cache.free_pages() == llm.runner.cache.num_pages
        if look:
            assert llm.last_stats["ahead_steps"] > 10, "the lookahead path did run"
    assert out[True] == out[False]
    assert {r for _, r in out[True]} >= {"max_new_tokens", "stop"}


def test_gpu_check_compares_with_the_cpp_model_and_fails_when_both_engine_paths_share_a_fault(model_b, monkeypatch, capsys):
    """`qorvix gpu-check` holds both engine paths against the plain C++ decoder; an error common to
    the float32 and the bfloat16 path (here: every RMS norm built with another eps) must not pass."""
    from qorvix_b200.cli.main import cmd_gpu_check
    from qorvix_b200.parts import rmsnorm
    d, _ = model_b
    assert cmd_gpu_check(["gpu-check", str(d), "--random-prompt", "40"]) == 0
    assert "PASS" in capsys.readouterr().out
    real_init = rmsnorm.RMSNorm.__init__

    def wrong_eps(self, spec, source, rt):
        real_init(self, spec, source, rt)
        self.eps = 0.5

    monkeypatch.setattr(rmsnorm.RMSNorm, "__init__", wrong_eps)
    assert cmd_gpu_check(["gpu-check", str(d), "--random-prompt", "40"]) == 1
    assert "FAIL" in capsys.readouterr().out
