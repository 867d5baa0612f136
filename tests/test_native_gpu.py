"""The native engine (csrc/host/: loader, cache, executor, scheduler, sampler) through its command
line: greedy generation against the plain implementation and the Python entry point, trace replay in
all four modes, its gpu-check; and the native step executor behind the Python step function against
the part-by-part path."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import TINY, PlainModel, assert_close_logits, make_model_dir, random_tokens
from qorvix_b200 import ModelRunner, StepEntry
from test_generate_gpu import _four_mode_trace

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
NATIVE = str(ROOT / "bin" / "qorvix-native")


def _run(*args, stdin=None, timeout=900):
    return subprocess.run([sys.executable, NATIVE, *args], input=stdin, capture_output=True, text=True, timeout=timeout)


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("E", "float32"), ("D", "float32")])
def test_native_generate_prints_the_plain_implementations_greedy_tokens(name, dtype):
    """--temp 0 is greedy after the penalties, as in the reference (runtime/src/sampler.cpp:43-50 applies
    the penalties, whose repetition penalty defaults to 1.1, before it looks at the temperature): the
    expected tokens are the plain implementation's logits through the plain penalties and argmax."""
    import plain_llama as plain
    cfg = TINY[name]
    d = make_model_dir(cfg, seed=4, sharpen=6.0)
    pm = PlainModel(d)
    prompt = random_tokens(cfg.vocab_size, 70, 8)
    want, seq = [], list(prompt)
    for _ in range(12):
        row = plain.apply_penalties(pm.logits(seq)[-1].numpy(), seq, repetition_penalty=1.1, penalty_last_n=64)
        want.append(int(np.argmax(row)))
        seq.append(want[-1])
    p = _run("generate", str(d), "--tokens", ",".join(map(str, prompt)), "--max", "12", "--temp", "0", "--dtype", dtype)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = p.stdout.strip().split("\n")
    assert [int(t) for t in lines[0].split()] == prompt
    assert [int(t) for t in lines[1].split()] == want
    assert "70 prompt tokens, 12 generated" in p.stdout
    # the Python command line prints the same tokens
    q = subprocess.run([sys.executable, str(ROOT / "bin" / "qorvix"), "generate", str(d), "--tokens", ",".join(map(str, prompt)), "--max", "12",
                        "--temp", "0", "--dtype", dtype], capture_output=True, text=True, timeout=600)
    assert q.stdout.strip().split("\n")[1].split() == lines[1].split()


def test_native_generate_samples_reproducibly_and_stops_at_eos():
    cfg = TINY["E"]
    d = make_model_dir(cfg, seed=4, sharpen=6.0)
    prompt = ",".join(map(str, random_tokens(cfg.vocab_size, 20, 3)))
    outs = [_run("generate", str(d), "--tokens", prompt, "--max", "16", "--seed", str(s)).stdout.strip().split("\n")[1].split() for s in (7, 7, 8)]
    assert outs[0] == outs[1] and len(outs[0]) == 16 and outs[0] != outs[2]
    # an end-of-sequence id from config.json ends the generation and is not printed
    greedy = _run("generate", str(d), "--tokens", prompt, "--max", "8", "--temp", "0").stdout.strip().split("\n")[1].split()
    conf = json.loads((d / "config.json").read_text())
    conf["eos_token_id"] = int(greedy[3])
    (d / "config.json").write_text(json.dumps(conf))
    p = _run("generate", str(d), "--tokens", prompt, "--max", "8", "--temp", "0")
    assert p.stdout.strip().split("\n")[1].split() == greedy[:greedy.index(greedy[3])] and ", eos]" in p.stdout


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_native_replay_in_all_four_modes(tmp_path, dtype):
    cfg = TINY["D"]
    d = make_model_dir(cfg, seed=17, sharpen=8.0)
    pm = PlainModel(d)
    reqs = {f"r{i}": random_tokens(cfg.vocab_size, n, 700 + i) for i, n in enumerate((170, 45, 120, 33, 90, 64))}
    steps, where = _four_mode_trace(reqs, 448)
    p = _run("replay", "--model", str(d), "--dtype", dtype, "--out", str(tmp_path), "--max-tokens", "448",
             stdin="\n".join(json.dumps(s) for s in steps) + "\n")
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(len(steps))]
    by_step = {}
    for n, k, a, c in where:
        by_step.setdefault(n, []).append((k, a, c))
    for n, parts in by_step.items():
        got = torch.from_numpy(np.fromfile(tmp_path / f"{n}.f32", dtype="<f4").reshape(-1, cfg.vocab_size))
        ref = torch.cat([pm.logits(reqs[k])[a:a + c] for k, a, c in parts])
        assert_close_logits(got, ref, dtype, f"step {n} {parts}", sharp=True)


def test_native_gpu_check_and_bench():
    d = make_model_dir(TINY["E"], seed=9, sharpen=4.0)
    p = _run("gpu-check", str(d), "--random-prompt", "48")
    assert p.returncode == 0 and "PASS" in p.stdout, p.stdout + p.stderr[-2000:]
    b = _run("bench", str(d), "--prompt", "40", "--gen", "24", "--batch", "3", "--runs", "2", "--json")
    assert b.returncode == 0, b.stderr[-2000:]
    res = json.loads(b.stdout)
    assert res["batch"] == 3 and res["decode_tok_per_sec"] > 0 and res["prefill_tok_per_sec"] > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "E"])
def test_native_executor_and_the_part_by_part_path_give_the_same_logits(name, dtype, monkeypatch):
    """The same steps (a whole prompt of more than 64 tokens, portions, mixed steps with decoded tokens
    first, captured decode steps) through the Python step function with the native executor and with
    the parts one by one: both against the plain implementation, float32 bit for bit alike."""
    cfg = TINY[name]
    d = make_model_dir(cfg, seed=23, sharpen=5.0)
    pm = PlainModel(d)
    a, b = random_tokens(cfg.vocab_size, 150, 1), random_tokens(cfg.vocab_size, 90, 2)
    results = {}
    for native in ("1", "0"):
        monkeypatch.setenv("QORVIX_NATIVE_EXECUTOR", native)
        r = ModelRunner(d, dtype=dtype, max_tokens=512, page_size=16, max_requests=8)
        outs_a = [r.step([StepEntry("a", a[:100], list(range(100)))])]
        used = bool(r.model._native)
        assert used == (native == "1")
        small = {f"s{i}": random_tokens(cfg.vocab_size, 9 + i, 30 + i) for i in range(4)}
        for k, t in small.items():
            r.step([StepEntry(k, t[:-1], [])])
        out = r.step([StepEntry(k, [t[-1]], [0]) for k, t in small.items()] + [StepEntry("a", a[100:140], list(range(40))), StepEntry("b", b[:70], list(range(70)))])
        outs_small = out[:4]; outs_a.append(out[4:44]); outs_b = [out[44:]]
        out = r.step([StepEntry("b", b[70:80], list(range(10))), StepEntry("a", a[140:142], [0, 1])])
        outs_b.append(out[:10]); outs_a.append(out[10:])
        for i in range(8):
            out = r.step([StepEntry("a", [a[142 + i]], [0]), StepEntry("b", [b[80 + i]], [0])])
            outs_a.append(out[:1]); outs_b.append(out[1:])
        got_a, got_b = torch.cat(outs_a), torch.cat(outs_b)
        assert_close_logits(got_a, pm.logits(a), dtype, f"a, native executor {native}", sharp=True)
        assert_close_logits(got_b, pm.logits(b)[:88], dtype, f"b, native executor {native}", sharp=True)
        for i, (k, t) in enumerate(small.items()):
            assert_close_logits(outs_small[i:i + 1], pm.logits(t)[-1:], dtype, f"{k}, native executor {native}", sharp=True)
        results[native] = (got_a, got_b)
        r.cache.check_invariants()
    if dtype == "float32":
        assert torch.equal(results["1"][0], results["0"][0]) and torch.equal(results["1"][1], results["0"][1])
