"""The native host code without a GPU: the command line's configuration reading and errors, and the
shape tables the benchmark's per-kernel figures rest on."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

from helpers import TINY, make_model_dir
from qorvix_b200 import LlamaConfig

ROOT = Path(__file__).resolve().parent.parent
NATIVE = str(ROOT / "bin" / "qorvix-native")


def _run(*args):
    return subprocess.run([sys.executable, NATIVE, *args], capture_output=True, text=True, timeout=600)


def test_native_model_info_reads_the_configuration_like_the_python_side():
    cfg = TINY["B"]
    d = make_model_dir(cfg, seed=2)
    p = _run("model-info", str(d))
    assert p.returncode == 0, p.stderr[-2000:]
    info = json.loads(p.stdout)
    q = subprocess.run([sys.executable, str(ROOT / "bin" / "qorvix"), "model-info", str(d)], capture_output=True, text=True, timeout=120)
    want = json.loads(q.stdout)
    for key in ("vocab_size", "hidden_size", "intermediate_size", "num_attention_heads", "num_key_value_heads", "head_dim", "parameters"):
        assert info[key] == want[key], key
    assert info["num_hidden_layers"] == cfg.num_hidden_layers and info["rope_scaling"] == "llama3" and info["tie_word_embeddings"] is True


def test_native_command_line_names_what_is_wrong_with_a_configuration(tmp_path):
    cfg = TINY["A"].to_dict()
    for change, message in ((dict(architectures=["MysteryLM"]), "architecture 'MysteryLM' is not registered (known: LlamaForCausalLM)"),
                            (dict(num_key_value_heads=3), "num_attention_heads 4 is not a multiple of num_key_value_heads 3"),
                            (dict(hidden_act="gelu"), "hidden_act 'gelu' is not supported"),
                            (dict(vocab_size=None), "required key 'vocab_size' is missing")):
        (tmp_path / "config.json").write_text(json.dumps({k: v for k, v in dict(cfg, **change).items() if v is not None or k != "vocab_size"}))
        p = _run("model-info", str(tmp_path))
        assert p.returncode == 1 and message in p.stderr, (p.stderr, message)
    assert _run().returncode == 1 and _run("--help").returncode == 0


def test_kernel_bench_takes_its_shapes_from_the_configuration():
    from qorvix_b200.kernel_bench import layer_products
    cfg = LlamaConfig.from_dict(dict(architectures=["LlamaForCausalLM"], vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                                     num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128))
    assert layer_products(cfg) == [("qkv", 6144, 4096, False), ("o", 4096, 4096, False), ("gate_up", 28672, 4096, True),
                                   ("down", 4096, 14336, False), ("lm_head", 128256, 4096, False)]


def test_native_scheduler_decisions_with_a_fake_engine(tmp_path):
    """tests/native/scheduler_test.cpp: the C++ scheduler (token budget, portions, priority, admission on
    whole-prompt pages, preemption by recompute, finishes, sampling rows) over the real page bookkeeping
    with a fake engine; compiled with the host compiler and run here."""
    from qorvix_b200.csrc.build import CSRC, find_host_compiler
    exe = tmp_path / "scheduler_test"
    cmd = [find_host_compiler(), "-O1", "-std=c++17", "-I", str(CSRC), "-o", str(exe), str(ROOT / "tests" / "native" / "scheduler_test.cpp"),
           str(CSRC / "host_runtime.cpp")]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert build.returncode == 0, build.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0 and run.stdout.strip() == "ok", run.stderr[-2000:]
