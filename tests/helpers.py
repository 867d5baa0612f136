"""Tiny configurations, model folders and comparison helpers shared by the tests."""
from __future__ import annotations

import json
import tempfile
from pathlib import Path

import numpy as np
import torch

import plain_llama as plain
from qorvix_b200 import LlamaConfig
from qorvix_b200.config import RopeScaling
from qorvix_b200.weights import random_tensors, write_safetensors

ARCH = "LlamaForCausalLM"

# Tiny configurations that differ in every size and option.
TINY_A = LlamaConfig(architecture=ARCH, vocab_size=256, hidden_size=64, intermediate_size=172,
                     num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, head_dim=16,
                     max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0,
                     tie_word_embeddings=False)
TINY_B = LlamaConfig(architecture=ARCH, vocab_size=384, hidden_size=192, intermediate_size=512,
                     num_hidden_layers=3, num_attention_heads=6, num_key_value_heads=2, head_dim=32,
                     max_position_embeddings=256, rms_norm_eps=1e-6, rope_theta=500000.0,
                     rope_scaling=RopeScaling("llama3", 8.0, 1.0, 4.0, 64), tie_word_embeddings=True)
# head_dim 48 (a step of 16 that is no power of two), one kv head, odd vocabulary and widths
TINY_C = LlamaConfig(architecture=ARCH, vocab_size=331, hidden_size=144, intermediate_size=200,
                     num_hidden_layers=4, num_attention_heads=5, num_key_value_heads=1, head_dim=48,
                     max_position_embeddings=512, rms_norm_eps=3e-6, rope_theta=25000.0,
                     rope_scaling=RopeScaling("llama3", 4.0, 1.0, 2.0, 128), tie_word_embeddings=False)
# head sizes 64 and 128: the sizes the tcgen05 attention kernel, the tiled mma.sync kernel and the
# projection with rotation and cache write in its epilogue are written for
TINY_D = LlamaConfig(architecture=ARCH, vocab_size=410, hidden_size=256, intermediate_size=512,
                     num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                     max_position_embeddings=640, rms_norm_eps=2e-6, rope_theta=300000.0,
                     rope_scaling=RopeScaling("llama3", 16.0, 1.0, 4.0, 96), tie_word_embeddings=True)
TINY_E = LlamaConfig(architecture=ARCH, vocab_size=275, hidden_size=512, intermediate_size=1024,
                     num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1, head_dim=128,
                     max_position_embeddings=768, rms_norm_eps=1e-5, rope_theta=40000.0,
                     tie_word_embeddings=False)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}

FP32_TOL = 1e-4       # of max |logit|, float32 engine against the float64 plain implementation
BF16_TOL = 2e-2       # of max |logit|, bfloat16 engine against the same
# Models with sharpened attention have scores of magnitude ~8; rounding q and k to bfloat16
# (3 significant digits) then moves probabilities by several percent.  That is the price of the
# storage type, not a fault, so those models get a wider bound in bfloat16 (never in float32).
# A wrong, missing or stale key in such a model moves logits by tens of percent.
BF16_TOL_SHARP = 1e-1


def make_model_dir(cfg, seed: int, sharpen: float = 1.0, root=None) -> Path:
    """A model folder with random bfloat16 weights.  sharpen > 1 multiplies the q and k
    projections so that attention is peaked: a wrong, missing or stale key then changes the
    logits visibly instead of drowning among near-equal weights."""
    d = Path(tempfile.mkdtemp(prefix="qv_model_", dir=root))
    (d / "config.json").write_text(json.dumps(cfg.to_dict()))

    def tensors():
        for name, t in random_tensors(cfg, seed, "cpu", torch.bfloat16):
            if sharpen != 1.0 and (".q_proj." in name or ".k_proj." in name):
                t = (t.float() * sharpen).to(torch.bfloat16)
            yield name, t

    write_safetensors(d / "model.safetensors", tensors())
    return d


def random_tokens(vocab: int, n: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return [int(t) for t in torch.randint(0, vocab, (n,), generator=g)]


class PlainModel:
    """The plain implementation on a model folder, with a cache of whole-sequence logits."""

    def __init__(self, model_dir):
        self.cfg, self.weights = plain.read_model_dir(model_dir)
        self._memo = {}

    def logits(self, tokens) -> torch.Tensor:
        key = tuple(tokens)
        if key not in self._memo:
            self._memo[key] = plain.forward(self.cfg, self.weights, list(tokens))
        return self._memo[key]

    def greedy(self, prompt, n):
        return plain.generate_greedy(self.cfg, self.weights, list(prompt), n)


def tol_of(dtype: str, sharp: bool = False) -> float:
    if dtype == "float32":
        return FP32_TOL
    return BF16_TOL_SHARP if sharp else BF16_TOL


def assert_close_logits(got: torch.Tensor, ref: torch.Tensor, dtype: str, what: str = "", sharp: bool = False):
    """max |got - ref| <= tol * max |ref|; on failure names the first wrong row."""
    got = got.detach().double().cpu()
    ref = ref.double()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    scale = float(ref.abs().max())
    err = (got - ref).abs().amax(dim=-1)
    bad = torch.nonzero(err > tol_of(dtype, sharp) * scale)
    if bad.numel():
        first = int(bad[0])
        raise AssertionError(f"{what}: {bad.numel()} of {err.numel()} rows off; first wrong row {first} "
                             f"(err {float(err[first]):.3e}, allowed {tol_of(dtype, sharp) * scale:.3e}, max err {float(err.max()):.3e})")


class CallCounter:
    """Counts how often kernels of qorvix_b200.csrc.ops served, so that a test can prove its route:
    the successful calls of the Python functions of those names, plus what the native step executor
    (which launches the same kernels itself) counted since this object was made.
        counts = CallCounter(monkeypatch, "attention_prefill_tc"); ...; counts["attention_prefill_tc"]"""

    def __init__(self, monkeypatch, *names):
        from qorvix_b200.csrc import ops
        from qorvix_b200.engine import native_executor
        self._native = native_executor
        self._calls = {n: 0 for n in names}
        self._base = native_executor.route_counts()
        for n in names:
            monkeypatch.setattr(ops, n, self._wrap(n, getattr(ops, n)))

    def _wrap(self, name, fn):
        def counted(*a, **kw):
            res = fn(*a, **kw)
            if res is None or res:
                self._calls[name] += 1
            return res
        return counted

    @property
    def counts(self):
        now = self._native.route_counts()
        return {n: c + now.get(n, 0) - self._base.get(n, 0) for n, c in self._calls.items()}

    def __getitem__(self, name):
        return self.counts[name]


def assert_greedy_follows_plain(pm, prompt, got, what: str = "", gap: float = 0.05, at_least: int = 1) -> int:
    """`got` must be the plain implementation's greedy tokens, token for token, up to the first place
    where the plain top-2 gap is under `gap` of max |logit| (a near tie that rounding may decide
    either way; nothing after it is compared).  Returns how many tokens were compared and raises when
    fewer than `at_least` were."""
    seq = list(prompt)
    compared = 0
    for i, tok in enumerate(got):
        full = pm.logits(seq)[-1]
        top = torch.topk(full, 2)
        if float(top.values[0] - top.values[1]) < gap * float(full.abs().max()):
            break
        want = int(top.indices[0])
        assert int(tok) == want, f"{what}: generated token {i} is {tok}, the plain implementation's is {want} (so far {list(got[:i])})"
        seq.append(int(tok))
        compared += 1
    assert compared >= at_least, f"{what}: only {compared} tokens could be compared before a near tie; pick another prompt"
    return compared
