"""The plain implementation against the reference's own CPU TextModel (stored logits)."""
import importlib.util
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_llama as plain

GOLDEN = Path(__file__).resolve().parent / "golden"
_spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)


@pytest.mark.parametrize("name", ["golden_a", "golden_b"])
def test_plain_matches_reference_textmodel(name):
    m = make_golden.MODELS[name]
    stored = np.load(GOLDEN / f"{name}.npz")
    tokens = [int(t) for t in stored["tokens"]]
    assert tokens == make_golden.golden_tokens(m)
    weights = {k: torch.from_numpy(v) for k, v in make_golden.golden_weights(m).items()}
    logits = plain.forward(make_golden.golden_config(m), weights, tokens).numpy()
    ref = stored["logits"].astype(np.float64)
    scale = np.abs(ref).max()
    assert np.abs(logits - ref).max() <= 2e-5 * scale
    assert (logits.argmax(-1) == ref.argmax(-1)).all()


def test_rope_closed_forms():
    # identity at position 0, one radian at position 1 for the first pair, norm kept
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]], dtype=torch.float64)
    f = plain.plain_inv_freq(4, 10000.0)
    assert torch.equal(plain.rope(x, torch.tensor([0]), f), x)
    y = plain.rope(x, torch.tensor([1]), f)
    assert abs(float(y[0, 0, 0]) - (1.0 * np.cos(1.0) - 3.0 * np.sin(1.0))) < 1e-12
    assert abs(float(y.norm()) - float(x.norm())) < 1e-12


def test_llama3_scaling_regimes():
    base, hd = 500000.0, 32
    f = plain.plain_inv_freq(hd, base)
    same = plain.llama3_inv_freq(hd, base, 1.0, 1.0, 4.0, 64)
    assert torch.allclose(same, f, rtol=0, atol=0)
    g = plain.llama3_inv_freq(hd, base, 8.0, 1.0, 4.0, 64)
    wl = 2 * np.pi / f.numpy()
    hi, lo = 64 / 4.0, 64 / 1.0
    assert (wl < hi).any() and (wl > lo).any() and ((wl >= hi) & (wl <= lo)).any()
    for i in range(hd // 2):
        if wl[i] < hi:
            assert g[i] == f[i]
        elif wl[i] > lo:
            assert abs(float(g[i]) - float(f[i]) / 8.0) < 1e-18
        else:
            assert float(f[i]) / 8.0 <= float(g[i]) <= float(f[i])


def test_rmsnorm_softmax_silu_closed_forms():
    x = torch.tensor([3.0, 4.0], dtype=torch.float64)
    out = plain.rmsnorm(x, torch.ones(2, dtype=torch.float64), 0.0)
    assert torch.allclose(out, x / np.sqrt(12.5))
    s = plain.softmax(torch.tensor([1000.0, 1000.0], dtype=torch.float64))
    assert torch.allclose(s, torch.tensor([0.5, 0.5], dtype=torch.float64))
    assert abs(float(plain.silu(torch.tensor(1.0, dtype=torch.float64))) - 0.7310585786300049) < 1e-12


def test_attention_zero_qk_is_running_mean_of_v():
    T, H, hd = 5, 2, 4
    v = torch.randn(T, 1, hd, dtype=torch.float64)
    out = plain.attention(torch.zeros(T, H, hd, dtype=torch.float64),
                          torch.zeros(T, 1, hd, dtype=torch.float64), v)
    for t in range(T):
        assert torch.allclose(out[t, 0], v[: t + 1, 0].mean(0))
    w = plain.attention(torch.zeros(T, H, hd, dtype=torch.float64),
                        torch.zeros(T, 1, hd, dtype=torch.float64), v, window=2)
    assert torch.allclose(w[4, 1], v[3:5, 0].mean(0))


def test_sampler_filters():
    logits = np.array([0.0, 3.0, 1.0, 2.0], dtype=np.float32)
    ids, _ = plain.candidate_set(logits, 1.0, top_k=2)
    assert list(ids) == [1, 3]
    ids, _ = plain.candidate_set(logits, 1.0, top_p=0.6)
    assert list(ids) == [1]
    ids, _ = plain.candidate_set(logits, 1.0, min_p=0.3)
    assert list(ids) == [1, 3]
    assert plain.sample_with_uniform(logits, 0.999, 1.0, top_k=1) == 1
    pen = plain.apply_penalties(logits, [1, 1], repetition_penalty=2.0, frequency_penalty=0.5)
    assert abs(pen[1] - (3.0 / 2.0 - 1.0)) < 1e-6


def test_llama3_scaling_is_one_continuous_rule_and_both_implementations_state_it_alike():
    """The llama3 rule has no counterpart in the reference, so nothing of the reference can pin it.
    Two things do: its defining properties (the blend meets the kept range at wavelength orig/high
    and the divided range at orig/low, so the scaled frequencies are continuous and decreasing in
    i; factor 1 changes nothing), and two statements of it written apart (the loop of the plain
    implementation and the vectorised one of the engine's rotary part) agreeing at the parameter
    sets of the configurations the benchmark names."""
    from qorvix_b200.config import RopeScaling
    from qorvix_b200.parts.rotary import inverse_frequencies
    sets = [(128, 500000.0, 8.0, 1.0, 4.0, 8192), (64, 500000.0, 32.0, 1.0, 4.0, 8192), (32, 500000.0, 8.0, 1.0, 4.0, 64),
            (48, 25000.0, 4.0, 1.0, 2.0, 128), (64, 300000.0, 16.0, 1.0, 4.0, 96), (96, 10000.0, 3.0, 0.5, 8.0, 1000)]
    for hd, base, factor, low, high, orig in sets:
        a = plain.llama3_inv_freq(hd, base, factor, low, high, orig)
        b = inverse_frequencies(hd, base, RopeScaling("llama3", factor, low, high, orig))
        assert torch.allclose(a, b.double(), rtol=1e-14, atol=0), (hd, base, factor)
        assert bool((a[1:] < a[:-1]).all()), "scaled frequencies decrease with i"
        f = plain.plain_inv_freq(hd, base)
        assert bool((a <= f * (1 + 1e-15)).all()) and bool((a >= f / factor * (1 - 1e-15)).all())
    # continuity at the two edges: a frequency a hair inside the blend equals the neighbouring regime's value
    orig, low, high, factor = 8192.0, 1.0, 4.0, 8.0
    for wavelen, want in ((orig / high, 1.0), (orig / low, 1.0 / factor)):
        fi = 2 * np.pi / wavelen
        s = (orig / wavelen - low) / (high - low)
        blended = (1.0 - s) * fi / factor + s * fi
        assert abs(blended / fi - want) < 1e-12
