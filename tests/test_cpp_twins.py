"""The plain C++ twins of the kernels (qorvix_b200/csrc/ref/): pinned to the reference's own CPU model
through the stored logits of tests/golden/, and operation by operation to the plain Python
implementation.  Host only."""
import importlib.util
import json
import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_llama as plain
from helpers import TINY, make_model_dir, random_tokens
from qorvix_b200.csrc import ref
from qorvix_b200.weights import write_safetensors

GOLDEN = Path(__file__).resolve().parent / "golden"
_spec = importlib.util.spec_from_file_location("make_golden", GOLDEN / "make_golden.py")
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)


@pytest.mark.parametrize("name", ["golden_a", "golden_b"])
def test_cpp_model_matches_the_reference_textmodel(name, tmp_path):
    m = make_golden.MODELS[name]
    stored = np.load(GOLDEN / f"{name}.npz")
    tokens = [int(t) for t in stored["tokens"]]
    (tmp_path / "config.json").write_text(json.dumps(make_golden.golden_config(m)))
    write_safetensors(tmp_path / "model.safetensors", ((k, torch.from_numpy(v)) for k, v in make_golden.golden_weights(m).items()))
    got = ref.RefModel(tmp_path).logits(tokens).astype(np.float64)
    want = stored["logits"].astype(np.float64)
    assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()
    assert (got.argmax(-1) == want.argmax(-1)).all()


@pytest.mark.parametrize("name", ["B", "D"])
def test_cpp_model_matches_the_plain_implementation_with_llama3_scaling_and_bfloat16_weights(name):
    cfg = TINY[name]
    d = make_model_dir(cfg, seed=31)
    toks = random_tokens(cfg.vocab_size, 40, 5)
    pc, pw = plain.read_model_dir(d)
    want = plain.forward(pc, pw, toks).numpy()
    got = ref.RefModel(d).logits(toks).astype(np.float64)
    assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()


def test_cpp_model_reports_everything_wrong_with_a_checkpoint_at_once(tmp_path):
    cfg = TINY["A"]
    d = make_model_dir(cfg, seed=1, root=tmp_path)
    _, w = plain.read_model_dir(d)
    w.pop("model.layers.0.mlp.up_proj.weight")
    w["surplus.weight"] = torch.zeros(3)
    w["model.norm.weight"] = torch.zeros(cfg.hidden_size + 1, dtype=torch.bfloat16)
    write_safetensors(d / "model.safetensors", w.items())
    with pytest.raises(ValueError) as e:
        ref.RefModel(d)
    msg = str(e.value)
    assert "missing tensors (1): model.layers.0.mlp.up_proj.weight" in msg and "unexpected tensors (1): surplus.weight" in msg
    assert "model.norm.weight: stored [65], expected [64]" in msg
    (d / "config.json").write_text(json.dumps(dict(cfg.to_dict(), architectures=["NoSuchLM"])))
    with pytest.raises(ValueError, match="not registered .known: LlamaForCausalLM"):
        ref.RefModel(d)


def test_cpp_operations_one_by_one():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(5, 48, generator=g, dtype=torch.float64)
    w = 1 + 0.1 * torch.randn(48, generator=g, dtype=torch.float64)
    assert np.allclose(ref.rmsnorm(x.numpy(), w.numpy(), 1e-5), plain.rmsnorm(x, w, 1e-5).numpy(), rtol=1e-6, atol=1e-6)
    W = torch.randn(33, 48, generator=g, dtype=torch.float64)
    assert np.allclose(ref.gemm(x.numpy(), W.numpy()), plain.linear(x, W).numpy(), rtol=1e-5, atol=1e-5)
    from qorvix_b200.config import RopeScaling
    for sc in (None, RopeScaling("llama3", 8.0, 1.0, 4.0, 64)):
        f = ref.inverse_frequencies(32, 5e5, sc)
        want = plain.plain_inv_freq(32, 5e5) if sc is None else plain.llama3_inv_freq(32, 5e5, 8.0, 1.0, 4.0, 64)
        assert np.allclose(f, want.numpy(), rtol=1e-13, atol=0)
        v = torch.randn(4, 3, 32, generator=g, dtype=torch.float64)
        pos = torch.tensor([0, 1, 17, 200])
        assert np.allclose(ref.rope(v.reshape(4, 96).numpy(), pos.numpy(), 3, 32, 32, f), plain.rope(v, pos, want).reshape(4, 96).numpy(),
                           rtol=1e-5, atol=1e-6)
    gte, up = torch.randn(70, generator=g, dtype=torch.float64), torch.randn(70, generator=g, dtype=torch.float64)
    assert np.allclose(ref.swiglu(gte.numpy(), up.numpy()), plain.swiglu(gte, up).numpy(), rtol=1e-6, atol=1e-6)
    assert ref.argmax(np.array([1.0, 5.0, 5.0, 2.0])) == 1                        # the first maximum wins


def test_cpp_paged_attention_matches_plain_attention_over_scattered_pages():
    g = torch.Generator().manual_seed(4)
    H, Hkv, hd, page = 6, 2, 16, 16
    lens = [(5, 37), (1, 20), (30, 30)]                       # (queries this step, tokens cached)
    n_blocks = [-(-c // page) for _, c in lens]
    perm = torch.randperm(sum(n_blocks) + 2, generator=g).tolist()
    bt = np.full((len(lens), max(n_blocks)), len(perm) - 1, dtype=np.int32)
    cache = np.zeros((len(perm), 2, Hkv, page, hd), dtype=np.float32)
    qs, refs, pos, seg = [], [], [], []
    for i, (ql, c) in enumerate(lens):
        pages = [perm.pop() for _ in range(n_blocks[i])]
        bt[i, :len(pages)] = pages
        k, v = torch.randn(c, Hkv, hd, generator=g, dtype=torch.float64), torch.randn(c, Hkv, hd, generator=g, dtype=torch.float64)
        q = torch.randn(c, H, hd, generator=g, dtype=torch.float64)
        for t in range(c):
            cache[pages[t // page], 0, :, t % page] = k[t].numpy()
            cache[pages[t // page], 1, :, t % page] = v[t].numpy()
        refs.append(plain.attention(q, k, v, window=11 if i == 2 else 0, rows=range(c - ql, c))[c - ql:].reshape(ql, H * hd))
        qs.append(q[c - ql:].reshape(ql, H * hd))
        pos += list(range(c - ql, c)); seg += [i] * ql
    q = torch.cat(qs).numpy()
    for window, rows in ((0, slice(0, 6)), (11, slice(6, 36))):
        out = ref.attention_paged(q, cache, pos, seg, bt, H, Hkv, hd, page, window, hd ** -0.5)
        assert np.allclose(out[rows], torch.cat(refs).numpy()[rows], rtol=1e-5, atol=1e-5)


def test_cpp_sampler_follows_the_reference_order_of_filters():
    logits = np.array([0.0, 3.0, 1.0, 2.0], dtype=np.float32)
    assert list(ref.candidates(logits, 1.0, top_k=2)[0]) == [1, 3]
    assert list(ref.candidates(logits, 1.0, top_p=0.6)[0]) == [1]
    assert list(ref.candidates(logits, 1.0, min_p=0.3)[0]) == [1, 3]
    rng = np.random.RandomState(5)
    for _ in range(20):
        l = rng.randn(300).astype(np.float32) * 2
        t, k, p, mp, u = float(rng.uniform(0.3, 1.5)), int(rng.choice([0, 5, 40])), float(rng.choice([1.0, 0.9, 0.5])), float(rng.choice([0.0, 0.05])), float(rng.uniform())
        ids, probs = ref.candidates(l, t, k, p, mp)
        pi, pp = plain.candidate_set(l, t, k, p, mp)
        assert list(ids) == list(pi) and np.allclose(probs, pp, rtol=1e-9)
        recent = [int(x) for x in rng.randint(0, 300, 9)]
        want = plain.sample_with_uniform(plain.apply_penalties(l, recent, 1.2, 0.3, 0.1), u, t, k, p, mp)
        assert ref.sample(l, u, t, k, p, mp, recent, 1.2, 0.3, 0.1) == want
    assert ref.sample(logits, 0.7, 0.0) == 1                                      # temperature 0: greedy
