"""The fused decode kernel (all layers of a decode step in one launch) against the plain
implementation, and against the parts' own path, which it must match beyond rounding."""
import pytest
import torch

from helpers import TINY, PlainModel, assert_close_logits, make_model_dir, random_tokens
from qorvix_b200 import ModelRunner, StepEntry
from qorvix_b200.csrc import ops

pytestmark = pytest.mark.gpu

# B: 3 layers, 6 heads on 2 kv heads, head size 32, interleaved feed-forward, llama3 rope scaling;
# C: 4 layers, 5 heads on 1 kv head, head size 48, a feed-forward width that is no multiple of 16.
CASES = [("B", 1.0), ("C", 1.0), ("B", 8.0)]


@pytest.fixture(scope="module")
def models():
    out = {}
    for name, sharpen in CASES:
        d = make_model_dir(TINY[name], seed=21 + len(out), sharpen=sharpen)
        out[(name, sharpen)] = (d, PlainModel(d))
    return out


def _decode(model_dir, toks, head, fused, monkeypatch, max_requests=4):
    monkeypatch.setenv("QORVIX_FUSED_DECODE", "1" if fused else "0")
    r = ModelRunner(model_dir, dtype="bfloat16", max_tokens=sum(len(t) for t in toks) + 64 * len(toks), page_size=16, max_requests=max_requests)
    r.step([StepEntry(i, t[:head], []) for i, t in enumerate(toks)])
    rows = []
    for j in range(head, min(len(t) for t in toks)):
        rows.append(r.step([StepEntry(i, [t[j]], [0]) for i, t in enumerate(toks)]))
    ops.check_kernel_errors()
    plan = r.decode_graph(len(toks)).ctx.fused
    return torch.stack(rows, 1), plan                    # [requests, steps, vocab]


@pytest.mark.parametrize("case", CASES)
def test_fused_decode_matches_plain_and_parts(models, case, monkeypatch):
    d, pm = models[case]
    cfg = TINY[case[0]]
    toks = [random_tokens(cfg.vocab_size, 90 + 7 * i, 30 + i) for i in range(3)]
    head = 37                                             # decoding crosses page edges (pages of 16)
    fused, plan = _decode(d, toks, head, True, monkeypatch)
    assert plan is not None, "the model is one the fused kernel takes"
    parts, none = _decode(d, toks, head, False, monkeypatch)
    assert none is None
    for i, t in enumerate(toks):
        ref = pm.logits(t)[head:90]
        assert_close_logits(fused[i], ref, "bfloat16", f"fused, request {i}", sharp=case[1] > 1)
        assert_close_logits(parts[i], ref, "bfloat16", f"parts, request {i}", sharp=case[1] > 1)


def test_fused_decode_single_request_and_long_context(models, monkeypatch):
    d, pm = models[("C", 1.0)]
    cfg = TINY["C"]
    toks = [random_tokens(cfg.vocab_size, 300, 5)]
    out, plan = _decode(d, toks, 250, True, monkeypatch, max_requests=1)
    assert plan is not None
    assert_close_logits(out[0], pm.logits(toks[0])[250:], "bfloat16", "fused, one request at positions 250..299")
