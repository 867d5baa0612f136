"""The engine against the plain implementation under every way of cutting and batching."""
import pytest
import torch

from helpers import TINY, PlainModel, assert_close_logits, make_model_dir, random_tokens
from qorvix_b200 import LlamaConfig, ModelRunner, StepEntry

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
CASES = [("A", 1.0), ("B", 1.0), ("C", 1.0), ("B", 8.0), ("A", 12.0)]


@pytest.fixture(scope="module")
def models():
    out = {}
    for name, sharpen in CASES:
        d = make_model_dir(TINY[name], seed=7 + len(out), sharpen=sharpen)
        out[(name, sharpen)] = (d, PlainModel(d))
    return out


def _runner(model_dir, dtype, max_tokens, **kw):
    return ModelRunner(model_dir, dtype=dtype, max_tokens=max_tokens, page_size=16, max_requests=4, **kw)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_whole_requests(models, case, dtype):
    d, pm = models[case]
    cfg = TINY[case[0]]
    r = _runner(d, dtype, 128)
    for n, seed in ((1, 1), (2, 2), (3, 3), (17, 4), (64, 5), (100, 6)):
        toks = random_tokens(cfg.vocab_size, n, seed)
        out = r.step([StepEntry("w", toks, list(range(n)))], end=["w"])
        assert_close_logits(out, pm.logits(toks), dtype, f"whole n={n}", sharp=case[1] > 1)
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_prefill_then_decode_last_32(models, case, dtype):
    d, pm = models[case]
    cfg = TINY[case[0]]
    n = 100
    toks = random_tokens(cfg.vocab_size, n, 11)
    ref = pm.logits(toks)
    r = _runner(d, dtype, 128)
    head = n - 32
    outs = [r.step([StepEntry("p", toks[:head], list(range(head)))])]
    for i in range(head, n):
        outs.append(r.step([StepEntry("p", [toks[i]], [0])]))
    r.step([], end=["p"])
    assert_close_logits(torch.cat(outs), ref, dtype, "prefill + 32 decoded", sharp=case[1] > 1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_portions_of_changing_size(models, case, dtype):
    d, pm = models[case]
    cfg = TINY[case[0]]
    toks = random_tokens(cfg.vocab_size, 111, 12)
    ref = pm.logits(toks)
    r = _runner(d, dtype, 128)
    outs, i = [], 0
    for n in (7, 2, 19, 3, 2, 16, 1, 31, 2, 17, 11):
        outs.append(r.step([StepEntry("c", toks[i:i + n], list(range(n)))]))
        i += n
    assert i == 111
    r.step([], end=["c"])
    assert_close_logits(torch.cat(outs), ref, dtype, "portions", sharp=case[1] > 1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_mixed_batches_with_page_reuse(models, case, dtype):
    """Up to four live requests, portions of some beside decoded tokens of others, in a pool
    so small (256 tokens) that pages of finished requests are handed to later ones."""
    d, pm = models[case]
    cfg = TINY[case[0]]
    lengths = [70, 45, 100, 33, 90, 64, 21, 58]
    reqs = {f"r{i}": random_tokens(cfg.vocab_size, n, 100 + i) for i, n in enumerate(lengths)}
    r = _runner(d, dtype, 256)
    cursor = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    waiting = list(reqs)
    live = []
    portion_sizes = [13, 2, 24, 5, 16, 3, 30, 7]
    step = 0
    pages_seen = set()
    reused = False
    while waiting or live:
        while waiting and len(live) < 4:
            need = -(-len(reqs[waiting[0]]) // 64) * 64
            held = sum(-(-len(reqs[k]) // 64) * 64 for k in live)
            if held + need > 256:
                break
            live.append(waiting.pop(0))
        entries, ends = [], []
        for j, k in enumerate(live):
            toks, c = reqs[k], cursor[k]
            prefill_len = len(toks) - 12           # the last 12 tokens are fed one by one
            if c < prefill_len:
                n = min(portion_sizes[(step + j) % len(portion_sizes)], prefill_len - c)
            else:
                n = 1
            if (step + j) % 5 == 4 and len(live) > 1:
                continue                           # this request sits the step out
            entries.append(StepEntry(k, toks[c:c + n], list(range(n))))
        if not entries:
            step += 1
            continue
        for e in entries:
            if cursor[e.req_id] + len(e.tokens) == len(reqs[e.req_id]):
                ends.append(e.req_id)
        out = r.step(entries, end=[])
        for e in entries:
            if cursor[e.req_id] == 0 and pages_seen & set(r.cache.block_table(e.req_id, 0)):
                reused = True
        row = 0
        for e in entries:
            n = len(e.tokens)
            got[e.req_id].append(out[row:row + n])
            row += n
            cursor[e.req_id] += n
        for k in ends:
            pages_seen.update(r.cache.block_table(k, 0))
            r.release(k)
            live.remove(k)
        r.cache.check_invariants()
        step += 1
    assert reused, "the pool was meant to be small enough for pages to be used again"
    assert r.cache.free_pages() == 256 // 16
    for k, toks in reqs.items():
        assert_close_logits(torch.cat(got[k]), pm.logits(toks), dtype, f"mixed {k}", sharp=case[1] > 1)


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(models, dtype):
    d, pm = models[("B", 8.0)]
    cfg = TINY["B"]
    toks = random_tokens(cfg.vocab_size, 250, 21)
    ref = pm.logits(toks)
    r = _runner(d, dtype, 256)
    outs = [r.step([StepEntry("l", toks[:5], list(range(5)))])]
    for i in range(5, 250):
        outs.append(r.step([StepEntry("l", [toks[i]], [0])]))
    assert_close_logits(torch.cat(outs), ref, dtype, "long decoding", sharp=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_want_subset_and_order(models, dtype):
    d, pm = models[("A", 12.0)]
    cfg = TINY["A"]
    a = random_tokens(cfg.vocab_size, 20, 31)
    b = random_tokens(cfg.vocab_size, 9, 32)
    r = _runner(d, dtype, 128)
    out = r.step([StepEntry("a", a, [19, 0, 7]), StepEntry("b", b, []), StepEntry("c", b[:4], [3])])
    ref = torch.stack([pm.logits(a)[19], pm.logits(a)[0], pm.logits(a)[7], pm.logits(b[:4])[3]])
    assert_close_logits(out, ref, dtype, "wanted rows", sharp=True)
    assert r.step([StepEntry("b", [b[0]], [])]) is None


def test_float32_is_bitwise_stable_across_cuts(models):
    """The 32-bit path accumulates every output in an order fixed by its position alone."""
    d, _ = models[("B", 8.0)]
    cfg = TINY["B"]
    toks = random_tokens(cfg.vocab_size, 80, 41)
    r = _runner(d, "float32", 256)
    whole = r.step([StepEntry("x", toks, list(range(80)))], end=["x"])
    outs, i = [], 0
    other = random_tokens(cfg.vocab_size, 30, 42)
    r.step([StepEntry("o", other[:10], [])])
    for n in (5, 2, 33, 1, 1, 38):
        res = r.step([StepEntry("o", [other[10 + len(outs)]], [0]), StepEntry("y", toks[i:i + n], list(range(n)))])
        outs.append(res[1:])
        i += n
    assert torch.equal(torch.cat(outs), whole)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", [("B", 8.0), ("C", 1.0)])
def test_decoded_tokens_before_a_portion(models, case, dtype):
    """Five requests bring one decoded token each, a sixth a prompt portion, in one step: the step
    is served by the single-token kernel and the portion kernel together."""
    d, pm = models[case]
    cfg = TINY[case[0]]
    r = ModelRunner(d, dtype=dtype, max_tokens=1024, page_size=16, max_requests=8)
    dec = {f"d{i}": random_tokens(cfg.vocab_size, 20 + 7 * i, 200 + i) for i in range(5)}
    long = random_tokens(cfg.vocab_size, 90, 300)
    for k, t in dec.items():
        r.step([StepEntry(k, t[:-2], [])])
    r.step([StepEntry("p", long[:40], [])])
    outs = {k: [] for k in dec}
    got_p = []
    for stepi, (a, b) in enumerate(((40, 73), (73, 90))):
        entries = [StepEntry(k, [t[len(t) - 2 + stepi]], [0]) for k, t in dec.items()] + [StepEntry("p", long[a:b], list(range(b - a)))]
        out = r.step(entries)
        for i, k in enumerate(dec):
            outs[k].append(out[i:i + 1])
        got_p.append(out[5:])
    for k, t in dec.items():
        assert_close_logits(torch.cat(outs[k]), pm.logits(t)[-2:], dtype, f"decoded {k}", sharp=case[1] > 1)
    assert_close_logits(torch.cat(got_p), pm.logits(long)[40:], dtype, "portion beside decoded tokens", sharp=case[1] > 1)


@pytest.mark.parametrize("dtype", DTYPES)
def test_logits_keep_the_callers_order_when_portions_come_before_decoded_tokens(models, dtype):
    """Entries in the order portion, token, portion, token, token, token, each with wanted places:
    the engine runs the single tokens first, the logits come back in the order given."""
    d, pm = models[("B", 8.0)]
    cfg = TINY["B"]
    r = ModelRunner(d, dtype=dtype, max_tokens=1024, page_size=16, max_requests=8)
    dec = {f"d{i}": random_tokens(cfg.vocab_size, 18 + 5 * i, 400 + i) for i in range(4)}
    p1, p2 = random_tokens(cfg.vocab_size, 50, 410), random_tokens(cfg.vocab_size, 37, 411)
    for k, t in dec.items():
        r.step([StepEntry(k, t[:-1], [])])
    r.step([StepEntry("p1", p1[:12], [])])
    names = list(dec)
    entries = [StepEntry("p1", p1[12:], [0, 37, 5]), StepEntry(names[0], [dec[names[0]][-1]], [0]),
               StepEntry("p2", p2, [36]), StepEntry(names[1], [dec[names[1]][-1]], [0]),
               StepEntry(names[2], [dec[names[2]][-1]], []), StepEntry(names[3], [dec[names[3]][-1]], [0])]
    out = r.step(entries)
    assert out.shape[0] == 7
    ref = torch.cat([pm.logits(p1)[[12, 49, 17]], pm.logits(dec[names[0]])[-1:], pm.logits(p2)[-1:],
                     pm.logits(dec[names[1]])[-1:], pm.logits(dec[names[3]])[-1:]])
    assert_close_logits(out, ref, dtype, "caller's order", sharp=True)
    r.cache.check_invariants()


def test_norms_folded_into_the_products_around_them(monkeypatch):
    """Steps of up to 64 tokens in bfloat16 at sizes where the few-token products are split along K:
    the output projections add into the residual stream and prepare the next norm's input, the
    projections after the norm scale their sums.  Against the plain implementation, and against the
    same engine with the norm kernel (QORVIX_FOLDED_NORM=0)."""
    cfg = LlamaConfig(architecture="LlamaForCausalLM", vocab_size=300, hidden_size=512, intermediate_size=1024, num_hidden_layers=3, num_attention_heads=4,
                      num_key_value_heads=2, head_dim=128, max_position_embeddings=256, rms_norm_eps=1e-5, rope_theta=10000.0,
                      rope_scaling=None, tie_word_embeddings=False)
    d = make_model_dir(cfg, seed=21, sharpen=4.0)
    pm = PlainModel(d)
    a, b = random_tokens(300, 60, 31), random_tokens(300, 41, 32)
    ref_a, ref_b = pm.logits(a), pm.logits(b)
    results = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("QORVIX_FOLDED_NORM", mode)
        r = ModelRunner(d, dtype="bfloat16", max_tokens=512, page_size=16, max_requests=4)
        got_a = [r.step([StepEntry("a", a[:33], list(range(33)))])]                       # a portion of few tokens
        out = r.step([StepEntry("a", a[33:50], list(range(17))), StepEntry("b", b[:30], list(range(30)))])
        got_a.append(out[:17]); got_b = [out[17:]]
        for i in range(10):                                                               # captured decode steps
            out = r.step([StepEntry("a", [a[50 + i]], [0]), StepEntry("b", [b[30 + i]], [0])])
            got_a.append(out[:1]); got_b.append(out[1:])
        got_b.append(r.step([StepEntry("b", [b[40]], [0])]))
        results[mode] = (torch.cat(got_a), torch.cat(got_b))
        assert_close_logits(results[mode][0], ref_a, "bfloat16", f"request a, folded norms {mode}", sharp=True)
        assert_close_logits(results[mode][1], ref_b, "bfloat16", f"request b, folded norms {mode}", sharp=True)
    # the two routes round differently, so they are close to each other but not equal: both ran
    assert not torch.equal(results["1"][0], results["0"][0])


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_layer_of_llama31_8b_sizes(dtype):
    """The real sizes (hidden 4096, 32 heads over 8 kv heads of 128, feed-forward 14336, vocabulary
    128256, llama3 scaling from 8192) on one layer: whole, in portions and token by token, against
    the plain implementation (run in float64 on the GPU, or it would take minutes)."""
    import plain_llama as plain
    from qorvix_b200 import LlamaConfig
    from qorvix_b200.config import RopeScaling
    from qorvix_b200.weights import random_tensors
    cfg = LlamaConfig(architecture="LlamaForCausalLM", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                      num_hidden_layers=1, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                      max_position_embeddings=8192, rms_norm_eps=1e-5, rope_theta=500000.0,
                      rope_scaling=RopeScaling("llama3", 8.0, 1.0, 4.0, 8192), tie_word_embeddings=False)
    # N(0, 0.02) weights at this width already give scores with a standard deviation of about 1.6,
    # so keys matter without any sharpening
    tensors = dict(random_tensors(cfg, 3, "cuda", torch.bfloat16))
    toks = random_tokens(cfg.vocab_size, 200, 77)
    ref = plain.forward(cfg.to_dict() | {"rope_scaling": cfg.rope_scaling.to_dict()}, tensors, toks).cpu()
    r = ModelRunner(config=cfg, tensors=tensors, dtype=dtype, max_tokens=512, max_requests=2)
    whole = r.step([StepEntry("w", toks, list(range(200)))], end=["w"])
    assert_close_logits(whole, ref, dtype, "8B-size layer, whole")
    outs = [r.step([StepEntry("p", toks[:130], list(range(130)))]), r.step([StepEntry("p", toks[130:190], list(range(60)))])]
    for i in range(190, 200):
        outs.append(r.step([StepEntry("p", [toks[i]], [0])]))
    assert_close_logits(torch.cat(outs), ref, dtype, "8B-size layer, portions and decoding")
