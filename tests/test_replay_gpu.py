"""The engine against the plain implementation under every way of cutting and batching."""
import pytest
import torch

from helpers import TINY, CallCounter, PlainModel, assert_close_logits, make_model_dir, random_tokens
from qorvix_b200 import LlamaConfig, ModelRunner, StepEntry

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
CASES = [("A", 1.0), ("B", 1.0), ("C", 1.0), ("B", 8.0), ("A", 12.0), ("D", 1.0), ("E", 1.0), ("D", 8.0), ("E", 6.0)]
ROUTES = ("attention_prefill_tc", "gemm_qkv_rope", "attention_decode_bf16", "attention_prefill_bf16", "attention_generic")


def _big(cfg) -> bool:
    """Head sizes 64 and 128: what the tcgen05 attention kernel and the projection with rotation and
    cache write in its epilogue take.  Tests of these configurations bring portions of more than 64
    tokens and assert that those kernels served them."""
    return cfg.head_dim in (64, 128)


def _assert_routes(cfg, dtype, counts, *names):
    if _big(cfg) and dtype == "bfloat16":
        for n in names:
            assert counts[n] > 0, f"{n} was meant to serve this test and never ran ({counts.counts})"


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
def test_whole_requests(models, case, dtype, monkeypatch):
    d, pm = models[case]
    cfg = TINY[case[0]]
    counts = CallCounter(monkeypatch, *ROUTES)
    r = _runner(d, dtype, 384)
    sizes = ((1, 1), (2, 2), (3, 3), (17, 4), (64, 5), (100, 6)) + (((65, 7), (129, 8), (300, 9)) if _big(cfg) else ())
    for n, seed in sizes:
        toks = random_tokens(cfg.vocab_size, n, seed)
        out = r.step([StepEntry("w", toks, list(range(n)))], end=["w"])
        assert_close_logits(out, pm.logits(toks), dtype, f"whole n={n}", sharp=case[1] > 1)
    r.cache.check_invariants()
    _assert_routes(cfg, dtype, counts, "attention_prefill_tc", "gemm_qkv_rope")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_prefill_then_decode_last_32(models, case, dtype, monkeypatch):
    d, pm = models[case]
    cfg = TINY[case[0]]
    counts = CallCounter(monkeypatch, *ROUTES)
    n = 230 if _big(cfg) else 100
    toks = random_tokens(cfg.vocab_size, n, 11)
    ref = pm.logits(toks)
    r = _runner(d, dtype, 256)
    head = n - 32
    outs = [r.step([StepEntry("p", toks[:head], list(range(head)))])]
    for i in range(head, n):
        outs.append(r.step([StepEntry("p", [toks[i]], [0])]))
    r.step([], end=["p"])
    assert_close_logits(torch.cat(outs), ref, dtype, "prefill + 32 decoded", sharp=case[1] > 1)
    _assert_routes(cfg, dtype, counts, "attention_prefill_tc", "gemm_qkv_rope", "attention_decode_bf16")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_portions_of_changing_size(models, case, dtype, monkeypatch):
    d, pm = models[case]
    cfg = TINY[case[0]]
    counts = CallCounter(monkeypatch, *ROUTES)
    # head sizes 64/128: portions of 65 to 130 tokens too, so that steps of more than 64 tokens (the
    # many-token products, rotation in the projection's epilogue, tcgen05 attention over earlier pages) are cut as well
    sizes = (7, 2, 19, 3, 2, 16, 1, 31, 2, 17, 11) + ((70, 3, 130, 2, 65, 33, 97, 2) if _big(cfg) else ())
    total = sum(sizes)
    toks = random_tokens(cfg.vocab_size, total, 12)
    ref = pm.logits(toks)
    r = _runner(d, dtype, 64 * -(-total // 64))
    outs, i = [], 0
    for n in sizes:
        outs.append(r.step([StepEntry("c", toks[i:i + n], list(range(n)))]))
        i += n
    assert i == total
    r.step([], end=["c"])
    assert_close_logits(torch.cat(outs), ref, dtype, "portions", sharp=case[1] > 1)
    _assert_routes(cfg, dtype, counts, "attention_prefill_tc", "gemm_qkv_rope", "attention_prefill_bf16")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", CASES)
def test_mixed_batches_with_page_reuse(models, case, dtype, monkeypatch):
    """Up to four live requests, portions of some beside decoded tokens of others, in a pool
    so small (256 tokens) that pages of finished requests are handed to later ones."""
    d, pm = models[case]
    cfg = TINY[case[0]]
    counts = CallCounter(monkeypatch, *ROUTES)
    big = _big(cfg)
    lengths = [170, 45, 200, 33, 190, 64, 121, 158] if big else [70, 45, 100, 33, 90, 64, 21, 58]
    pool = 640 if big else 256
    reqs = {f"r{i}": random_tokens(cfg.vocab_size, n, 100 + i) for i, n in enumerate(lengths)}
    r = _runner(d, dtype, pool)
    cursor = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    waiting = list(reqs)
    live = []
    portion_sizes = [13, 2, 70, 5, 36, 3, 90, 7] if big else [13, 2, 24, 5, 16, 3, 30, 7]
    step = 0
    pages_seen = set()
    reused = False
    while waiting or live:
        while waiting and len(live) < 4:
            need = -(-len(reqs[waiting[0]]) // 64) * 64
            held = sum(-(-len(reqs[k]) // 64) * 64 for k in live)
            if held + need > pool:
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
    assert r.cache.free_pages() == pool // 16
    for k, toks in reqs.items():
        assert_close_logits(torch.cat(got[k]), pm.logits(toks), dtype, f"mixed {k}", sharp=case[1] > 1)
    _assert_routes(cfg, dtype, counts, "attention_prefill_tc", "gemm_qkv_rope", "attention_decode_bf16")


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


def test_float32_is_bitwise_stable_in_captured_decode_steps(models):
    """Decode-only steps of 1, 3 and 5 requests run as replayed graphs of 1, 4 and 8 rows, the rows
    beyond the live requests being padding that reads the scratch page: the logits of each request are
    bit for bit those of the same request run whole, whatever stands beside it and in whichever row."""
    d, _ = models[("B", 8.0)]
    cfg = TINY["B"]
    r = ModelRunner(d, dtype="float32", max_tokens=1024, page_size=16, max_requests=8)
    reqs = {f"q{i}": random_tokens(cfg.vocab_size, 40 + 9 * i, 500 + i) for i in range(5)}
    whole = {k: r.step([StepEntry(k, t, list(range(len(t))))], end=[k]) for k, t in reqs.items()}
    tail = 12
    for k, t in reqs.items():
        r.step([StepEntry(k, t[:-tail], [])])
    got = {k: [] for k in reqs}
    names = list(reqs)
    j = 0
    while any(len(v) < tail for v in got.values()):
        # 1, 3 or 5 live rows in turn, those that are furthest behind first
        pending = sorted((k for k in names if len(got[k]) < tail), key=lambda k: (len(got[k]), k))
        batch = pending[: (1, 3, 5)[j % 3]]
        entries = [StepEntry(k, [reqs[k][len(reqs[k]) - tail + len(got[k])]], [0]) for k in batch]
        out = r.step(entries)
        for row, e in enumerate(entries):
            got[e.req_id].append(out[row:row + 1].clone())
        j += 1
    assert len(r._graphs) >= 3, "the decode-only steps were meant to run as captured graphs of several sizes"
    for k in names:
        assert torch.equal(torch.cat(got[k]), whole[k][-tail:]), f"request {k}: captured decode steps differ from the whole run"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", [("B", 8.0), ("C", 1.0), ("D", 8.0), ("E", 6.0), ("E", 1.0)])
def test_decoded_tokens_before_a_portion(models, case, dtype, monkeypatch):
    """Five requests bring one decoded token each, a sixth a prompt portion of 70 and then of 50
    tokens, in one step: the step is served by the single-token kernel and the portion kernel
    together, the latter from the segment arrays and block table cut after the decoded tokens (at
    head sizes 64/128 that is the tcgen05 kernel, and the step's projection rotates and writes the
    cache in its epilogue)."""
    d, pm = models[case]
    cfg = TINY[case[0]]
    r = ModelRunner(d, dtype=dtype, max_tokens=1024, page_size=16, max_requests=8)
    dec = {f"d{i}": random_tokens(cfg.vocab_size, 20 + 7 * i, 200 + i) for i in range(5)}
    long = random_tokens(cfg.vocab_size, 160, 300)
    for k, t in dec.items():
        r.step([StepEntry(k, t[:-2], [])])
    r.step([StepEntry("p", long[:40], [])])
    outs = {k: [] for k in dec}
    got_p = []
    counts = CallCounter(monkeypatch, *ROUTES)
    for stepi, (a, b) in enumerate(((40, 110), (110, 160))):
        before = dict(counts.counts)
        entries = [StepEntry(k, [t[len(t) - 2 + stepi]], [0]) for k, t in dec.items()] + [StepEntry("p", long[a:b], list(range(b - a)))]
        out = r.step(entries)
        if _big(cfg) and dtype == "bfloat16":
            layers = cfg.num_hidden_layers
            assert counts["attention_decode_bf16"] - before["attention_decode_bf16"] == layers, "decoded tokens go to the split-KV kernel"
            assert counts["attention_prefill_tc"] - before["attention_prefill_tc"] == layers, "the portion goes to the tcgen05 kernel"
            assert counts["attention_generic"] == 0
        for i, k in enumerate(dec):
            outs[k].append(out[i:i + 1])
        got_p.append(out[5:])
    for k, t in dec.items():
        assert_close_logits(torch.cat(outs[k]), pm.logits(t)[-2:], dtype, f"decoded {k}", sharp=case[1] > 1)
    assert_close_logits(torch.cat(got_p), pm.logits(long)[40:], dtype, "portion beside decoded tokens", sharp=case[1] > 1)
    _assert_routes(cfg, dtype, counts, "gemm_qkv_rope")


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


def _llama31_8b_one_layer():
    from qorvix_b200.config import RopeScaling
    return LlamaConfig(architecture="LlamaForCausalLM", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                       num_hidden_layers=1, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                       max_position_embeddings=8192, rms_norm_eps=1e-5, rope_theta=500000.0,
                       rope_scaling=RopeScaling("llama3", 8.0, 1.0, 4.0, 8192), tie_word_embeddings=False)


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_layer_of_llama31_8b_sizes(dtype):
    """The real sizes (hidden 4096, 32 heads over 8 kv heads of 128, feed-forward 14336, vocabulary
    128256, llama3 scaling from 8192) on one layer: whole, in portions and token by token, and with a
    second request beside it (its prompt portion beside the first one's decoded token, then both
    decoding), against the plain implementation (run in float64 on the GPU, or it would take minutes)."""
    import plain_llama as plain
    from qorvix_b200.weights import random_tensors
    cfg = _llama31_8b_one_layer()
    # N(0, 0.02) weights at this width already give scores with a standard deviation of about 1.6,
    # so keys matter without any sharpening
    tensors = dict(random_tensors(cfg, 3, "cuda", torch.bfloat16))
    cfgd = cfg.to_dict() | {"rope_scaling": cfg.rope_scaling.to_dict()}
    toks = random_tokens(cfg.vocab_size, 200, 77)
    ref = plain.forward(cfgd, tensors, toks).cpu()
    r = ModelRunner(config=cfg, tensors=tensors, dtype=dtype, max_tokens=1024, max_requests=4)
    whole = r.step([StepEntry("w", toks, list(range(200)))], end=["w"])
    assert_close_logits(whole, ref, dtype, "8B-size layer, whole")
    outs = [r.step([StepEntry("p", toks[:130], list(range(130)))]), r.step([StepEntry("p", toks[130:190], list(range(60)))])]
    for i in range(190, 196):
        outs.append(r.step([StepEntry("p", [toks[i]], [0])]))
    # mixed steps: a second and a third request come in beside the first one's decoded tokens
    other = random_tokens(cfg.vocab_size, 120, 78)
    third = random_tokens(cfg.vocab_size, 9, 79)
    ref_o = plain.forward(cfgd, tensors, other).cpu()
    ref_t = plain.forward(cfgd, tensors, third).cpu()
    out = r.step([StepEntry("q", other[:100], list(range(100))), StepEntry("p", [toks[196]], [0])])
    outs.append(out[100:]); got_o = [out[:100]]
    out = r.step([StepEntry("p", [toks[197]], [0]), StepEntry("q", other[100:118], list(range(18))), StepEntry("t", third[:8], list(range(8)))])
    outs.append(out[:1]); got_o.append(out[1:19]); got_t = [out[19:]]
    for i in range(2):                                           # all three decode together
        out = r.step([StepEntry("q", [other[118 + i]], [0]), StepEntry("p", [toks[198 + i]], [0])] + ([StepEntry("t", [third[8]], [0])] if i == 0 else []))
        got_o.append(out[:1]); outs.append(out[1:2])
        if i == 0:
            got_t.append(out[2:])
    assert_close_logits(torch.cat(outs), ref, dtype, "8B-size layer, portions, decoding and mixed steps")
    assert_close_logits(torch.cat(got_o), ref_o, dtype, "8B-size layer, second request")
    assert_close_logits(torch.cat(got_t), ref_t, dtype, "8B-size layer, third request")
    r.cache.check_invariants()


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_layer_of_llama31_8b_sizes_at_long_context(dtype):
    """The lengths the benchmark runs: a prompt of 8,100 tokens in portions of 2,048 (the first of them
    a whole 2,048-token prefill), then two decoded tokens at positions beyond 8,000, with logits at a
    few places of every step against the plain implementation in float64."""
    import plain_llama as plain
    from qorvix_b200.weights import random_tensors
    cfg = _llama31_8b_one_layer()
    tensors = dict(random_tensors(cfg, 4, "cuda", torch.bfloat16))
    cfgd = cfg.to_dict() | {"rope_scaling": cfg.rope_scaling.to_dict()}
    n = 8102
    toks = random_tokens(cfg.vocab_size, n, 91)
    r = ModelRunner(config=cfg, tensors=tensors, dtype=dtype, max_tokens=8192 + 64, max_requests=2)
    rows, outs = [], []
    for a in range(0, 8100, 2048):
        b = min(a + 2048, 8100)
        want = sorted({0, 1, (b - a) // 2, b - a - 17, b - a - 1})
        outs.append(r.step([StepEntry("L", toks[a:b], want)]))
        rows += [a + w for w in want]
    for i in (8100, 8101):
        outs.append(r.step([StepEntry("L", [toks[i]], [0])]))
        rows.append(i)
    ref = plain.forward(cfgd, tensors, toks, rows=rows).cpu()
    assert_close_logits(torch.cat(outs), ref, dtype, "8B-size layer, 8,100-token context")
