"""Each kernel alone against a plain PyTorch float32/float64 reference of the same op, at sizes
other than the tiny models': widths and vocabularies that are no power of two, head sizes in
steps of 16, odd numbers of heads and groups."""
import math

import numpy as np
import pytest
import torch

import plain_llama as plain
from qorvix_b200.csrc import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, seed=0, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(dtype):
    table = rnd(333, 72, seed=1, dtype=dtype)
    ids = torch.tensor([0, 332, 5, 5, 100], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, device=DEV)
    ops.embed(out, table, ids)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d", [72, 1000, 4096, 5120])
def test_add_rmsnorm(dtype, d):
    res = rnd(9, d, seed=2)
    delta = rnd(9, d, seed=3, dtype=dtype)
    w = rnd(d, seed=4) * 0.1 + 1.0
    ref_sum = res.double() + delta.double()
    ref = plain.rmsnorm(ref_sum, w.double(), 1e-6)
    out = torch.empty(9, d, device=DEV, dtype=dtype)
    r2 = res.clone()
    ops.add_rmsnorm(out, r2, delta, w, 1e-6)
    assert torch.allclose(r2.double(), ref_sum, rtol=1e-6, atol=1e-6)            # the sum is float32
    assert torch.allclose(out.double(), ref, **tol(dtype))
    # no delta: the residual stays as it is
    r3 = res.clone()
    ops.add_rmsnorm(out, r3, None, w, 1e-6)
    assert torch.equal(r3, res)
    assert torch.allclose(out.double(), plain.rmsnorm(res.double(), w.double(), 1e-6), **tol(dtype))
    # gathered rows: only those are normed, nothing is written back
    rows = torch.tensor([7, 0, 7], dtype=torch.int32, device=DEV)
    out3 = torch.empty(3, d, device=DEV, dtype=dtype)
    r4 = res.clone()
    ops.add_rmsnorm(out3, r4, delta, w, 1e-6, row_idx=rows)
    assert torch.equal(r4, res)
    assert torch.allclose(out3.double(), ref[rows.long()], **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(dtype):
    gu = rnd(7, 2 * 172, seed=5, dtype=dtype, scale=3.0)
    out = torch.empty(7, 172, device=DEV, dtype=dtype)
    ops.swiglu(out, gu)
    ref = plain.swiglu(gu[:, :172].double(), gu[:, 172:].double())
    assert torch.allclose(out.double(), ref, **tol(dtype))


@pytest.mark.parametrize("dt", [(torch.float32, torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16, torch.bfloat16),
                                (torch.bfloat16, torch.bfloat16, torch.float32), (torch.bfloat16, torch.float32, torch.bfloat16)])
@pytest.mark.parametrize("shape", [(1, 100, 72), (5, 331, 200), (70, 64, 172), (130, 257, 1000)])
def test_gemm_simt(dt, shape):
    M, N, K = shape
    a = rnd(M, K, seed=6, dtype=dt[0])
    w = rnd(N, K, seed=7, dtype=dt[1], scale=0.1)
    c = torch.empty(M, N, device=DEV, dtype=dt[2])
    ops.gemm_simt(c, a, w)
    ref = a.double() @ w.double().t()
    if dt[2] == torch.float32:
        assert torch.allclose(c.double(), ref, rtol=1e-5, atol=1e-5 * math.sqrt(K))
    else:
        assert torch.allclose(c.double(), ref, rtol=1e-2, atol=1e-2)
    if dt[2] == torch.float32:
        c2 = c.clone()
        ops.gemm_simt(c2, a, w, accumulate=True)
        assert torch.allclose(c2.double(), 2 * ref, rtol=1e-5, atol=2e-5 * math.sqrt(K))


def _paged_setup(dtype, T_ctx, H, Hkv, hd, page, seed, rot=None, n_pages=None, sharp=1.5):
    """One request of T_ctx tokens whose pages are scattered through the pool.  Inputs have
    standard deviation `sharp`: 1.5 gives scores of a few units, peaked enough to tell keys apart
    and small enough that float32 rounding of a score stays below the comparison's bound."""
    rot = hd if rot is None else rot
    n_blocks = -(-T_ctx // page)
    n_pages = n_pages or n_blocks + 5
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed))[:n_blocks]
    bt = perm.to(torch.int32).reshape(1, -1).to(DEV)
    qkv = rnd(T_ctx, (H + 2 * Hkv) * hd, seed=seed + 1, dtype=dtype, scale=sharp)
    cache = torch.zeros(n_pages, 2, Hkv, page, hd, device=DEV, dtype=dtype)
    pos = torch.arange(T_ctx, dtype=torch.int32, device=DEV)
    seg = torch.zeros(T_ctx, dtype=torch.int32, device=DEV)
    inv = plain.plain_inv_freq(rot, 10000.0) if rot else None
    table = None
    if rot:
        ang = torch.arange(T_ctx, dtype=torch.float64)[:, None] * inv[None, :]
        table = torch.stack([ang.cos(), ang.sin()], -1).float().contiguous().to(DEV)
    return qkv, cache, bt, pos, seg, table, inv


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,hd,rot,page", [(4, 4, 16, 16, 16), (6, 2, 48, 48, 16), (5, 1, 80, 32, 32), (8, 2, 128, 128, 64)])
def test_rope_kv_write(dtype, H, Hkv, hd, rot, page):
    T = 150
    qkv, cache, bt, pos, seg, table, inv = _paged_setup(dtype, T, H, Hkv, hd, page, seed=11, rot=rot)
    src = qkv.clone().double().cpu().reshape(T, H + 2 * Hkv, hd)
    ops.rope_kv_write(qkv, cache, table, pos, seg, bt, H, Hkv, hd, rot, page)
    ref_rot = plain.rope(src[:, : H + Hkv, :rot], torch.arange(T), inv)
    ref = src.clone()
    ref[:, : H + Hkv, :rot] = ref_rot
    got_q = qkv[:, : H * hd].double().cpu().reshape(T, H, hd)
    assert torch.allclose(got_q, ref[:, :H], **tol(dtype))
    btl = bt[0].tolist()
    for t in (0, 1, page - 1, page, T - 1):
        k = cache[btl[t // page], 0, :, t % page, :].double().cpu()
        v = cache[btl[t // page], 1, :, t % page, :].double().cpu()
        assert torch.allclose(k, ref[t, H:H + Hkv], **tol(dtype))
        assert torch.equal(v, src[t, H + Hkv:])
    # the untouched part of the qkv buffer (k, v) is as it was
    assert torch.equal(qkv[:, H * hd:].double().cpu().reshape(T, 2 * Hkv, hd), src[:, H:])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,Hkv,hd,page,window", [(4, 4, 16, 16, 0), (6, 2, 48, 16, 0), (5, 1, 80, 32, 0),
                                                  (8, 2, 128, 64, 0), (3, 3, 32, 16, 37), (16, 2, 64, 16, 0)])
def test_attention_generic(dtype, H, Hkv, hd, page, window):
    T = 150
    qkv, cache, bt, pos, seg, table, inv = _paged_setup(dtype, T, H, Hkv, hd, page, seed=21, rot=0)
    ops.rope_kv_write(qkv, cache, None, pos, seg, bt, H, Hkv, hd, 0, page)
    out = torch.empty(T, H * hd, device=DEV, dtype=dtype)
    scale = 1.0 / math.sqrt(hd)

    class Ctx:
        tok_pos, tok_seg = pos, seg
    ops.attention_generic(out, qkv[:, : H * hd], cache, pos, seg, bt, H, Hkv, hd, page, window, scale)
    src = qkv.double().cpu().reshape(T, H + 2 * Hkv, hd)
    ref = plain.attention(src[:, :H], src[:, H:H + Hkv], src[:, H + Hkv:], window=window).reshape(T, H * hd)
    assert torch.allclose(out.double().cpu(), ref, **tol(dtype))


def test_attention_generic_finds_a_far_key():
    """One early key is made to match the last query strongly; missing it changes the output wholly."""
    H, Hkv, hd, page, T = 2, 1, 64, 16, 700
    qkv, cache, bt, pos, seg, _, _ = _paged_setup(torch.float32, T, H, Hkv, hd, page, seed=31, rot=0, sharp=0.3)
    q = qkv.view(T, H + 2, hd)
    q[3, H] = q[T - 1, 0] * 40.0                       # key of position 3 lines up with the last query of head 0
    q[3, H + 1] = 100.0                                # and its value stands out
    ops.rope_kv_write(qkv, cache, None, pos, seg, bt, H, Hkv, hd, 0, page)
    out = torch.empty(T, H * hd, device=DEV)
    ops.attention_generic(out, qkv[:, : H * hd], cache, pos, seg, bt, H, Hkv, hd, page, 0, 1.0 / 8.0)
    assert float(out[T - 1, :hd].min()) > 99.0
    src = qkv.double().cpu().reshape(T, H + 2, hd)
    ref = plain.attention(src[:, :H], src[:, H:H + 1], src[:, H + 1:]).reshape(T, H * hd)
    assert torch.allclose(out.double().cpu(), ref, rtol=1e-4, atol=1e-4)


def test_argmax_first_maximum_wins():
    logits = rnd(6, 1001, seed=41)
    logits[2, 17] = logits[2, 900] = 50.0
    logits[3] = 0.0
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    ops.argmax(out, logits)
    ref = [plain.argmax(row) for row in logits.cpu()]
    assert out.tolist() == ref and ref[2] == 17 and ref[3] == 0


def _sample(logits, temperature, top_k, top_p, min_p, u, recent=None, pens=(1.0, 0.0, 0.0)):
    rows = logits.shape[0]
    f = lambda v: torch.full((rows,), float(v), device=DEV)
    out = torch.empty(rows, dtype=torch.int32, device=DEV)
    uu = torch.tensor(u, dtype=torch.float32, device=DEV) if not isinstance(u, float) else f(u)
    rc = None
    if recent is not None:
        rc = torch.tensor(recent, dtype=torch.int32, device=DEV)
    ops.sample(out, logits.clone(), f(temperature), torch.full((rows,), top_k, dtype=torch.int32, device=DEV),
               f(top_p), f(min_p), uu, rc, f(pens[0]) if rc is not None else None,
               f(pens[1]) if rc is not None else None, f(pens[2]) if rc is not None else None)
    return out.tolist()


@pytest.mark.parametrize("top_k,top_p,min_p", [(0, 1.0, 0.0), (5, 1.0, 0.0), (0, 0.7, 0.0), (0, 1.0, 0.2),
                                               (40, 0.95, 0.05), (1, 1.0, 0.0), (7, 0.5, 0.1)])
def test_sampler_draws_only_from_the_reference_candidate_set(top_k, top_p, min_p):
    V, rows = 777, 64
    logits = rnd(1, V, seed=51, scale=2.0).repeat(rows, 1)
    us = [(i + 0.5) / rows for i in range(rows)]
    got = _sample(logits, 0.9, top_k, top_p, min_p, us)
    ids, probs = plain.candidate_set(logits[0].cpu().numpy(), 0.9, top_k, top_p, min_p)
    allowed = set(int(i) for i in ids)
    assert set(got) <= allowed
    # inverse CDF in id order over the same set: the draws must follow it exactly
    order = sorted(allowed)
    p = {int(i): float(pr) for i, pr in zip(ids, probs)}
    cdf = np.cumsum([p[i] for i in order]) / sum(p.values())
    for u, g in zip(us, got):
        j = int(np.searchsorted(cdf, u, side="right"))
        assert g == order[min(j, len(order) - 1)] or abs(cdf[min(j, len(cdf) - 1)] - u) < 1e-4 or (j > 0 and abs(cdf[j - 1] - u) < 1e-4)


def test_sampler_statistics_follow_the_distribution():
    V, rows = 50, 4096
    logits = rnd(1, V, seed=52, scale=1.5).repeat(rows, 1)
    g = torch.Generator().manual_seed(3)
    us = torch.rand(rows, generator=g).tolist()
    got = np.bincount(_sample(logits, 1.0, 0, 1.0, 0.0, us), minlength=V) / rows
    p = torch.softmax(logits[0].double().cpu(), 0).numpy()
    assert np.abs(got - p).max() < 0.03


def test_sampler_greedy_ties_and_penalties():
    V = 300
    logits = torch.zeros(3, V, device=DEV)
    assert _sample(logits, 0.0, 0, 1.0, 0.0, 0.3) == [0, 0, 0]                 # all equal: lowest id
    assert _sample(logits, 1.0, 1, 1.0, 0.0, 0.9) == [0, 0, 0]                 # top-k 1 among ties keeps exactly one
    logits = rnd(2, V, seed=53)
    logits[:, 10] = 9.0
    logits[:, 20] = 8.5
    assert _sample(logits, 0.0, 0, 1.0, 0.0, 0.5) == [10, 10]
    recent = [[10, 10, 3, -1], [4, 5, 6, -1]]                                    # row 0 has seen token 10 twice
    got = _sample(logits, 0.0, 0, 1.0, 0.0, 0.5, recent=recent, pens=(1.1, 0.5, 0.0))
    ref = [int(np.argmax(plain.apply_penalties(logits[r].cpu().numpy(), [t for t in recent[r] if t >= 0], 1.1, 0.5, 0.0)))
           for r in range(2)]
    assert got == ref == [20, 10]


def test_sampler_same_row_same_number_same_token_whatever_the_batch():
    V = 5000
    a = rnd(1, V, seed=54, scale=2.0)
    alone = _sample(a, 0.8, 40, 0.95, 0.05, 0.4321)[0]
    batch = torch.cat([rnd(3, V, seed=55), a, rnd(2, V, seed=56)])
    us = [0.1, 0.9, 0.5, 0.4321, 0.7, 0.2]
    assert _sample(batch, 0.8, 40, 0.95, 0.05, us)[3] == alone


# ------------------------------------------------------------------ tensor-core attention (bfloat16)

def _segments(lens_ctx, H, Hkv, hd, page, seed, window=0):
    """Several requests; request i has ctx tokens cached of which the last q are this step's
    queries.  Pages are scattered.  Returns everything the kernels need and the plain reference."""
    g = torch.Generator().manual_seed(seed)
    S = len(lens_ctx)
    n_blocks = [-(-c // page) for _, c in lens_ctx]
    n_pages = sum(n_blocks) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(n_blocks)
    bt = torch.full((S, width), n_pages - 1, dtype=torch.int32)
    cache = torch.zeros(n_pages, 2, Hkv, page, hd, dtype=torch.bfloat16)
    qs, refs, pos, seg, qstart, pos0 = [], [], [], [], [0], []
    for i, (qlen, c) in enumerate(lens_ctx):
        pages = [perm.pop() for _ in range(n_blocks[i])]
        bt[i, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        k = (torch.randn(c, Hkv, hd, generator=g) * 1.5).to(torch.bfloat16)
        v = torch.randn(c, Hkv, hd, generator=g).to(torch.bfloat16)
        qfull = (torch.randn(c, H, hd, generator=g) * 1.5).to(torch.bfloat16)
        for t in range(c):
            cache[pages[t // page], 0, :, t % page] = k[t]
            cache[pages[t // page], 1, :, t % page] = v[t]
        ref = plain.attention(qfull.double(), k.double(), v.double(), window=window, rows=range(c - qlen, c))[c - qlen:]
        qs.append(qfull[c - qlen:].reshape(qlen, H * hd))
        refs.append(ref.reshape(qlen, H * hd))
        pos += list(range(c - qlen, c))
        seg += [i] * qlen
        qstart.append(qstart[-1] + qlen)
        pos0.append(c - qlen)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return dict(q=torch.cat(qs).to(DEV), cache=cache.to(DEV), bt=bt.to(DEV), pos=i32(pos), seg=i32(seg), qstart=i32(qstart),
                pos0=i32(pos0), ref=torch.cat(refs), S=S, max_q=max(q for q, _ in lens_ctx), max_ctx=max(c for _, c in lens_ctx))


ATT_SHAPES = [(4, 4, 16, 16, 0), (6, 2, 32, 16, 0), (5, 1, 48, 32, 0), (8, 2, 64, 16, 0), (3, 3, 80, 16, 0),
              (12, 4, 96, 64, 0), (14, 2, 112, 16, 0), (32, 8, 128, 16, 0), (16, 1, 128, 16, 0), (4, 2, 64, 16, 37)]


@pytest.mark.parametrize("variant", [0, 1])        # 0: shared-memory tiles where they exist; 1: register-direct
@pytest.mark.parametrize("H,Hkv,hd,page,window", ATT_SHAPES)
def test_attention_prefill_bf16(H, Hkv, hd, page, window, variant):
    d = _segments([(70, 70), (1, 33), (130, 200), (2, 2), (16, 48), (1, 1), (64, 64), (65, 129)], H, Hkv, hd, page, seed=61, window=window)
    out = torch.full_like(d["q"], float("nan"))
    assert ops.attention_prefill_bf16(out, d["q"], d["cache"], d["qstart"], d["pos0"], d["bt"], d["S"], d["max_q"], H, Hkv, hd,
                                      page, window, 1.0 / math.sqrt(hd), variant)
    assert torch.allclose(out.double().cpu(), d["ref"], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("variant", [0, 1])        # 0: bulk copies into a shared-memory ring; 1: per-thread loads
@pytest.mark.parametrize("splits", [1, 3, 16])
@pytest.mark.parametrize("H,Hkv,hd,page,window", ATT_SHAPES)
def test_attention_decode_bf16(H, Hkv, hd, page, window, splits, variant):
    d = _segments([(1, 70), (1, 1), (1, 333), (1, 16), (1, 17), (1, 1024), (1, 64)], H, Hkv, hd, page, seed=62, window=window)
    out = torch.full_like(d["q"], float("nan"))
    ops.attention_set_decode_variant(variant)
    try:
        assert ops.attention_decode_bf16(out, d["q"], d["cache"], d["pos"], d["seg"], d["bt"], H, Hkv, hd, page, window,
                                         1.0 / math.sqrt(hd), splits)
        ops.check_kernel_errors()
    finally:
        ops.attention_set_decode_variant(None)
    assert torch.allclose(out.double().cpu(), d["ref"], rtol=2e-2, atol=2e-2)


def test_attention_bf16_finds_a_far_key_and_respects_page_edges():
    """A key deep in the context is made to dominate; both kernels must see it, at a page's edge too."""
    H, Hkv, hd, page = 8, 2, 128, 16
    for far in (0, 15, 16, 511, 512):
        d = _segments([(1, 900)], H, Hkv, hd, page, seed=70 + far)
        pages = d["bt"][0].tolist()
        q = d["q"].view(1, H, hd)
        d["cache"][pages[far // page], 0, 0, far % page] = (q[0, 1].float() * 6.0).to(torch.bfloat16)   # kv head 0 serves heads 0..3
        d["cache"][pages[far // page], 1, 0, far % page] = 50.0
        for fn in ("decode", "decode_bulk", "prefill"):
            out = torch.zeros_like(d["q"])
            if fn.startswith("decode"):
                ops.attention_set_decode_variant(0 if fn == "decode_bulk" else 1)
                try:
                    assert ops.attention_decode_bf16(out, d["q"], d["cache"], d["pos"], d["seg"], d["bt"], H, Hkv, hd, page, 0, 1 / math.sqrt(hd), 4)
                finally:
                    ops.attention_set_decode_variant(None)
            else:
                assert ops.attention_prefill_bf16(out, d["q"], d["cache"], d["qstart"], d["pos0"], d["bt"], 1, 1, H, Hkv, hd, page, 0, 1 / math.sqrt(hd))
            assert float(out.view(H, hd)[1].float().min()) > 49.0, f"{fn}: key {far} was not found"


def test_attention_bf16_refuses_what_it_cannot_do():
    d = _segments([(1, 20)], 4, 4, 16, 16, seed=80)
    q = torch.zeros(1, 4 * 144, dtype=torch.bfloat16, device=DEV)
    cache = torch.zeros(3, 2, 4, 16, 144, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros_like(q)
    assert not ops.attention_decode_bf16(out, q, cache, d["pos"], d["seg"], d["bt"], 4, 4, 144, 16, 0, 0.1, 1)    # head size 144
    assert not ops.attention_prefill_bf16(out, q, cache, d["qstart"], d["pos0"], d["bt"], 1, 1, 4, 4, 144, 16, 0, 0.1)


@pytest.mark.parametrize("H,Hkv,hd,page,window", [(8, 2, 64, 16, 0), (32, 8, 128, 16, 0), (16, 1, 128, 16, 0), (4, 2, 64, 16, 37),
                                                  (12, 4, 128, 64, 0), (6, 3, 128, 32, 150), (32, 8, 64, 16, 0), (32, 4, 128, 16, 200),
                                                  (40, 40, 64, 32, 90)])
def test_attention_prefill_tcgen05(H, Hkv, hd, page, window):
    """Segments of unequal lengths, some starting deep in their request.  With few heads the launch has fewer
    work items than SMs and takes query tiles one by one; with 32 or 40 heads it takes them in pairs (the
    300-row and 129-row segments then end in a pair with one tile only, and rows of other segments lie in the
    tiles' unused halves)."""
    d = _segments([(70, 70), (1, 33), (300, 420), (2, 2), (128, 128), (129, 257), (16, 48), (1, 1)], H, Hkv, hd, page, seed=91, window=window)
    out = torch.full_like(d["q"], float("nan"))
    assert ops.attention_prefill_tc(out, d["q"], d["cache"], d["qstart"], d["pos0"], d["bt"], d["S"], d["max_q"], H, Hkv, hd,
                                    page, window, 1.0 / math.sqrt(hd))
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    assert torch.allclose(out.double().cpu(), d["ref"], rtol=2e-2, atol=2e-2)


def test_attention_prefill_tcgen05_finds_a_far_key():
    H, Hkv, hd, page = 8, 2, 128, 16
    for far in (0, 15, 16, 127, 128, 511, 600):
        d = _segments([(140, 900)], H, Hkv, hd, page, seed=170 + far)
        pages = d["bt"][0].tolist()
        q = d["q"].view(140, H, hd)
        d["cache"][pages[far // page], 0, 0, far % page] = (q[139, 1].float() * 6.0).to(torch.bfloat16)
        d["cache"][pages[far // page], 1, 0, far % page] = 50.0
        out = torch.zeros_like(d["q"])
        assert ops.attention_prefill_tc(out, d["q"], d["cache"], d["qstart"], d["pos0"], d["bt"], 1, 140, H, Hkv, hd, page, 0, 1 / math.sqrt(hd))
        torch.cuda.synchronize()
        ops.check_kernel_errors()
        assert float(out.view(140, H, hd)[139, 1].float().min()) > 49.0, f"key {far} was not found"


# ------------------------------------------------------------------ the lengths the benchmark runs

@pytest.mark.parametrize("variant", [0, 1])
@pytest.mark.parametrize("H,Hkv,hd", [(32, 8, 128), (32, 8, 64)])
def test_attention_decode_bf16_at_8192_keys(H, Hkv, hd, variant):
    """Single tokens over 8,192 and 5,000 cached keys (512 block-table entries a row), with the slice
    count the dispatcher picks for such a step and with the most slices; one far key per request is
    made to dominate one head, so that a slice that is skipped or read twice shows."""
    page = 16
    d = _segments([(1, 8192), (1, 5000), (1, 31)], H, Hkv, hd, page, seed=300 + hd)
    q = d["q"].view(3, H, hd)
    for s_i, far in ((0, 4097), (1, 0), (0, 8191)):
        pages = d["bt"][s_i].tolist()
        head = 1 if far != 8191 else 5                          # kv head 0 serves heads 0..3, kv head 1 heads 4..7
        kvh = head // (H // Hkv)
        d["cache"][pages[far // page], 0, kvh, far % page] = (q[s_i, head].float() * 6.0).to(torch.bfloat16)
        d["cache"][pages[far // page], 1, kvh, far % page] = 50.0
    ops.attention_set_decode_variant(variant)
    try:
        for splits in (ops.decode_splits(3, Hkv, 8192), ops.decode_splits(3, Hkv, 8192, known=False), 16):
            out = torch.full_like(d["q"], float("nan"))
            assert ops.attention_decode_bf16(out, d["q"], d["cache"], d["pos"], d["seg"], d["bt"], H, Hkv, hd, page, 0,
                                             1.0 / math.sqrt(hd), splits)
            ops.check_kernel_errors()
            o = out.view(3, H, hd).float()
            assert float(o[0, 1].min()) > 49.0 and float(o[1, 1].min()) > 49.0 and float(o[0, 5].min()) > 49.0, f"splits {splits}: a far key was missed"
            untouched = torch.ones(3, H, dtype=torch.bool)
            untouched[0, 0:8] = False; untouched[1, 0:4] = False       # heads that share a kv head with a planted key
            ref = d["ref"].view(3, H, hd)
            assert torch.allclose(out.view(3, H, hd).double().cpu()[untouched], ref[untouched], rtol=2e-2, atol=2e-2), f"splits {splits}"
    finally:
        ops.attention_set_decode_variant(None)


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_attention_prefill_tcgen05_on_random_mixes_of_segments(seed):
    """Random head counts, page sizes, windows, segment lengths and depths (few heads: tiles taken singly; 32
    or 40 heads: in pairs), with and without the hint of the portions' longest context, twice each, against
    float64: what a warp running ahead of the others, a tile without its pair or a phase counted wrongly
    would break."""
    import random
    rnd = random.Random(seed)
    for case in range(6):
        hd = rnd.choice([64, 128])
        Hkv, group = rnd.choice([(1, 4), (2, 2), (4, 5), (8, 4), (10, 4)])
        H = Hkv * group
        page = rnd.choice([16, 32, 64])
        window = rnd.choice([0, 0, rnd.randint(20, 400)])
        lens = []
        for _ in range(rnd.randint(1, 4)):
            qlen = rnd.choice([1, 33, 100, 128, 129, 256, 300, 511, 640])
            lens.append((qlen, qlen + rnd.choice([0, 0, 5, 128, 500, 1000])))
        if max(q for q, _ in lens) < 32:
            lens[0] = (77, 300)
        d = _segments(lens, H, Hkv, hd, page, seed=seed * 100 + case, window=window)
        for hint in (0, d["max_ctx"]):
            for _ in range(2):
                out = torch.full_like(d["q"], float("nan"))
                assert ops.attention_prefill_tc(out, d["q"], d["cache"], d["qstart"], d["pos0"], d["bt"], d["S"], d["max_q"], H, Hkv,
                                                hd, page, window, 1.0 / math.sqrt(hd), max_ctx_len=hint)
                torch.cuda.synchronize()
                ops.check_kernel_errors()
                assert torch.allclose(out.double().cpu(), d["ref"], rtol=2e-2, atol=2e-2), (H, Hkv, hd, page, window, lens, hint)


@pytest.mark.parametrize("H,Hkv,hd", [(32, 8, 128), (32, 8, 64)])
def test_attention_prefill_tcgen05_of_portions_deep_in_their_requests(H, Hkv, hd):
    """Told the portions' longest context, the kernel takes the query tiles of deep portions one by one; not told,
    in pairs (288 pairs here): both ways against float64, two portions of unequal length, one of them with an
    odd number of tiles."""
    page = 16
    d = _segments([(2048, 4200), (300, 2500)], H, Hkv, hd, page, seed=500 + hd)
    for hint in (4200, 0):
        out = torch.full_like(d["q"], float("nan"))
        assert ops.attention_prefill_tc(out, d["q"], d["cache"], d["qstart"], d["pos0"], d["bt"], d["S"], d["max_q"], H, Hkv, hd,
                                        page, 0, 1.0 / math.sqrt(hd), max_ctx_len=hint)
        torch.cuda.synchronize()
        ops.check_kernel_errors()
        assert torch.allclose(out.double().cpu(), d["ref"], rtol=2e-2, atol=2e-2), f"hint {hint}"


@pytest.mark.parametrize("variant", [0, 1])
def test_attention_decode_bf16_at_32768_keys(variant):
    """Single tokens over 32,768 and 9,000 cached keys (2,048 block-table entries a row) with the slice counts the
    dispatcher picks for such a step; far keys in the first, a middle and the last page are made to dominate."""
    H, Hkv, hd, page = 8, 2, 128, 16
    d = _segments([(1, 32768), (1, 9000)], H, Hkv, hd, page, seed=777)
    q = d["q"].view(2, H, hd)
    for s_i, far, head in ((0, 3, 0), (0, 32767, 5), (1, 4500, 1)):
        pages = d["bt"][s_i].tolist()
        kvh = head // (H // Hkv)
        d["cache"][pages[far // page], 0, kvh, far % page] = (q[s_i, head].float() * 6.0).to(torch.bfloat16)
        d["cache"][pages[far // page], 1, kvh, far % page] = 50.0
    ops.attention_set_decode_variant(variant)
    try:
        for splits in (ops.decode_splits(2, Hkv, 32768), ops.decode_splits(2, Hkv, 32768, known=False), 1):
            out = torch.full_like(d["q"], float("nan"))
            assert ops.attention_decode_bf16(out, d["q"], d["cache"], d["pos"], d["seg"], d["bt"], H, Hkv, hd, page, 0,
                                             1.0 / math.sqrt(hd), splits)
            ops.check_kernel_errors()
            o = out.view(2, H, hd).float()
            assert float(o[0, 0].min()) > 49.0 and float(o[0, 5].min()) > 49.0 and float(o[1, 1].min()) > 49.0, f"splits {splits}: a far key was missed"
            untouched = torch.zeros(2, H, dtype=torch.bool)
            untouched[1, 4:8] = True                                  # the only kv head without a planted key
            ref = d["ref"].view(2, H, hd)
            assert torch.allclose(out.view(2, H, hd).double().cpu()[untouched], ref[untouched], rtol=2e-2, atol=2e-2), f"splits {splits}"
    finally:
        ops.attention_set_decode_variant(None)


@pytest.mark.parametrize("H,Hkv,hd,lens", [(32, 8, 128, [(2048, 2048)]), (8, 2, 128, [(2048, 4096), (100, 100)]),
                                           (8, 2, 64, [(2048, 2048), (1, 700)]), (32, 8, 64, [(2048, 2048)]),
                                           (16, 4, 128, [(1920, 4096), (700, 700)])])
def test_attention_prefill_tcgen05_at_2048_tokens(H, Hkv, hd, lens):
    """A whole 2,048-token prompt (the benchmark's prefill), and a 2,048-token portion that follows
    2,048 cached tokens, against float64."""
    page = 16
    d = _segments(lens, H, Hkv, hd, page, seed=400 + hd + H)
    out = torch.full_like(d["q"], float("nan"))
    assert ops.attention_prefill_tc(out, d["q"], d["cache"], d["qstart"], d["pos0"], d["bt"], d["S"], d["max_q"], H, Hkv, hd,
                                    page, 0, 1.0 / math.sqrt(hd))
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    assert torch.allclose(out.double().cpu(), d["ref"], rtol=2e-2, atol=2e-2)
