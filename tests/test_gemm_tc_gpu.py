"""The tcgen05 matrix product alone, against a float64 product of the same bfloat16 inputs."""
import pytest
import torch

from qorvix_b200.csrc import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).to(DEV)


def check(M, N, K, out_dtype, force_splits=0, lda=None):
    a_full = rnd(M, lda or K, seed=M + K)
    a = a_full[:, :K]
    w = rnd(N, K, seed=N + 1, scale=0.05)
    c = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
    assert ops.gemm_bf16_tc(c, a, w, force_splits=force_splits)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    ref = a.double() @ w.double().t()
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-3
    err = (c.double() - ref).abs().max().item()
    assert err <= tol * max(1.0, ref.abs().max().item()), f"M={M} N={N} K={K}: max err {err}"


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 256), (256, 384, 4096), (200, 1000, 328),
                                   (2048, 6144, 4096), (65, 136, 72), (300, 331, 1000), (4000, 2000, 136)])
def test_many_tokens(M, N, K, out_dtype):
    check(M, N, K, out_dtype)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(256, 4096, 14336), (130, 2560, 8192), (384, 2048, 16384), (200, 2000, 9000), (700, 1500, 8200),
                                   (96, 4096, 14336), (256, 4096, 4096), (130, 6144, 4104), (512, 4096, 4096), (544, 5120, 5120)])
def test_tiles_shared_between_ctas_give_the_sums_of_whole_tiles(M, N, K, out_dtype):
    """A product with a long walk along K whose tiles fill at most three quarters of the SMs shares them (the
    first eight shapes; the last two are not shared): a CTA that has only later k blocks of a tile leaves its
    float32 sums in the workspace, the tile's owner adds them to its own.  The
    result stays within the product's tolerance, is the same on every launch (the flags come down again), and
    equals the unshared product up to the rounding of a few float32 additions per element."""
    check(M, N, K, out_dtype)
    a, w = rnd(M, K, seed=3), rnd(N, K, seed=4, scale=0.05)
    outs = []
    for shared in (True, True, False):
        ops.gemm_share_tiles(shared)
        c = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
        assert ops.gemm_bf16_tc(c, a, w)
        outs.append(c)
    ops.gemm_share_tiles(True)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    assert torch.equal(outs[0], outs[1])
    whole = outs[2].double()
    assert (outs[0].double() - whole).abs().max().item() <= (2e-5 if out_dtype == torch.float32 else 2e-2) * max(1.0, whole.abs().max().item())


@pytest.mark.parametrize("bn", [16, 48, 112, 128, 144, 240, 256])
@pytest.mark.parametrize("M,N,K", [(300, 1000, 520), (129, 272, 64), (512, 5120, 1024), (200, 336, 136)])
def test_many_tokens_at_every_tile_width(M, N, K, bn):
    """The persistent kernel's tile width is a run-time value (a product picks 128 or 256): any multiple of
    16 gives the same product, from packed tiles (pieces of one to three tiles per stage) and from rows."""
    ops.gemm_bf16_set_prefill_tile_width(bn)
    try:
        check(M, N, K, torch.float32)
        a, w = rnd(M, K, seed=M + K), rnd(N, K, seed=N + 1, scale=0.05)
        c = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
        assert ops.gemm_bf16_packed(c, a, ops.pack_weight(w), N)
        torch.cuda.synchronize()
        ops.check_kernel_errors()
        ref = a.double() @ w.double().t()
        assert (c.double() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    finally:
        ops.gemm_bf16_set_prefill_tile_width(0)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 6144, 4096), (8, 4096, 14336), (16, 256, 128), (17, 1000, 328),
                                   (33, 4096, 4096), (64, 28672, 4096), (5, 331, 72), (64, 128256, 1024)])
def test_few_tokens_swapped(M, N, K, out_dtype):
    check(M, N, K, out_dtype)


@pytest.mark.parametrize("splits", [1, 2, 3, 8])
def test_split_k_sums_in_a_fixed_order(splits):
    M, N, K = 8, 512, 4096
    a, w = rnd(M, K, seed=1), rnd(N, K, seed=2, scale=0.05)
    outs = []
    for _ in range(3):
        c = torch.empty(M, N, device=DEV, dtype=torch.float32)
        assert ops.gemm_bf16_tc(c, a, w, force_splits=splits)
        outs.append(c)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[1], outs[2])      # run to run identical
    ref = a.double() @ w.double().t()
    assert (outs[0].double() - ref).abs().max().item() < 2e-3 * ref.abs().max().item()


def test_strided_activations_and_refused_shapes():
    check(40, 256, 128, torch.bfloat16, lda=384)            # a column slice of a wider buffer
    a, w = rnd(4, 100, seed=3), rnd(64, 100, seed=4)
    c = torch.zeros(4, 64, device=DEV, dtype=torch.bfloat16)
    assert not ops.gemm_bf16_tc(c, a, w)                    # K = 100 is no multiple of 8: refused, untouched
    assert float(c.abs().sum()) == 0.0
    ops.gemm(c, a, w)                                       # the dispatcher falls back to the CUDA cores
    ref = a.double() @ w.double().t()
    assert (c.double() - ref).abs().max().item() < 2e-2 * ref.abs().max().item()


@pytest.mark.parametrize("M,f,K", [(8, 256, 128), (3, 14336, 256), (40, 512, 4096), (64, 1008, 72), (128, 64, 64),
                                   (300, 1008, 328), (2048, 1024, 512)])
def test_fused_swiglu_epilogue(M, f, K):
    g, u = rnd(f, K, seed=5, scale=0.1), rnd(f, K, seed=6, scale=0.1)
    w = torch.stack([g.view(f // 16, 16, K), u.view(f // 16, 16, K)], dim=1).reshape(2 * f, K).contiguous()
    a = rnd(M, K, seed=7)
    out = torch.full((M, f), float("nan"), device=DEV, dtype=torch.bfloat16)
    assert ops.gemm_bf16_tc(out, a, w, swiglu=True)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    gg, uu = a.double() @ g.double().t(), a.double() @ u.double().t()
    ref = gg / (1 + torch.exp(-gg)) * uu
    assert (out.double() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    # the unfused route over the same interleaved weight agrees
    gu = torch.empty(M, 2 * f, device=DEV, dtype=torch.bfloat16)
    ops.gemm(gu, a, w)
    out2 = torch.empty_like(out)
    ops.swiglu(out2, gu, interleaved=True)
    assert (out2.double() - ref).abs().max().item() <= 3e-2 * max(1.0, ref.abs().max().item())


def test_packed_weight_tiles_are_the_swizzled_image_of_the_rows():
    """pack_weight stores tile (t, kb) of 128 rows x 64 k at ((t * kblocks + kb) * 8192) elements, row r at
    128-byte pitch with its 16-byte chunk c at position c ^ (r % 8), zero where the matrix ends."""
    N, K = 200, 328                                   # two row tiles (the second ragged), six k blocks (the last ragged)
    w = rnd(N, K, seed=3)
    packed = ops.pack_weight(w).cpu().view(2, 6, 128, 8, 8)      # [tile][kb][row][chunk position][8 elements]
    wc = torch.zeros(256, 384, dtype=torch.bfloat16)
    wc[:N, :K] = w.cpu()
    for t in range(2):
        for kb in range(6):
            for r in (0, 1, 7, 8, 63, 127):
                for c in range(8):
                    got = packed[t, kb, r, c ^ (r & 7)]
                    want = wc[t * 128 + r, kb * 64 + c * 8: kb * 64 + c * 8 + 8]
                    assert torch.equal(got, want), (t, kb, r, c)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (8, 6144, 4096), (8, 4096, 14336), (3, 200, 96), (17, 1000, 328),
                                   (40, 520, 1024), (64, 4096, 4096)])
def test_packed_weights_give_the_same_product_bit_for_bit(M, N, K, out_dtype):
    a, w = rnd(M, K, seed=M + K), rnd(N, K, seed=N + 1, scale=0.05)
    packed = ops.pack_weight(w)
    c_rows = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
    c_tiles = torch.full((M, N), float("nan"), device=DEV, dtype=out_dtype)
    assert ops.gemm_bf16_tc(c_rows, a, w)
    assert ops.gemm_bf16_packed(c_tiles, a, packed, N)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    assert torch.equal(c_rows, c_tiles)
    ref = a.double() @ w.double().t()
    tol = 2e-2 if out_dtype == torch.bfloat16 else 2e-3
    assert (c_tiles.double() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())


def test_packed_weights_with_the_fused_swiglu_epilogue():
    M, f, K = 8, 1008, 328
    g, u = rnd(f, K, seed=5, scale=0.1), rnd(f, K, seed=6, scale=0.1)
    w = torch.stack([g.view(f // 16, 16, K), u.view(f // 16, 16, K)], dim=1).reshape(2 * f, K).contiguous()
    a = rnd(M, K, seed=7)
    o_rows = torch.empty((M, f), device=DEV, dtype=torch.bfloat16)
    o_tiles = torch.empty_like(o_rows)
    assert ops.gemm_bf16_tc(o_rows, a, w, swiglu=True)
    assert ops.gemm_bf16_packed(o_tiles, a, ops.pack_weight(w), 2 * f, swiglu=True)
    ops.check_kernel_errors()
    assert torch.equal(o_rows, o_tiles)


@pytest.mark.parametrize("H,Hkv,hd,T,d", [(4, 2, 128, 300, 256), (6, 2, 64, 129, 192), (8, 8, 64, 700, 512), (32, 8, 128, 2048, 1024),
                                         (3, 1, 64, 65, 136)])
def test_qkv_product_with_rotation_and_cache_write_in_its_epilogue(H, Hkv, hd, T, d):
    """The fused product against the product followed by the rotary kernel: rotated queries in the
    output, rotated keys and plain values in each token's page slot; tokens of several requests at
    different positions, pages handed out in a shuffled order."""
    page = 16
    N = (H + 2 * Hkv) * hd
    w = rnd(N, d, seed=11, scale=0.05)
    x = rnd(T, d, seed=12)
    g = torch.Generator().manual_seed(13)
    lens = [T // 3, T - T // 3 - 3, 3]                       # three requests, the tokens of each contiguous
    starts = [7, 0, 100]                                     # position of each request's first token in the step
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)]).to(torch.int32)
    seg = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).to(torch.int32)
    blocks = [-(-(s + n) // page) for s, n in zip(starts, lens)]
    perm = torch.randperm(sum(blocks), generator=g).to(torch.int32)
    bt = torch.zeros(3, max(blocks), dtype=torch.int32)
    o = 0
    for i, nb in enumerate(blocks):
        bt[i, :nb] = perm[o:o + nb]
        o += nb
    P = int(max(s + n for s, n in zip(starts, lens)))
    ang = torch.arange(P, dtype=torch.float64)[:, None] * torch.exp(-torch.arange(hd // 2, dtype=torch.float64) * 0.3)[None, :]
    table = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).float().contiguous().to(DEV)
    pos, seg, bt = pos.to(DEV), seg.to(DEV), bt.to(DEV)
    cache_a = torch.zeros(sum(blocks) + 1, 2, Hkv, page, hd, device=DEV, dtype=torch.bfloat16)
    cache_b = torch.zeros_like(cache_a)
    qkv_a = torch.empty(T, N, device=DEV, dtype=torch.bfloat16)
    ops.gemm(qkv_a, x, w)
    ops.rope_kv_write(qkv_a, cache_a, table, pos, seg, bt, H, Hkv, hd, hd, page)
    qkv_b = torch.full((T, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    assert ops.gemm_qkv_rope(qkv_b, x, ops.pack_weight(w), cache_b, table, pos, seg, bt, H, Hkv, hd, page)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    # the fused path rotates the float32 sums, the other one their bfloat16 roundings: equal within that rounding
    scale = float(qkv_a[:, : H * hd].float().abs().max())
    assert float((qkv_a[:, : H * hd].float() - qkv_b[:, : H * hd].float()).abs().max()) <= 2e-2 * scale
    assert float((cache_a.float() - cache_b.float()).abs().max()) <= 2e-2 * max(1.0, float(cache_a.float().abs().max()))
    assert float(cache_b.float().abs().sum()) > 0
    # pages that no token of the step lies in stay untouched
    touched = torch.zeros(sum(blocks) + 1, dtype=torch.bool)
    for t in range(T):
        touched[int(bt[int(seg[t]), int(pos[t]) // page])] = True
    assert float(cache_b[~touched.to(DEV)].float().abs().sum()) == 0.0


@pytest.mark.parametrize("M,N,K", [(8, 512, 4096), (1, 4096, 4096), (33, 1000, 2048), (64, 264, 1024)])
def test_few_tokens_product_added_to_the_stream_with_the_next_norms_input(M, N, K):
    """residual += a w^T in the split-K product's epilogue; c = residual * norm weight; per tile of 128
    features the sums of squares of the updated rows."""
    a, w = rnd(M, K, seed=31), rnd(N, K, seed=32, scale=0.05)
    g = torch.Generator().manual_seed(33)
    base = torch.randn(M, N, generator=g).to(DEV)
    nw = (1 + 0.1 * torch.randn(N, generator=g)).to(DEV)
    res = base.clone()
    c = torch.full((M, N), float("nan"), device=DEV, dtype=torch.bfloat16)
    tiles = -(-N // 128)
    ssq = torch.full((tiles, 64), float("nan"), device=DEV)
    assert ops.gemm_bf16_norm(c, a, ops.pack_weight(w), N, residual=res, norm_weight=nw, ssq_out=ssq)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    ref = base.double() + a.double() @ w.double().t()
    assert (res.double() - ref).abs().max().item() <= 2e-3 * max(1.0, ref.abs().max().item())
    want_c = ref * nw.double()
    assert (c.double() - want_c).abs().max().item() <= 2e-2 * max(1.0, want_c.abs().max().item())
    pad = torch.zeros(M, tiles * 128, dtype=torch.float64, device=DEV)
    pad[:, :N] = res.double() ** 2                            # of the stream as the kernel left it
    want_ssq = pad.view(M, tiles, 128).sum(-1).t()            # [tiles, M]
    assert (ssq[:, :M].double() - want_ssq).abs().max().item() <= 1e-4 * max(1.0, want_ssq.abs().max().item())


@pytest.mark.parametrize("M,N,K,swiglu", [(8, 512, 4096, False), (8, 12800, 256, False), (40, 1024, 512, True), (3, 28672, 4096, True),
                                          (64, 6144, 4096, False)])
def test_few_tokens_product_scaled_by_the_norm_of_its_input(M, N, K, swiglu):
    """Each token's sums times rsqrt(mean of squares + eps), the mean given as per-tile sums of squares."""
    a, w = rnd(M, K, seed=41), rnd(N, K, seed=42, scale=0.05)
    g = torch.Generator().manual_seed(43)
    tiles_in, width, eps = 5, 600, 1e-5
    ssq = (torch.rand(tiles_in, 64, generator=g) * 100).to(DEV)
    rs = torch.rsqrt(ssq[:, :M].double().sum(0) / width + eps)            # [M]
    prod = (a.double() @ w.double().t()) * rs[:, None]
    if swiglu:
        gate = prod.view(M, N // 32, 2, 16)[:, :, 0].reshape(M, N // 2)
        up = prod.view(M, N // 32, 2, 16)[:, :, 1].reshape(M, N // 2)
        ref = gate / (1 + torch.exp(-gate)) * up
    else:
        ref = prod
    c = torch.full(tuple(ref.shape), float("nan"), device=DEV, dtype=torch.bfloat16)
    assert ops.gemm_bf16_norm(c, a, ops.pack_weight(w), N, swiglu=swiglu, ssq_in=ssq, stream_width=width, eps=eps)
    torch.cuda.synchronize()
    ops.check_kernel_errors()
    assert (c.double() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())


def test_a_linear_that_kept_only_its_packed_tiles_still_takes_float32_and_sliced_inputs():
    """Linear drops a bfloat16 matrix's rows once the packed tiles exist; an input the packed kernel
    refuses as it is (float32 values, a view whose rows do not start on 16 bytes) is then copied
    into aligned bfloat16 rows instead of failing."""
    from qorvix_b200.parts.linear import Linear
    w = rnd(200, 136, seed=3, scale=0.05)
    lin = Linear(w.clone())
    assert lin.weight is None and lin.packed is not None
    x32 = torch.randn(5, 136, device=DEV, generator=torch.Generator(device=DEV).manual_seed(1))
    ref = x32.to(torch.bfloat16).double() @ w.double().t()
    out = lin(x32, out_dtype=torch.float32)
    assert (out.double() - ref).abs().max().item() <= 2e-3 * ref.abs().max().item()
    wide = rnd(7, 141, seed=4)
    xs = wide[:, 5:]                                   # rows start 10 bytes into a 16-byte line
    assert xs.data_ptr() % 16 != 0
    out = lin(xs, out_dtype=torch.bfloat16)
    ref = xs.double() @ w.double().t()
    assert (out.double() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
