"""Timings of single kernels at named layer shapes: the numbers that choices in csrc/ops.py and
csrc/gemm_bf16.cu (kernel variants, tile widths, split counts) rest on.

    python -m qorvix_b200.microbench gemm --shape llama8b --tokens 2048 --variants 0,3
    python -m qorvix_b200.microbench gemm --shape llama1b --tokens 8 --splits 0,1,2,4,8
    python -m qorvix_b200.microbench gemm --shape llama8b --tokens 512 --widths 256,192,128
    python -m qorvix_b200.microbench attention --batch 8 --ctx 2048 --heads 40 --kv-heads 40 --head-dim 128

Each launch is timed inside a captured chain of 8 to 24 launches over rotating weight (or cache)
buffers larger than L2, with CUDA events around three replays.  There is no counterpart in the
reference, whose benchmark times whole generations only (runtime/include/qorvix/runtime/benchmark.hpp:54-115).
"""
from __future__ import annotations

import argparse

import torch

from .csrc import ops

SHAPES = {      # (name, output rows N, inner size K) of the four products of a layer
    "llama8b": (("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336)),
    "llama1b": (("qkv", 3072, 2048), ("o", 2048, 2048), ("gate_up", 16384, 2048), ("down", 2048, 8192)),
    "llama13b": (("qkv", 15360, 5120), ("o", 5120, 5120), ("gate_up", 27648, 5120), ("down", 5120, 13824)),
}


def timed_chain(fn, launches: int = 24) -> float:
    """Microseconds per call of fn(i) inside a captured chain of `launches` calls."""
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(launches):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(3):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (3 * launches) * 1e3


def _ints(text: str):
    return [int(t) for t in text.split(",") if t != ""]


def bench_gemm(args) -> None:
    dev = "cuda"
    M = args.tokens
    print(f"{args.shape}, {M} tokens, bfloat16, packed weight tiles")
    for name, N, K in SHAPES[args.shape]:
        fused = name == "gate_up"
        copies = max(2, int(300e6 // (N * K * 2)) + 1)          # rotate over more bytes than L2 holds
        ws = [ops.pack_weight(torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02) for _ in range(copies)]
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        out = torch.empty(M, N // 2 if fused else N, device=dev, dtype=torch.bfloat16)
        cells = []
        for variant in _ints(args.variants):
            for width in _ints(args.widths):
                for splits in _ints(args.splits):
                    ops.gemm_bf16_set_prefill_variant(variant)
                    ops.gemm_bf16_set_prefill_tile_width(width)
                    us = timed_chain(lambda i: ops.gemm_bf16_packed(out, x, ws[i % copies], N, force_splits=splits, swiglu=fused),
                                     launches=24 if M <= 64 else 8)
                    cells.append(f"variant {variant} width {width} splits {splits}: {us:7.1f} us "
                                 f"{N * K * 2 / us / 1e6:5.2f} TB/s {2.0 * M * N * K / us / 1e6:6.0f} TFLOP/s")
        ops.gemm_bf16_set_prefill_variant(0)
        ops.gemm_bf16_set_prefill_tile_width(0)
        print(f"  {name:8s} {N:6d} x {K:5d}: " + " | ".join(cells), flush=True)
        del ws
    ops.check_kernel_errors()


def bench_attention(args) -> None:
    dev = "cuda"
    B, ctx, H, Hkv, hd, page = args.batch, args.ctx, args.heads, args.kv_heads, args.head_dim, 16
    blocks = -(-ctx // page)
    kv_bytes = B * ctx * 2 * Hkv * hd * 2
    copies = max(2, min(8, int(400e6 // kv_bytes) + 1))
    caches = torch.randn(copies, B * blocks + 1, 2, Hkv, page, hd, device=dev, dtype=torch.bfloat16)
    table = torch.arange(B * blocks, dtype=torch.int32, device=dev).view(B, blocks)
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
    seg = torch.arange(B, dtype=torch.int32, device=dev)
    q = torch.randn(B, H * hd, device=dev, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    print(f"decode attention, batch {B}, context {ctx}, {H}/{Hkv} heads of {hd}: keys and values {kv_bytes / 1e6:.1f} MB; "
          f"the engine takes variant {ops.decode_variant(B, Hkv)} with {ops.decode_splits(B, Hkv, ctx)} slices")
    for variant in (0, 1):
        ops.attention_set_decode_variant(variant)
        cells = []
        for s in _ints(args.splits):
            if s > 1 and ctx // s < 64:
                continue
            us = timed_chain(lambda i: ops.attention_decode_bf16(out, q, caches[i % copies], pos, seg, table, H, Hkv, hd, page,
                                                                 0, hd ** -0.5, max(1, s)))
            cells.append(f"{max(1, s)}: {us:.1f} us")
        print(f"  variant {variant} by slices: " + ", ".join(cells), flush=True)
    ops.attention_set_decode_variant(None)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--shape", choices=sorted(SHAPES), default="llama8b")
    g.add_argument("--tokens", type=int, default=2048)
    g.add_argument("--variants", default="0", help="kernels for more than 64 tokens: 0 persistent, 1 one tile per CTA, 3 CTA pairs")
    g.add_argument("--widths", default="0", help="tile widths of the persistent kernel (0: its own choice)")
    g.add_argument("--splits", default="0", help="K splits of the few-token kernel (0: its own choice)")
    a = sub.add_parser("attention")
    a.add_argument("--batch", type=int, default=8)
    a.add_argument("--ctx", type=int, default=1024)
    a.add_argument("--heads", type=int, default=32)
    a.add_argument("--kv-heads", type=int, default=8)
    a.add_argument("--head-dim", type=int, default=128)
    a.add_argument("--splits", default="1,2,3,4,6,8,12,16")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("qorvix_b200.microbench needs a CUDA device")
    (bench_gemm if args.what == "gemm" else bench_attention)(args)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
