"""Timings of single kernels at a configuration's layer shapes, with their roofline fractions.

bench.py puts these figures beside the step's own (`kernels` in its JSON line); run as a program
it prints them for any of the named shapes:

    python -m qorvix_b200.kernel_bench --config baseline/configs/llama31_8b.json --batch 8 --ctx 1024 --prefill 2048 [--only prefill_attention]

Each launch is timed inside a captured chain of launches over rotating weight (or cache) buffers
larger than L2, with CUDA events around three replays, so the figure is a warm launch's device
time without the host's share.  There is no counterpart in the reference, whose benchmark times
whole generations only (runtime/include/qorvix/runtime/benchmark.hpp:54-115).
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, List, Tuple

import torch

from .csrc import ops

L2_BYTES = 126e6          # rotate over more than this, so that no launch finds its operands in L2


def layer_products(cfg) -> List[Tuple[str, int, int, bool]]:
    """(name, output rows N, inner size K, fused SwiGLU) of the four matrix products of a layer and of
    the output head, from the configuration's sizes."""
    d, f = cfg.hidden_size, cfg.intermediate_size
    q = cfg.num_attention_heads * cfg.head_dim
    kv = cfg.num_key_value_heads * cfg.head_dim
    return [("qkv", q + 2 * kv, d, False), ("o", d, q, False), ("gate_up", 2 * f, d, True), ("down", d, f, False),
            ("lm_head", cfg.vocab_size, d, False)]


def timed_chain(fn, launches: int = 24, replays: int = 3) -> float:
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
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (replays * launches) * 1e3


def _figures(us: float, nbytes: float, flops: float, peaks: dict) -> dict:
    """Time, algorithmic bytes and flops of one launch, and its fraction of the bound that is nearer."""
    gbs, tfl = nbytes / us / 1e3, flops / us / 1e6
    f_mem, f_cmp = gbs / peaks["hbm_gbs"], tfl / peaks["bf16_tflops"]
    bound = "hbm" if f_mem >= f_cmp else "bf16"
    return {"us": round(us, 2), "bytes": int(nbytes), "flops": int(flops), "gb_s": round(gbs, 1), "tflop_s": round(tfl, 1),
            "bound": bound, "frac": round(max(f_mem, f_cmp), 4)}


def gemm_case(M: int, N: int, K: int, swiglu: bool, peaks: dict, out_dtype=torch.bfloat16, device="cuda") -> dict:
    """x[M,K] @ W[N,K]^T from packed weight tiles, as the engine runs it for M tokens."""
    copies = max(2, int(2.5 * L2_BYTES // (N * K * 2)) + 1)
    ws = [ops.pack_weight(torch.randn(N, K, device=device, dtype=torch.bfloat16) * 0.02) for _ in range(copies)]
    x = torch.randn(M, K, device=device, dtype=torch.bfloat16)
    out = torch.empty(M, N // 2 if swiglu else N, device=device, dtype=out_dtype)
    us = timed_chain(lambda i: ops.gemm_bf16_packed(out, x, ws[i % copies], N, swiglu=swiglu), launches=24 if M <= 64 else 8)
    nbytes = N * K * 2 + M * K * 2 + out.numel() * out.element_size()
    return _figures(us, nbytes, 2.0 * M * N * K, peaks)


def decode_attention_case(B: int, ctx: int, H: int, Hkv: int, hd: int, page: int, peaks: dict, device="cuda") -> dict:
    """One query token for each of B requests over ctx cached keys, with the kernel and slice count the
    engine's dispatcher takes for that step."""
    blocks = -(-ctx // page)
    kv_bytes = B * ctx * 2 * Hkv * hd * 2
    copies = max(2, min(8, int(2.5 * L2_BYTES // kv_bytes) + 1))
    caches = torch.randn(copies, B * blocks + 1, 2, Hkv, page, hd, device=device, dtype=torch.bfloat16)
    table = torch.arange(B * blocks, dtype=torch.int32, device=device).view(B, blocks)
    pos = torch.full((B,), ctx - 1, dtype=torch.int32, device=device)
    seg = torch.arange(B, dtype=torch.int32, device=device)
    q = torch.randn(B, H * hd, device=device, dtype=torch.bfloat16)
    out = torch.empty_like(q)
    splits = ops.decode_splits(B, Hkv, ctx)
    us = timed_chain(lambda i: ops.attention_decode_bf16(out, q, caches[i % copies], pos, seg, table, H, Hkv, hd, page, 0,
                                                         hd ** -0.5, splits))
    res = _figures(us, kv_bytes + 2 * q.numel() * 2, 4.0 * B * H * hd * ctx, peaks)
    res["splits"] = splits
    return res


def prefill_attention_case(T: int, H: int, Hkv: int, hd: int, page: int, peaks: dict, device="cuda") -> dict:
    """Causal attention of one whole prompt of T tokens over its own pages (the tcgen05 kernel where it
    takes the head size, else the mma.sync kernel)."""
    blocks = -(-T // page)
    cache = torch.randn(blocks + 1, 2, Hkv, page, hd, device=device, dtype=torch.bfloat16)
    table = torch.arange(blocks, dtype=torch.int32, device=device).view(1, blocks)
    qstart = torch.tensor([0, T], dtype=torch.int32, device=device)
    pos0 = torch.zeros(1, dtype=torch.int32, device=device)
    q = torch.randn(T, H * hd, device=device, dtype=torch.bfloat16)
    out = torch.empty_like(q)

    def run(i):
        if not ops.attention_prefill_tc(out, q, cache, qstart, pos0, table, 1, T, H, Hkv, hd, page, 0, hd ** -0.5):
            ops.attention_prefill_bf16(out, q, cache, qstart, pos0, table, 1, T, H, Hkv, hd, page, 0, hd ** -0.5)

    us = timed_chain(run, launches=8)
    flops = 4.0 * H * hd * (T * (T + 1) / 2)
    return _figures(us, 2 * q.numel() * 2 + T * 2 * Hkv * hd * 2, flops, peaks)


def headline_kernels(cfg, batch: int, ctx: int, prefill_tokens: int, peaks: dict, page: int = 16, only: str = "") -> Dict[str, dict]:
    """The kernels a decode step of `batch` requests at `ctx` tokens and a prefill of `prefill_tokens`
    spend their time in, each alone: the few-token products, decode attention, the many-token products
    and prefill attention.  `only`: just the cases whose name contains it."""
    H, Hkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    cases = []
    for name, N, K, fused in layer_products(cfg):
        cases.append((f"decode_{name}_m{batch}", lambda N=N, K=K, fused=fused, name=name: gemm_case(
            batch, N, K, fused, peaks, torch.float32 if name == "lm_head" else torch.bfloat16)))
    cases.append((f"decode_attention_b{batch}_ctx{ctx}", lambda: decode_attention_case(batch, ctx, H, Hkv, hd, page, peaks)))
    for name, N, K, fused in layer_products(cfg)[:4]:
        cases.append((f"prefill_{name}_m{prefill_tokens}", lambda N=N, K=K, fused=fused: gemm_case(prefill_tokens, N, K, fused, peaks)))
    cases.append((f"prefill_attention_t{prefill_tokens}", lambda: prefill_attention_case(prefill_tokens, H, Hkv, hd, page, peaks)))
    out = {name: run() for name, run in cases if only in name}
    ops.check_kernel_errors()
    return out


def main() -> int:
    from .config import architecture_of, lookup_architecture
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True, help="a config.json of a registered architecture")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--prefill", type=int, default=2048)
    ap.add_argument("--only", default="", help="just the cases whose name contains this (e.g. prefill_attention, decode_attention, decode_o)")
    ap.add_argument("--whole-tiles", action="store_true", help="many-token products without sharing tiles between CTAs (for comparison)")
    ap.add_argument("--hbm-gbs", type=float, default=6650.0)
    ap.add_argument("--bf16-tflops", type=float, default=1590.0)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("qorvix_b200.kernel_bench needs a CUDA device")
    raw = json.load(open(args.config))
    cfg = lookup_architecture(architecture_of(raw)).config_from_dict(raw)
    peaks = {"hbm_gbs": args.hbm_gbs, "bf16_tflops": args.bf16_tflops}
    if args.whole_tiles:
        ops.gemm_share_tiles(False)
    for name, fig in headline_kernels(cfg, args.batch, args.ctx, args.prefill, peaks, only=args.only).items():
        print(f"{name:34s} {json.dumps(fig)}", flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
