#!/usr/bin/env python3
"""Decode and prefill throughput of the Llama-3.1-8B shape with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  `value` is decoded tokens per second at batch 8 with 1,024-token
contexts, timed on the device with CUDA events around K decode steps of the engine's step
function (greedy sampling on the device feeds each step's tokens to the next).  `e2e` is the
same through the public Python API (LLM / Scheduler.step): host token lists in, sampled ids
back to the host every step, pinned-memory copies counted.  `prefill` is one 2,048-token
prompt; `roofline` is the bytes a decode step must read (every weight it uses once, the cache
of the live requests) over its time, against the measured copy bandwidth; `points` holds
decode at batch 1 and 64.  The reference has no Python package and no batched, bfloat16 or
sm_100 path; its arm prints an `unavailable` line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}

LLAMA31_8B = dict(architectures=["LlamaForCausalLM"], vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                  num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                  max_position_embeddings=8192, rms_norm_eps=1e-5, rope_theta=500000.0,
                  rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                    original_max_position_embeddings=8192),
                  tie_word_embeddings=False, hidden_act="silu")


LLAMA32_1B = dict(architectures=["LlamaForCausalLM"], vocab_size=128256, hidden_size=2048, intermediate_size=8192,
                  num_hidden_layers=16, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
                  max_position_embeddings=8192, rms_norm_eps=1e-5, rope_theta=500000.0,
                  rope_scaling=dict(rope_type="llama3", factor=32.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                    original_max_position_embeddings=8192),
                  tie_word_embeddings=True, hidden_act="silu")

LLAMA2_13B = dict(architectures=["LlamaForCausalLM"], vocab_size=32000, hidden_size=5120, intermediate_size=13824,
                  num_hidden_layers=40, num_attention_heads=40, num_key_value_heads=40, head_dim=128,
                  max_position_embeddings=4096, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False,
                  hidden_act="silu")

SHAPES = {"llama31_8b": ("Llama-3.1-8B shape", LLAMA31_8B), "llama32_1b": ("Llama-3.2-1B shape", LLAMA32_1B),
          "llama2_13b": ("Llama-2-13B shape", LLAMA2_13B)}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs (reading only)."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self._proc = None

    def start(self):
        try:
            self._proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                           "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self._proc = None

    def _read(self):
        for line in self._proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self._proc:
            self._proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def weight_bytes(cfg, dtype_bytes=2):
    """Bytes of every weight a decode step reads once: all layer matrices and norms, the final
    norm and the output head (the embedding table is read one row per token)."""
    d, f, H, Hkv, hd, L, V = (cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                              cfg.head_dim, cfg.num_hidden_layers, cfg.vocab_size)
    per_layer = (H + 2 * Hkv) * hd * d + d * H * hd + 3 * f * d
    return (L * per_layer + V * d) * dtype_bytes + (2 * L + 1) * d * 4


def gemm_flops_per_token(cfg):
    d, f, H, Hkv, hd, L = (cfg.hidden_size, cfg.intermediate_size, cfg.num_attention_heads, cfg.num_key_value_heads,
                           cfg.head_dim, cfg.num_hidden_layers)
    return 2 * L * ((H + 2 * Hkv) * hd * d + d * H * hd + 3 * f * d)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--shape", default="llama31_8b", choices=sorted(SHAPES), help="the other shapes the baseline names")
    ap.add_argument("--mixed", action="store_true",
                    help="also time mixed steps: a 512-token prompt portion beside 32 decoded tokens at 2,048-token contexts")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a CMake C++ project with no setup.py or pyproject.toml, so the offline pip install "
                          "fails; it has no Python API, no batched step, no bfloat16 and no sm_100 build"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch
    from qorvix_b200 import LLM, LlamaConfig, SamplingParams, StepEntry
    from qorvix_b200.csrc import ops
    from qorvix_b200.weights import random_tensors

    pk = peaks()
    model_name, shape = SHAPES[args.shape]
    raw = dict(shape)
    full_layers = raw["num_hidden_layers"]
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    cfg = LlamaConfig.from_dict(raw)
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    B, ctx, K, W = args.batch, args.ctx, args.steps, args.warmup
    max_len = min(8192, cfg.max_position_embeddings)
    pool_tokens = max(64 * (ctx + K + W + 64), args.prefill_tokens + 64, B * (ctx + 2 * (K + W) + 64 + (-(-B * ctx // 4096) + B)),
                      34 * (2048 + 256) if args.mixed else 0, 0 if args.skip_points else B * (max_len + 64))
    t0 = time.time()
    tensors = dict(random_tensors(cfg, seed=0, device=dev, dtype=torch.bfloat16))
    llm = LLM(config=cfg, tensors=tensors, dtype="bfloat16", max_tokens=pool_tokens, max_concurrent=64,
              max_batch_tokens=4096, max_model_len=max_len, device=dev)
    del tensors
    runner = llm.runner
    torch.cuda.synchronize()
    load_s = time.time() - t0
    g = torch.Generator().manual_seed(1)

    def prompt(n):
        return [int(t) for t in torch.randint(0, cfg.vocab_size, (n,), generator=g)]

    def decode_device(batch, n_ctx, steps, warm):
        """Device-timed decode: `batch` requests at context n_ctx, K steps, tokens stay on the device."""
        ids = list(range(1000, 1000 + batch))
        for i in ids:                                             # real prefill of each context
            p = prompt(n_ctx - 1)
            for c in range(0, len(p), 2048):
                runner.step([StepEntry(i, p[c:c + 2048], [])])
        dec = runner.decoder(ids)                                 # greedy decode loop with device-side tokens
        dec.start([1] * batch)
        for _ in range(warm):
            dec.step()
        torch.cuda.synchronize()
        launches0 = ops.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            dec.step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        launches = ops.launch_count() - launches0
        dec.finish()
        for i in ids:
            runner.release(i)
        return ms / steps, launches

    # ---- prefill: one prompt of T tokens
    T = args.prefill_tokens
    pre_ms = []
    for it in range(3 + 2):
        p = prompt(T)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        runner.step([StepEntry("pre", p, [T - 1])], end=["pre"])
        e1.record()
        torch.cuda.synchronize()
        if it >= 2:
            pre_ms.append(e0.elapsed_time(e1))
    pre = statistics.median(pre_ms)
    H, hd, L = cfg.num_attention_heads, cfg.head_dim, cfg.num_hidden_layers
    pre_flops = T * gemm_flops_per_token(cfg) + L * 4 * H * hd * (T * (T + 1) // 2) + 2 * cfg.vocab_size * cfg.hidden_size
    prefill = {"value": T / (pre / 1e3), "tokens": T, "ms": pre, "frac": pre_flops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12)}

    # ---- decode, device-timed, with clocks sampled meanwhile
    clocks = ClockSampler()
    clocks.start()
    step_ms, launches = decode_device(B, ctx, K, W)
    clk = clocks.stop()
    value = B / (step_ms / 1e3)
    kv_bytes = B * (ctx + W + K / 2) * L * 2 * cfg.num_key_value_heads * hd * 2
    step_bytes = weight_bytes(cfg) + kv_bytes + B * cfg.hidden_size * 2
    achieved = step_bytes / (step_ms / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                "peaks": pk["source"]}

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            ms, _ = decode_device(b, ctx, max(16, K // 2), W)
            points[f"decode_b{b}"] = b / (ms / 1e3)
        ms, _ = decode_device(B, max_len - 64, max(16, K // 2), W)   # the longest context the configuration names
        points[f"decode_b{B}_ctx{max_len}"] = B / (ms / 1e3)
    if args.mixed:
        # 32 requests decode at 2,048-token contexts while a 2,048-token prompt comes in 512 tokens a step
        ids = list(range(2000, 2032))
        for i in ids:
            runner.step([StepEntry(i, prompt(2047), [])])
        times = []
        for rep in range(2):
            p = prompt(2048)
            for c in range(0, 2048, 512):
                entries = [StepEntry(i, [1], [0]) for i in ids] + [StepEntry("mixed", p[c:c + 512], [511] if c == 1536 else [])]
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                runner.step(entries, end=["mixed"] if c == 1536 else [])
                e1.record()
                torch.cuda.synchronize()
                if rep:
                    times.append(e0.elapsed_time(e1))
        for i in ids:
            runner.release(i)
        ms = statistics.median(times)
        L_, H_, hd_ = cfg.num_hidden_layers, cfg.num_attention_heads, cfg.head_dim
        flops = 544 * gemm_flops_per_token(cfg) + L_ * 4 * H_ * hd_ * (512 * 1024 + 32 * 2048) + 2 * 33 * cfg.vocab_size * cfg.hidden_size
        nbytes = weight_bytes(cfg) + (32 * 2048 + 1024) * L_ * 2 * cfg.num_key_value_heads * hd_ * 2
        points["mixed_512_prompt_32_decode"] = {"tokens_per_s": 544 / (ms / 1e3), "ms": ms,
                                                "flops_ms_at_peak": flops / (pk["bf16_tflops"] * 1e12) * 1e3,
                                                "bytes_ms_at_peak": nbytes / (pk["hbm_gbs"] * 1e9) * 1e3}

    # ---- end to end through the public API: host tokens in, sampled ids out, every step
    sched = llm.new_scheduler()
    # requests that are prefilled first decode while the others' prompts still come in: room for those rounds too
    prefill_rounds = -(-B * ctx // 4096) + B
    sp = SamplingParams.greedy_params(max_new_tokens=W + K + 8 + prefill_rounds, ignore_eos=True)
    for _ in range(B):
        sched.submit(prompt(ctx - 1), sp)
    while not sched.decoding():
        sched.step()                                              # prefill until every request decodes
    for _ in range(W):
        sched.step()
    torch.cuda.synchronize()
    h2d0 = runner.h2d_bytes
    t0 = time.perf_counter()
    for _ in range(K):
        sched.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    h2d = (runner.h2d_bytes - h2d0) / K
    ahead = sched.stats.get("ahead_steps", 0)
    sched.run_to_completion()
    print(f"[bench] end to end: {ahead} of {sched.stats['steps']} rounds were launched ahead of the host", file=sys.stderr)
    e2e = {"value": B * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B,
           "ms_per_step": e2e_s / K * 1e3}

    out = {
        "metric": f"decode tok/s at batch {B}, {ctx:,}-token contexts ({model_name}, random weights)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": step_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": model_name, "layers": cfg.num_hidden_layers, "layers_full": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": B, "seq_len": ctx, "max_model_len": max_len, "page_size": runner.page_size,
                   "prefill_tokens": T, "parallelism": "single GPU", "weights": "random N(0,0.02) bf16",
                   "l2": f"inputs larger than L2 (weights {weight_bytes(cfg) / 1e9:.1f} GB per step)", "load_s": round(load_s, 1)},
        "clocks": clk, "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline, "points": points,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
