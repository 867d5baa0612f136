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
decode at batch 1 and 64, the other two shapes the baseline names (Llama-3.2-1B decode at batch
64 with 4,096-token contexts and its prefill; Llama-2-13B mixed steps of a 512-token portion
beside 32 decoded tokens) each with its own bound, and `kernels` the step's dominant kernels
alone (captured-chain timing) with their fractions of the measured peaks.

`--impl reference` times the UNMODIFIED reference CUDA backend (float32, one token of one session
per forward) at the same shape, batch, contexts, steps and warm-up through the small driver
baseline/reference_arm/ref_bench.cpp, built by baseline/build_reference.py into baseline/_ref/;
nothing of qorvix_b200 is imported on that path.
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

def _shape(name):
    """config.json of a shape the baseline names (baseline/configs/<name>.json)."""
    with open(os.path.join(ROOT, "baseline", "configs", name + ".json")) as f:
        return json.load(f)


SHAPES = {"llama31_8b": ("Llama-3.1-8B shape", _shape("llama31_8b")), "llama32_1b": ("Llama-3.2-1B shape", _shape("llama32_1b")),
          "llama2_13b": ("Llama-2-13B shape", _shape("llama2_13b"))}


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


def reference_arm(args) -> int:
    """Runs baseline/_ref/qorvix_ref_bench (the reference's own GpuModel::forward loop) and prints the
    bench line for it.  No module of this package is imported here."""
    binary = os.path.join(ROOT, "baseline", "_ref", "qorvix_ref_bench")
    if not os.path.isfile(binary):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/qorvix_ref_bench is not built (python baseline/build_reference.py "
                          "compiles the reference's CUDA backend from its source tree; pip cannot install it: it is a CMake project)"}))
        return 0
    model_name, c = SHAPES[args.shape]
    layers = args.layers or c["num_hidden_layers"]
    B, ctx, K, W, T = args.batch, args.ctx, args.steps, max(args.warmup, 3), args.prefill_tokens
    cmd = [binary, "--layers", str(layers), "--hidden", str(c["hidden_size"]), "--heads", str(c["num_attention_heads"]),
           "--kv-heads", str(c["num_key_value_heads"]), "--head-dim", str(c["head_dim"]), "--ffn", str(c["intermediate_size"]),
           "--vocab", str(c["vocab_size"]), "--eps", str(c["rms_norm_eps"]), "--rope-theta", str(c["rope_theta"]),
           "--batch", str(B), "--ctx", str(ctx), "--steps", str(K), "--warmup", str(W), "--prefill", str(T),
           "--fill", "1" if args.reference_fill == "all" else "0"]
    clocks = ClockSampler()
    clocks.start()
    try:
        proc = subprocess.run(cmd, capture_output=True, text=True, timeout=args.reference_timeout)
    except subprocess.TimeoutExpired:
        clocks.stop()
        print(json.dumps({"impl": "reference", "unavailable": f"the reference binary did not finish within {args.reference_timeout} s at this shape"}))
        return 0
    clk = clocks.stop()
    sys.stderr.write(proc.stderr[-2000:])
    try:
        r = json.loads(proc.stdout.strip().splitlines()[-1])
    except (IndexError, ValueError):
        r = {"error": f"exit code {proc.returncode}, no result line"}
    if proc.returncode != 0 or "error" in r:
        print(json.dumps({"impl": "reference", "unavailable": f"the reference binary failed: {r.get('error', proc.returncode)}"}))
        return 0
    ms = r["decode_ms_per_step"]
    launches_per_forward = 1 + layers * 19 + 2             # its kernels per forward (cuda/src/cuda_backend.cu:1488-1510)
    out = {
        "metric": f"decode tok/s at batch {B}, {ctx:,}-token contexts ({model_name}, random weights)",
        "value": B / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic", "impl": "reference",
        "config": {"model": model_name, "layers": layers, "layers_full": c["num_hidden_layers"], "hidden": c["hidden_size"],
                   "heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"],
                   "intermediate": c["intermediate_size"], "vocab": c["vocab_size"], "global_batch": B, "seq_len": ctx,
                   "prefill_tokens": T, "parallelism": "single GPU",
                   "weights": "random float32 (the reference's GPU model takes F32 or GGUF-quantized weights, no bfloat16)",
                   "step": "one GpuModel::forward per session, its forwardBatch default; llama3 rope scaling absent in the reference",
                   "contexts": "every session filled through forward()" if r.get("filled") else
                               "session 0 filled by the timed prefill, the others decode over unwritten cache slices (same bytes read)",
                   "l2": f"inputs larger than L2 (float32 weights {weight_bytes_raw(c, layers, 4) / 1e9:.1f} GB per forward)",
                   "load_s": r.get("load_s")},
        "clocks": clk,
        "e2e": {"value": B / (r["decode_wall_ms_per_step"] / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": r["h2d_bytes_per_step"],
                "d2h_bytes_per_step": r["d2h_bytes_per_step"], "ms_per_step": r["decode_wall_ms_per_step"]},
        "gpu_launches": launches_per_forward * B * K,
        "prefill": {"value": T / (r["prefill_ms"] / 1e3) if r["prefill_ms"] else None, "tokens": T, "ms": r["prefill_ms"]},
    }
    print(json.dumps(out))
    return 0


def weight_bytes_raw(c, layers, dtype_bytes):
    d, f, H, Hkv, hd, V = (c["hidden_size"], c["intermediate_size"], c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"],
                           c["vocab_size"])
    return (layers * ((H + 2 * Hkv) * hd * d + d * H * hd + 3 * f * d) + V * d) * dtype_bytes


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
    ap.add_argument("--skip-points", action="store_true", help="only the headline shape: no batch 1/64, no other shapes, no kernels")
    ap.add_argument("--shape", default="llama31_8b", choices=sorted(SHAPES), help="the headline shape")
    ap.add_argument("--reference-timeout", type=int, default=1500)
    ap.add_argument("--reference-fill", default="first", choices=["first", "all"],
                    help="reference arm: 'all' fills every session's context through its forward() (four more minutes at its speed); "
                         "'first' only the first session's, by the timed prefill (the step time is the same: its kernels read the same bytes)")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)

    import gc

    import torch
    from qorvix_b200 import LLM, LlamaConfig, SamplingParams, StepEntry
    from qorvix_b200 import kernel_bench
    from qorvix_b200.csrc import ops
    from qorvix_b200.weights import random_tensors

    pk = peaks()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    K, W = args.steps, args.warmup
    g = torch.Generator().manual_seed(1)

    def prompt(vocab, n):
        return [int(t) for t in torch.randint(0, vocab, (n,), generator=g)]

    def load(shape_key, layers, pool_tokens, max_len, concurrent=64):
        raw = dict(SHAPES[shape_key][1])
        if layers:
            raw["num_hidden_layers"] = layers
        cfg = LlamaConfig.from_dict(raw)
        t0 = time.time()
        tensors = dict(random_tensors(cfg, seed=0, device=dev, dtype=torch.bfloat16))
        llm = LLM(config=cfg, tensors=tensors, dtype="bfloat16", max_tokens=pool_tokens, max_concurrent=concurrent,
                  max_batch_tokens=4096, max_model_len=max_len, device=dev)
        del tensors
        torch.cuda.synchronize()
        return cfg, llm, time.time() - t0

    def decode_device(runner, cfg, batch, n_ctx, steps, warm):
        """Device-timed decode: `batch` requests at context n_ctx, `steps` steps, tokens stay on the device."""
        ids = list(range(1000, 1000 + batch))
        for i in ids:                                             # real prefill of each context
            p = prompt(cfg.vocab_size, n_ctx - 1)
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
        ops.check_kernel_errors()                                 # a kernel that gave up on a wait makes the number void
        for i in ids:
            runner.release(i)
        return ms / steps, launches

    def prefill_time(runner, cfg, T):
        pre_ms = []
        for it in range(3 + 2):
            p = prompt(cfg.vocab_size, T)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            runner.step([StepEntry("pre", p, [T - 1])], end=["pre"])
            e1.record()
            torch.cuda.synchronize()
            if it >= 2:
                pre_ms.append(e0.elapsed_time(e1))
        ops.check_kernel_errors()
        pre = statistics.median(pre_ms)
        H, hd, L = cfg.num_attention_heads, cfg.head_dim, cfg.num_hidden_layers
        flops = T * gemm_flops_per_token(cfg) + L * 4 * H * hd * (T * (T + 1) // 2) + 2 * cfg.vocab_size * cfg.hidden_size
        return {"value": T / (pre / 1e3), "tokens": T, "ms": pre, "frac": flops / (pre / 1e3) / (pk["bf16_tflops"] * 1e12)}

    def decode_roofline(cfg, batch, n_ctx, warm, steps, step_ms):
        L, hd = cfg.num_hidden_layers, cfg.head_dim
        kv_bytes = batch * (n_ctx + warm + steps / 2) * L * 2 * cfg.num_key_value_heads * hd * 2
        nbytes = weight_bytes(cfg) + kv_bytes + batch * cfg.hidden_size * 2      # a tied head is the embedding table, read once as the head
        achieved = nbytes / (step_ms / 1e3) / 1e9
        return {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                "peaks": pk["source"]}

    # ---------------------------------------------------------------- the headline shape
    model_name = SHAPES[args.shape][0]
    full_layers = SHAPES[args.shape][1]["num_hidden_layers"]
    B, ctx, T = args.batch, args.ctx, args.prefill_tokens
    max_len = min(8192, SHAPES[args.shape][1]["max_position_embeddings"])
    pool_tokens = max(64 * (ctx + K + W + 64), T + 64, B * (ctx + 2 * (K + W) + 64 + (-(-B * ctx // 4096) + B)),
                      0 if args.skip_points else B * (max_len + 64))
    cfg, llm, load_s = load(args.shape, args.layers, pool_tokens, max_len)
    runner = llm.runner
    prefill = prefill_time(runner, cfg, T)

    clocks = ClockSampler()
    clocks.start()
    step_ms, launches = decode_device(runner, cfg, B, ctx, K, W)
    clk = clocks.stop()
    value = B / (step_ms / 1e3)
    roofline = decode_roofline(cfg, B, ctx, W, K, step_ms)

    # ---------------------------------------------------------------- end to end through the public API: host tokens in, sampled ids out
    sched = llm.new_scheduler()
    # requests that are prefilled first decode while the others' prompts still come in: room for those rounds too
    prefill_rounds = -(-B * ctx // 4096) + B
    sp = SamplingParams.greedy_params(max_new_tokens=W + K + 8 + prefill_rounds, ignore_eos=True)
    for _ in range(B):
        sched.submit(prompt(cfg.vocab_size, ctx - 1), sp)
    while not sched.decoding():
        sched.step()                                              # prefill until every request decodes
    for _ in range(W):
        sched.step()
    torch.cuda.synchronize()
    h2d0 = runner.h2d_bytes
    ahead0 = sched.stats.get("ahead_steps", 0)
    t0 = time.perf_counter()
    for _ in range(K):
        sched.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    h2d = (runner.h2d_bytes - h2d0) / K
    ahead = sched.stats.get("ahead_steps", 0) - ahead0
    sched.run_to_completion()
    ops.check_kernel_errors()
    print(f"[bench] end to end: {ahead} of the {K} timed rounds were launched ahead of the host", file=sys.stderr)
    e2e = {"value": B * K / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B,
           "ms_per_step": e2e_s / K * 1e3, "rounds_ahead": ahead}

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            ms, _ = decode_device(runner, cfg, b, ctx, max(16, K // 2), W)
            points[f"decode_b{b}"] = b / (ms / 1e3)
            points[f"decode_b{b}_hbm_frac"] = round(decode_roofline(cfg, b, ctx, W, max(16, K // 2), ms)["frac"], 4)
        ms, _ = decode_device(runner, cfg, B, max_len - 64, max(16, K // 2), W)   # the longest context the configuration names
        points[f"decode_b{B}_ctx{max_len}"] = B / (ms / 1e3)
        points[f"decode_b{B}_ctx{max_len}_hbm_frac"] = round(decode_roofline(cfg, B, max_len - 64, W, max(16, K // 2), ms)["frac"], 4)

    kernels = {}
    if not args.skip_points:
        # ---------------------------------------------------------------- the step's dominant kernels, each alone
        kernels = kernel_bench.headline_kernels(cfg, B, ctx, T, pk, page=runner.page_size)
        del sched, runner, llm
        gc.collect()
        torch.cuda.empty_cache()

        # ---------------------------------------------------------------- Llama-3.2-1B: decode at batch 64, 4,096-token contexts; prefill
        b1, c1 = 64, 4096
        k1 = max(16, K // 2)
        cfg1, llm1, _ = load("llama32_1b", 0, b1 * (c1 + 2 * (k1 + W) + 64), 8192)
        ms, _ = decode_device(llm1.runner, cfg1, b1, c1, k1, W)
        points["llama32_1b_decode_b64_ctx4096"] = {"tokens_per_s": b1 / (ms / 1e3), "ms": ms,
                                                   "hbm_frac": round(decode_roofline(cfg1, b1, c1, W, k1, ms)["frac"], 4)}
        pre1 = prefill_time(llm1.runner, cfg1, 2048)
        points["llama32_1b_prefill_2048"] = {"tokens_per_s": pre1["value"], "ms": pre1["ms"], "bf16_frac": round(pre1["frac"], 4)}
        del llm1
        gc.collect()
        torch.cuda.empty_cache()

        # ---------------------------------------------------------------- Llama-2-13B: mixed steps
        # 32 requests decode at 2,048-token contexts while a 2,048-token prompt comes in 512 tokens a step
        cfg13, llm13, _ = load("llama2_13b", 0, 34 * (2048 + 256), 4096)
        r13 = llm13.runner
        ids = list(range(2000, 2032))
        for i in ids:
            r13.step([StepEntry(i, prompt(cfg13.vocab_size, 2047), [])])
        times = []
        for rep in range(3):
            p = prompt(cfg13.vocab_size, 2048)
            for c in range(0, 2048, 512):
                entries = [StepEntry(i, [1], [0]) for i in ids] + [StepEntry("mixed", p[c:c + 512], [511] if c == 1536 else [])]
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                r13.step(entries, end=["mixed"] if c == 1536 else [])
                e1.record()
                torch.cuda.synchronize()
                if rep:
                    times.append(e0.elapsed_time(e1))
        ops.check_kernel_errors()
        ms = statistics.median(times)
        L_, H_, hd_ = cfg13.num_hidden_layers, cfg13.num_attention_heads, cfg13.head_dim
        flops = 544 * gemm_flops_per_token(cfg13) + L_ * 4 * H_ * hd_ * (512 * 1024 + 32 * 2048) + 2 * 33 * cfg13.vocab_size * cfg13.hidden_size
        nbytes = weight_bytes(cfg13) + (32 * 2048 + 1024) * L_ * 2 * cfg13.num_key_value_heads * hd_ * 2
        flops_ms, bytes_ms = flops / (pk["bf16_tflops"] * 1e12) * 1e3, nbytes / (pk["hbm_gbs"] * 1e9) * 1e3
        points["llama2_13b_mixed_512_32"] = {"tokens_per_s": 544 / (ms / 1e3), "ms": ms, "flops_ms_at_peak": flops_ms,
                                             "bytes_ms_at_peak": bytes_ms, "frac_of_bound": round(max(flops_ms, bytes_ms) / ms, 4)}
        del r13, llm13
        gc.collect()
        torch.cuda.empty_cache()

    out = {
        "metric": f"decode tok/s at batch {B}, {ctx:,}-token contexts ({model_name}, random weights)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": step_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "impl": "ours",
        "config": {"model": model_name, "layers": cfg.num_hidden_layers, "layers_full": full_layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "global_batch": B, "seq_len": ctx, "max_model_len": max_len, "page_size": 16,
                   "prefill_tokens": T, "parallelism": "single GPU", "weights": "random N(0,0.02) bf16",
                   "l2": f"inputs larger than L2 (weights {weight_bytes(cfg) / 1e9:.1f} GB per step)", "load_s": round(load_s, 1)},
        "clocks": clk, "e2e": e2e, "gpu_launches": launches, "prefill": prefill, "roofline": roofline, "points": points,
        "kernels": kernels,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
