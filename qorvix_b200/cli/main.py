"""Command line in the reference's manner (core/src/main.cpp:4280-4324 dispatches on the first
word; flags are `--flag value`, core/src/main.cpp:269-303):

  qorvix generate <model_dir> --tokens 1,2,3 | --random-prompt N  [--max N] [--temp T] [--top-k K]
                  [--top-p P] [--seed S] [--dtype bfloat16|float32]
  qorvix bench <model_dir> [--prompt N] [--gen N] [--warmup N] [--runs N] [--batch B] [--json]
  qorvix model-info <model_dir>
  qorvix gpu-check <model_dir> [--tokens ...]      engine float32 and bfloat16 against the plain C++ CPU model
  qorvix random-model <out_dir> --config <config.json> [--seed S] [--dtype bfloat16|float32]

`generate` keeps the reference's option names and defaults (--max 128, --temp 0.8, --top-k 40,
--top-p 0.95, --seed 0; core/src/main.cpp:499-503) and its summary lines.  Prompts are token
ids, since tokenizers are out of scope.
"""
from __future__ import annotations

import json
import statistics
import sys
import time
from pathlib import Path
from typing import List


def flag_value(args: List[str], flag: str, default=None):
    for i in range(len(args) - 1):
        if args[i] == flag:
            return args[i + 1]
    return default


def has_flag(args: List[str], flag: str) -> bool:
    return flag in args


USAGE = __doc__.split("\n\n")[1]


def _prompt_from(args, vocab):
    import torch
    toks = flag_value(args, "--tokens")
    if toks:
        return [int(t) for t in toks.replace(" ", "").split(",") if t]
    n = flag_value(args, "--random-prompt")
    if n:
        g = torch.Generator().manual_seed(int(flag_value(args, "--seed", 0)))
        return [int(t) for t in torch.randint(0, vocab, (int(n),), generator=g)]
    return None


def cmd_generate(args) -> int:
    from ..config import load_config
    from ..engine.generate import LLM
    from ..sampling import SamplingParams
    if len(args) < 2:
        print("usage: qorvix generate <model_dir> --tokens 1,2,3 | --random-prompt N [--max N] [--temp T] "
              "[--top-k K] [--top-p P] [--seed S] [--dtype bfloat16|float32]", file=sys.stderr)
        return 1
    model = args[1]
    cfg = load_config(model)
    prompt = _prompt_from(args, cfg.vocab_size)
    if not prompt:
        print("error: give the prompt as --tokens 1,2,3 or --random-prompt N", file=sys.stderr)
        return 1
    d = SamplingParams()
    sp = SamplingParams(temperature=float(flag_value(args, "--temp", d.temperature)),
                        top_k=int(flag_value(args, "--top-k", d.top_k)),
                        top_p=float(flag_value(args, "--top-p", d.top_p)),
                        seed=int(flag_value(args, "--seed", d.seed)),
                        max_new_tokens=int(flag_value(args, "--max", d.max_new_tokens)))
    t0 = time.perf_counter()
    max_seq = len(prompt) + sp.max_new_tokens + 4            # as the reference sizes its engine (main.cpp:566)
    llm = LLM(model, dtype=flag_value(args, "--dtype", "bfloat16"), max_tokens=max_seq + 64,
              max_concurrent=1, max_model_len=max_seq)
    load_s = time.perf_counter() - t0
    print(" ".join(map(str, prompt)), flush=True)
    res = llm.generate([prompt], sp, on_token=lambda rid, tok: print(tok, end=" ", flush=True))[0]
    st = llm.last_stats
    forwards = len(prompt) + len(res.tokens)
    print(f"\n\n[cuda | {len(prompt)} prompt tokens, {len(res.tokens)} generated{', eos' if res.hit_eos else ''}]")
    print(f"[load {load_s:.1f}s | {forwards} forwards in {st['seconds']:.2f}s = {forwards / max(st['seconds'], 1e-9):.2f} tok/s]")
    return 0


def cmd_model_info(args) -> int:
    from ..config import load_config, lookup_architecture
    if len(args) < 2:
        print("usage: qorvix model-info <model_dir>", file=sys.stderr)
        return 1
    cfg = load_config(args[1])
    spec = lookup_architecture(cfg.architecture).build_spec(cfg)
    n_params = 0
    for shape, _ in spec.tensor_table().values():
        k = 1
        for s in shape:
            k *= s
        n_params += k
    print(json.dumps(dict(cfg.to_dict(), parameters=n_params, layers=len(spec.layers)), indent=1))
    return 0


def cmd_gpu_check(args) -> int:
    """The reference's gpu-check (core/src/main.cpp:3629-3680): the same prompt through the GPU engine and
    through a CPU model, logits compared position by position; PASS when the argmax agrees everywhere
    and the relative error is under 5e-2 (core/src/main.cpp:3660-3678).  The CPU side here is the plain
    C++ decoder of csrc/ref/, which shares nothing with the engine; both engine paths are checked,
    float32 by the reference's rule, bfloat16 with the argmax demanded only where the CPU model's two
    best logits lie further apart than twice the largest error."""
    import numpy as np
    from ..config import load_config
    from ..csrc import ops
    from ..csrc.ref import RefModel
    from ..engine import ModelRunner, StepEntry
    if len(args) < 2:
        print("usage: qorvix gpu-check <model_dir> [--tokens 1,2,3 | --random-prompt N]", file=sys.stderr)
        return 1
    cfg = load_config(args[1])
    prompt = _prompt_from(args, cfg.vocab_size) or _prompt_from(args + ["--random-prompt", "32"], cfg.vocab_size)
    want = RefModel(args[1]).logits(prompt).astype(np.float64)
    scale = max(float(np.abs(want).max()), 1e-30)
    top2 = np.sort(want, axis=-1)[:, -2:]
    gap = top2[:, 1] - top2[:, 0]
    all_ok = True
    for dt in ("float32", "bfloat16"):
        r = ModelRunner(args[1], dtype=dt, max_tokens=len(prompt) + 64, max_requests=1)
        got = r.step([StepEntry(0, prompt, list(range(len(prompt))))], end=[0]).double().cpu().numpy()
        ops.check_kernel_errors()
        del r
        max_abs = float(np.abs(got - want).max())
        rel = max_abs / scale
        same = got.argmax(-1) == want.argmax(-1)
        must = np.ones(len(prompt), dtype=bool) if dt == "float32" else gap > 2 * max_abs
        ok = rel < 5e-2 and bool(same[must].all())
        all_ok = all_ok and ok
        print(f"gpu-check {dt}: {len(prompt)} positions | max abs err {max_abs:.3e} | rel err {rel:.3e} | "
              f"argmax equal {int(same.sum())}/{len(prompt)} ({int(must.sum())} decisive) | {'ok' if ok else 'MISMATCH'}")
    print("PASS" if all_ok else "FAIL")
    return 0 if all_ok else 1


def cmd_random_model(args) -> int:
    import torch
    from ..config import architecture_of, lookup_architecture
    from ..weights import write_random_model
    cfg_path = flag_value(args, "--config")
    if len(args) < 2 or not cfg_path:
        print("usage: qorvix random-model <out_dir> --config <config.json> [--seed S] [--dtype bfloat16|float32]", file=sys.stderr)
        return 1
    raw = json.loads(Path(cfg_path).read_text())
    cfg = lookup_architecture(architecture_of(raw)).config_from_dict(raw)
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[flag_value(args, "--dtype", "bfloat16")]
    out = write_random_model(args[1], cfg, int(flag_value(args, "--seed", 0)), dt)
    print(f"wrote {out}/config.json and model.safetensors")
    return 0


def cmd_bench(args) -> int:
    """The reference's bench (runtime/include/qorvix/runtime/benchmark.hpp:54-115): prefill P tokens,
    then decode G tokens; warm-up runs discarded, medians reported.  --batch B decodes B requests at once."""
    import torch
    from ..config import load_config
    from ..engine import ModelRunner, StepEntry
    if len(args) < 2:
        print("usage: qorvix bench <model_dir> [--prompt N] [--gen N] [--warmup N] [--runs N] [--batch B] [--dtype D] [--json]", file=sys.stderr)
        return 1
    P, G = int(flag_value(args, "--prompt", 64)), int(flag_value(args, "--gen", 128))
    warm, runs, B = int(flag_value(args, "--warmup", 1)), int(flag_value(args, "--runs", 3)), int(flag_value(args, "--batch", 1))
    cfg = load_config(args[1])
    t0 = time.perf_counter()
    r = ModelRunner(args[1], dtype=flag_value(args, "--dtype", "bfloat16"), max_tokens=B * (P + G + 64), max_requests=B)
    load_s = time.perf_counter() - t0
    stream = [(i * 2654435761) % cfg.vocab_size for i in range(P + G)]      # the reference's token stream (benchmark.hpp:75)
    pre, dec = [], []
    for it in range(warm + runs):
        torch.cuda.synchronize()
        t = time.perf_counter()
        r.step([StepEntry(b, stream[:P], [P - 1]) for b in range(B)])
        torch.cuda.synchronize()
        t_pre = time.perf_counter() - t
        t = time.perf_counter()
        for g in range(G):
            r.step([StepEntry(b, [stream[P + g]], [0]) for b in range(B)])
        torch.cuda.synchronize()
        t_dec = time.perf_counter() - t
        for b in range(B):
            r.release(b)
        if it >= warm:
            pre.append(B * P / t_pre)
            dec.append(t_dec / G * 1e3)
    res = {"backend": "cuda", "prompt_tokens": P, "gen_tokens": G, "batch": B, "timed_runs": runs, "load_sec": load_s,
           "prefill_tok_per_sec": statistics.median(pre), "decode_tok_per_sec": B * 1e3 / statistics.median(dec),
           "decode_ms_per_tok_median": statistics.median(dec), "decode_ms_per_tok_min": min(dec),
           "decode_ms_per_tok_max": max(dec)}
    if has_flag(args, "--json"):
        print(json.dumps(res))
    else:
        print(f"\n==== qorvix bench: cuda ====\n  model          : {args[1]}\n  load           : {load_s:.2f} s\n"
              f"  prompt / gen   : {P} / {G} tokens (batch {B})\n  prefill        : {res['prefill_tok_per_sec']:.1f} tok/s\n"
              f"  decode         : {res['decode_tok_per_sec']:.1f} tok/s ({res['decode_ms_per_tok_median']:.2f} ms/step, "
              f"min {res['decode_ms_per_tok_min']:.2f} max {res['decode_ms_per_tok_max']:.2f})\n  timed runs     : {runs} (median reported)")
    return 0


COMMANDS = {"generate": cmd_generate, "bench": cmd_bench, "model-info": cmd_model_info,
            "gpu-check": cmd_gpu_check, "random-model": cmd_random_model}


def main(argv=None) -> int:
    args = list(sys.argv[1:] if argv is None else argv)
    if not args or args[0] in ("-h", "--help", "help") or args[0] not in COMMANDS:
        print(USAGE, file=sys.stderr)
        return 0 if args and args[0] in ("-h", "--help", "help") else 1
    try:
        return COMMANDS[args[0]](args)
    except Exception as e:  # the reference prints "error: ..." and returns 1
        print(f"error: {e}", file=sys.stderr)
        return 1
