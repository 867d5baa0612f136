"""Trace replay: feeds given token ids through a model step by step and writes logits.

It samples nothing and has no forward pass, cache or loader of its own: it drives
ModelRunner.step, the same step function, cache manager and kernels that generation uses.
The nearest things in the reference are `gpu-check` (core/src/main.cpp:3629-3680, logits
position by position against the CPU model) and its benchmark loop; neither takes a trace.

Input, one JSON object per line on standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, <out>/<step>.f32 holds the logits at the wanted
places (order of entries, then of `want`) as little-endian float32 [wanted, vocab].  After
every step a line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np

from ..csrc import ops
from .batch import StepEntry
from .runner import ModelRunner


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                   help="bfloat16: the kernels and precisions of serving; float32: everything in true 32-bit")
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to a multiple of 64); sizes the page pool")
    p.add_argument("--page-size", type=int, default=16, help="tokens per cache page (a multiple of 16 that divides 64)")
    p.add_argument("--max-requests", type=int, default=8, help="request slots")
    return p


def run(args, stdin=None, stdout=None) -> int:
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    if args.page_size <= 0 or 64 % args.page_size:
        print(f"trace_run: --page-size {args.page_size} must divide 64", file=sys.stderr)
        return 2
    runner = ModelRunner(args.model, dtype=args.dtype, max_tokens=args.max_tokens, page_size=args.page_size,
                         max_requests=args.max_requests)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", [])]
        logits = runner.step(entries, end=rec.get("end", []))
        if logits is not None and logits.shape[0] > 0:
            arr = logits.detach().float().cpu().numpy().astype("<f4", copy=False)
            tmp = out_dir / f".{step}.f32.tmp"
            arr.tofile(tmp)
            tmp.replace(out_dir / f"{step}.f32")
            ops.check_kernel_errors()              # a kernel that gave up on a barrier must not pass silently
        print(f"done {step}", file=stdout, flush=True)
    return 0


def main(argv=None) -> int:
    return run(build_parser().parse_args(argv))
