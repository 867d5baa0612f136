"""What issuing `tcgen05.mma` costs the issuing warp: builds and runs csrc/bench/mma_issue.cu.

    python -m qorvix_b200.issue_bench

Prints clocks per batch of eight products (M128 N128 K16, a commit after each batch) under a branch on the
lane number and with an elected lane, with barrier waits in the loop, beside warps that poll, run FMAs or
run ex2, and after the tensor pipe has idled.  The kernels' MMA and producer warps are written after these
figures: the whole warp walks the loop and one elected lane issues.  The reference has no tensor-core path
to compare with (its products run on the CUDA cores, cuda/src/cuda_backend.cu:291-312).
"""
from __future__ import annotations

import subprocess
import sys

from .csrc import build


def main() -> int:
    exe = build.build_issue_bench()
    return subprocess.run([str(exe)]).returncode


if __name__ == "__main__":
    sys.exit(main())
