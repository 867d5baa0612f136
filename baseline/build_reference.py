#!/usr/bin/env python3
"""Builds the reference arm of bench.py: the UNMODIFIED reference CUDA backend
(cuda/src/cuda_backend.cu and what it links: cuda/src/tensor_parallel.cpp, memory/src/*.cpp),
compiled for sm_100 straight from the reference's source tree, plus the small driver
baseline/reference_arm/ref_bench.cpp, into baseline/_ref/qorvix_ref_bench.

    python baseline/build_reference.py [--reference /path/to/QorVix]

The reference is a CMake project (no Python package), so `pip install` of it fails; this does what
its cuda/CMakeLists.txt does for the qorvix_cuda target (nvcc, cuBLAS linked), without vcpkg.
"""
import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("QORVIX_REFERENCE", "/root/reference"))
    args = ap.parse_args()
    ref = Path(args.reference)
    if not (ref / "cuda/src/cuda_backend.cu").is_file():
        print(f"no reference source tree at {ref}", file=sys.stderr)
        return 1
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    out = HERE / "_ref"
    out.mkdir(exist_ok=True)
    srcs = [ref / "cuda/src/cuda_backend.cu", ref / "cuda/src/tensor_parallel.cpp"]
    srcs += sorted((ref / "memory/src").glob("*.cpp"))
    srcs.append(HERE / "reference_arm/ref_bench.cpp")
    cmd = [nvcc, "-std=c++20", "-O2", "-gencode", "arch=compute_100,code=sm_100",
           "-I", str(ref / "cuda/include"), "-I", str(ref / "memory/include"),
           *map(str, srcs), "-lcublas", "-o", str(out / "qorvix_ref_bench")]
    print(" ".join(cmd))
    rc = subprocess.call(cmd)
    if rc == 0:
        (out / "BUILT_FROM").write_text(f"{ref}\n" + "\n".join(str(s) for s in srcs) + "\n")
        print(f"built {out / 'qorvix_ref_bench'}")
    return rc


if __name__ == "__main__":
    sys.exit(main())
