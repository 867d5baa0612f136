"""Compiles the .cu files of this folder for sm_100a, one shared library per file, on first
use, and loads them with ctypes.

Libraries are built in-tree (`csrc/_build/`) when that folder can be written, else in a
per-user folder under the system's temporary directory.  A library is named after its
source and a hash of everything it is built from, so a changed source never loads a stale
binary.  While nvcc runs, a line is printed now and then so that a first call does not look
hung.  There is no fallback: a missing compiler or a failed build raises.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path
from typing import Dict

CSRC = Path(__file__).resolve().parent
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--shared", "-Xcompiler", "-fPIC"]
HEADERS = ["common.cuh", "tc_common.cuh", "attention_mma.cuh", "attention_noalloc.h"]

# library name -> source file; every kernel family is its own library so that a model
# compiles only what it uses.
LIBRARIES = {
    "elementwise": "elementwise.cu",
    "gemm_simt": "gemm_simt.cu",
    "attention_generic": "attention_generic.cu",
    "sampling": "sampling.cu",
    "gemm_bf16": "gemm_bf16.cu",
    "attention_bf16": "attention_bf16.cu",
    "attention_tc": "attention_tc.cu",
    "host_runtime": "host_runtime.cpp",          # host-side cache bookkeeping: plain C++, no CUDA
    "ref": "ref/ref_model.cpp",                  # the kernels' plain C++ twins and a whole-model forward: host only
    "executor": "host/executor_api.cpp",         # the native step executor behind a C interface (host code, CUDA runtime calls)
}
# host code that calls the CUDA runtime: compiled and linked by nvcc (no device code in it)
CUDA_HOST_LIBRARIES = {"executor"}
# the native command line: an executable, built from these sources by nvcc
CLI_SOURCES = ["cli/qorvix_main.cpp", "host_runtime.cpp", "ref/ref_model.cpp"]
CLI_HEADERS = ["host/json.hpp", "host/safetensors.hpp", "host/model_config.hpp", "host/kernels.hpp", "host/dispatch.hpp",
               "host/executor.hpp", "host/engine.hpp", "host/scheduler.hpp", "host/step_types.hpp", "ref/ref_ops.hpp"]
KERNEL_LIBRARIES = ["elementwise", "gemm_simt", "gemm_bf16", "attention_generic", "attention_bf16", "attention_tc", "sampling"]
# what a library is built from beside its source and HEADERS (their bytes are part of its name's hash)
EXTRA_SOURCES = {
    "host_runtime": ["host/dispatch.hpp"],
    "executor": ["host/executor.hpp", "host/kernels.hpp", "host/dispatch.hpp"],
    "ref": ["ref/ref_ops.hpp", "host/json.hpp", "host/safetensors.hpp", "host/model_config.hpp"],
}
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[qorvix_b200] {msg}", file=sys.stderr, flush=True)


def find_host_compiler() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and (os.path.isfile(cand) or shutil.which(cand)):
            return shutil.which(cand) or cand
    return find_nvcc()             # nvcc hands .cpp files to its host compiler


def find_nvcc() -> str:
    for cand in (os.environ.get("QORVIX_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc was not found (looked at $QORVIX_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
                           "the CUDA kernels cannot be built and there is no fallback")


def build_dir() -> Path:
    override = os.environ.get("QORVIX_BUILD_DIR")
    cands = [Path(override)] if override else []
    cands += [CSRC / "_build", Path(tempfile.gettempdir()) / f"qorvix_b200_build_{os.getuid()}"]
    for d in cands:
        try:
            d.mkdir(parents=True, exist_ok=True)
            probe = d / f".w{os.getpid()}"
            probe.write_text("")
            probe.unlink()
            return d
        except OSError:
            continue
    raise KernelBuildError(f"no writable build folder among {', '.join(map(str, cands))}")


def _source_hash(src: Path, extra=()) -> str:
    h = hashlib.sha256()
    for p in [src] + [CSRC / x for x in HEADERS] + [CSRC / x for x in extra]:
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:12]


def library_path(name: str) -> Path:
    src = CSRC / LIBRARIES[name]
    return build_dir() / f"qv_{name}-{_source_hash(src, EXTRA_SOURCES.get(name, ()))}.so"


def compile_library(name: str, verbose: bool = True) -> Path:
    """Builds one library if it is not there yet; returns its path."""
    if name not in LIBRARIES:
        raise KernelBuildError(f"unknown kernel library '{name}'")
    src = CSRC / LIBRARIES[name]
    if not src.is_file():
        raise KernelBuildError(f"{src} is missing")
    out = library_path(name)
    if out.is_file():
        return out
    tmp = out.with_name(out.name + f".tmp{os.getpid()}")
    if name in CUDA_HOST_LIBRARIES:
        cmd = [find_nvcc(), "-O2", "-std=c++17", "--shared", "-Xcompiler", "-fPIC", "-Wno-deprecated-gpu-targets", "-I", str(CSRC),
               "-o", str(tmp), str(src), "-ldl"]
        if verbose:
            _say(f"compiling {src.name} ...")
    elif src.suffix == ".cpp":
        cxx = find_host_compiler()
        flags = ["--shared", "-Xcompiler", "-fPIC", "-O2", "-std=c++17"] if os.path.basename(cxx).startswith("nvcc") else HOST_FLAGS
        cmd = [cxx, *flags, "-I", str(CSRC), "-o", str(tmp), str(src)]
        if verbose:
            _say(f"compiling {src.name} ...")
    else:
        cmd = [find_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-o", str(tmp), str(src)]
        if verbose:
            _say(f"compiling {src.name} for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            _say(f"  still compiling {src.name} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    log, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        try:
            tmp.unlink()
        except OSError:
            pass
        raise KernelBuildError(f"the compiler failed on {src.name}:\n{log}")
    os.replace(tmp, out)
    for old in out.parent.glob(f"qv_{name}-*.so"):      # drop binaries of older sources
        if old != out:
            try:
                old.unlink()
            except OSError:
                pass
    if verbose:
        _say(f"  built {out.name} in {time.time() - t0:.1f} s")
    return out


def load_library(name: str) -> ctypes.CDLL:
    """The loaded library, compiled first if need be."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = compile_library(name)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise KernelBuildError(f"could not load {path}: {e}") from None
            _loaded[name] = lib
        return lib


def write_manifest() -> Path:
    """Builds the kernel libraries if need be and writes `kernels.manifest` beside them: the lines
    name=path that the native executor and the native command line load their kernels from."""
    lines = [f"{n}={compile_library(n)}" for n in KERNEL_LIBRARIES]
    out = build_dir() / "kernels.manifest"
    text = "\n".join(lines) + "\n"
    if not out.is_file() or out.read_text() != text:
        tmp = out.with_name(out.name + f".tmp{os.getpid()}")
        tmp.write_text(text)
        os.replace(tmp, out)
    return out


def build_cli(verbose: bool = True) -> Path:
    """The native command line (csrc/cli/qorvix_main.cpp with the engine, scheduler, cache bookkeeping
    and plain C++ decoder it is made of) as an executable beside the libraries; returns its path."""
    h = hashlib.sha256()
    for rel in CLI_SOURCES + CLI_HEADERS:
        h.update((CSRC / rel).read_bytes())
    out = build_dir() / f"qorvix_native-{h.hexdigest()[:12]}"
    write_manifest()
    if out.is_file():
        return out
    tmp = out.with_name(out.name + f".tmp{os.getpid()}")
    cmd = [find_nvcc(), "-O2", "-std=c++17", "-Wno-deprecated-gpu-targets", "-I", str(CSRC), "-o", str(tmp),
           *[str(CSRC / x) for x in CLI_SOURCES], "-ldl"]
    if verbose:
        _say("compiling the native command line ...")
    t0 = time.time()
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise KernelBuildError(f"the compiler failed on the native command line:\n{proc.stdout}")
    os.replace(tmp, out)
    for old in out.parent.glob("qorvix_native-*"):
        if old != out and ".tmp" not in old.name:
            try:
                old.unlink()
            except OSError:
                pass
    if verbose:
        _say(f"  built {out.name} in {time.time() - t0:.1f} s")
    return out


def build_issue_bench(verbose: bool = True) -> Path:
    """The microbenchmark of what issuing tensor-core products costs a warp (csrc/bench/mma_issue.cu), as an
    executable beside the libraries; returns its path."""
    src = CSRC / "bench" / "mma_issue.cu"
    out = build_dir() / f"mma_issue-{_source_hash(src)}"
    if out.is_file():
        return out
    tmp = out.with_name(out.name + f".tmp{os.getpid()}")
    cmd = [find_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-I", str(CSRC),
           "-o", str(tmp), str(src)]
    if verbose:
        _say("compiling the issue microbenchmark ...")
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise KernelBuildError(f"the compiler failed on {src.name}:\n{proc.stdout}")
    os.replace(tmp, out)
    for old in out.parent.glob("mma_issue-*"):
        if old != out and ".tmp" not in old.name:
            try:
                old.unlink()
            except OSError:
                pass
    return out


def build_all(verbose: bool = True) -> list:
    built = [compile_library(n, verbose) for n in LIBRARIES if (CSRC / LIBRARIES[n]).is_file()]
    built.append(build_cli(verbose))
    built.append(build_issue_bench(verbose))
    return built
