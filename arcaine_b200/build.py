"""In-tree build of the CUDA library (sm_100a only) and of the C++ host-interface demo.

``nvcc`` cross-compiles without a GPU; the resulting ``libarc_sdpa.so`` sits next
to this file so it travels with a source snapshot.
"""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libarc_sdpa.so")
BENCH_BIN = os.path.join(HERE, "arc_attention_bench")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
    "--cudart", "shared", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the CUDA library cannot be built")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def sources() -> list[str]:
    out = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh", ".hpp", ".cpp"))]
    out.append(os.path.join(os.path.dirname(HERE), "include", "arc_sdpa.h"))
    return out


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile every kernel and the C ABI into ``libarc_sdpa.so``."""
    if force or _stale(LIB, sources()):
        cmd = [_nvcc(), *NVCC_FLAGS, "-shared", "-o", LIB,
               os.path.join(CSRC, "arc_sdpa.cu"), os.path.join(CSRC, "arcaine_attention.cpp"),
               os.path.join(CSRC, "arc_multi_gpu.cpp"), "-ldl"]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        subprocess.check_call(cmd)
    return LIB


def build_attention_bench(force: bool = False) -> str:
    """Compile the kbench-style C++ program that drives the library through the
    reference-shaped C++ interface (``arcaine_attention.hpp``)."""
    src = os.path.join(CSRC, "attention_bench.cu")
    if force or _stale(BENCH_BIN, [src, *sources()]):
        build_library()
        cmd = [_nvcc(), "-O2", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "--cudart", "shared", "-o", BENCH_BIN, src,
               "-L" + HERE, "-larc_sdpa", "-Xlinker", "-rpath=" + HERE]
        subprocess.check_call(cmd)
    return BENCH_BIN


if __name__ == "__main__":
    print(build_library(force=True, verbose=True))
    print(build_attention_bench(force=True))
