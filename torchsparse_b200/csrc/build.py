"""Compile the tsb200 CUDA library for sm_100a into torchsparse_b200/csrc/libtsb200.so.

Usage: python torchsparse_b200/csrc/build.py [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libtsb200.so")
SOURCES = ["lib.cu", "kmap.cu", "conv.cu", "conv_simt.cu", "conv_umma.cu", "conv_pairs.cu", "pointops.cu",
           "quantize.cu"]
HEADERS = ["common.cuh", "conv_dispatch.h", os.path.join("..", "..", "include", "tsb200.h")]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]


def _newer(a: str, b: str) -> bool:
    return (not os.path.exists(b)) or os.path.getmtime(a) > os.path.getmtime(b)


def build(force: bool = False, verbose: bool = False) -> str:
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    hdrs = [os.path.join(HERE, h) for h in HEADERS]
    objs, jobs = [], []
    for src in SOURCES:
        s = os.path.join(HERE, src)
        o = os.path.join(HERE, "build", src.replace(".cu", ".o"))
        objs.append(o)
        if force or _newer(s, o) or any(_newer(h, o) for h in hdrs):
            jobs.append((s, o))
    os.makedirs(os.path.join(HERE, "build"), exist_ok=True)

    def cc(job):
        s, o = job
        extra = os.environ.get("TSB_NVCC_EXTRA", "").split()   # e.g. -DTSB_TRACE_BUILD for a debugging build
        r = subprocess.run([nvcc, *NVCC_FLAGS, *extra, "-c", s, "-o", o], capture_output=True, text=True)
        log = o.replace(".o", ".ptxas.log")
        with open(log, "w") as f:
            f.write(r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {s}:\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        list(ex.map(cc, jobs))
    if jobs or not os.path.exists(LIB):
        subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB, *objs, "-lcudart"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
