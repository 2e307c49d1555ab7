"""Builds libqlora_cuda.so (sm_100a only) in-tree with nvcc.

Usage: python vkqlora/rs_b200/build.py [--force] [--verbose]   (run as a script: importing the
package needs the library this script produces)
The shared library is written next to this file so that it travels with the source tree.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(HERE, "libqlora_cuda.so")
OBJ_DIR = os.path.join(HERE, "build")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall"]
# Translation units whose results must match the reference bit-for-bit never fuse a*b+c.
SOURCES = {
    "api.cu": [],
    "quant_kernels.cu": ["-fmad=false"],
    "gemm_exact.cu": ["-fmad=false"],
    "adam.cu": ["-fmad=false"],
    "umma_gemm.cu": [],
    "comm.cu": [],
    "llama.cu": [],
    "attention_tc.cu": [],
    "selftest.cu": [],
}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def _newest_header() -> float:
    t = 0.0
    for root in (CSRC, os.path.join(HERE, "..", "..", "include")):
        for f in os.listdir(root):
            if f.endswith((".cuh", ".h")):
                t = max(t, os.path.getmtime(os.path.join(root, f)))
    return t


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    hdr_t = _newest_header()
    objs, rebuilt = [], False
    for src, extra in SOURCES.items():
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(o)
        if not force and os.path.exists(o) and os.path.getmtime(o) >= max(os.path.getmtime(s), hdr_t):
            continue
        cmd = [nvcc, *ARCH, *COMMON, *extra, "-c", s, "-o", o]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        rebuilt = True
    if rebuilt or force or not os.path.exists(OUT):
        cmd = [nvcc, *ARCH, "-shared", "-o", OUT, *objs]
        if verbose:
            print(" ".join(cmd), flush=True)
        subprocess.check_call(cmd)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
