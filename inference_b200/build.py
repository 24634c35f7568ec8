"""Builds libinferop_b200.so (sm_100a only) in-tree with nvcc.

    python -m inference_b200.build [--verbose]

The shared object lands in ``inference_b200/lib/`` and is what the ctypes
binding, the tests and the benchmark load; there is no other code path.
"""
from __future__ import annotations

import os
import subprocess
import sys

_PKG = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG)
CSRC = os.path.join(_PKG, "csrc")
LIB_DIR = os.path.join(_PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libinferop_b200.so")

SOURCES = ["api.cu", "tensormap.cu", "quant.cu", "gemm_sm100.cu", "gemm_pair_sm100.cu", "gemm_decode_sm100.cu", "moe.cu", "reduce.cu", "norm_rope.cu", "attention.cu"]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _stale(obj: str, src: str) -> bool:
    if not os.path.exists(obj):
        return True
    newest = max(os.path.getmtime(os.path.join(CSRC, f)) for f in os.listdir(CSRC))
    newest = max(newest, *(os.path.getmtime(os.path.join(_ROOT, "include", f))
                           for f in ("inferop_b200.h",)))
    return os.path.getmtime(obj) < newest


def build(verbose: bool = False, force: bool = False) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    inc = ["-I", os.path.join(_ROOT, "include"), "-I", CSRC]
    objs = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(LIB_DIR, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, src):
            cmd = [_nvcc(), *NVCC_FLAGS, *inc, "-c", os.path.join(CSRC, src), "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
                print(" ".join(cmd), flush=True)
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT,
                                                text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            print(f"--- {src}\n{out}", flush=True)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if procs or not os.path.exists(LIB_PATH):
        cmd = [_nvcc(), "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fvisibility=hidden"]
        subprocess.run(cmd, check=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force="--force" in sys.argv))
