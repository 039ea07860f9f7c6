"""Builds libtq_b200.so in-tree with nvcc for sm_100a. No JIT cache, no torch."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libtq_b200.so")
ACL_LIB = os.path.join(PKG, "libtq_acl_shim.so")

CUDA_SOURCES = ["tq_ingest.cu", "tq_scatter.cu", "tq_decode.cu"]
HOST_SOURCES = ["tq_reference_abi.cpp"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "--use_fast_math=false"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libtq_b200.so cannot be built")
    return exe


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    deps = sources + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    deps.append(os.path.join(PKG, "..", "include", "tq_b200.h"))
    return any(os.path.getmtime(s) > t for s in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, f) for f in CUDA_SOURCES + HOST_SOURCES]
    if force or _stale(LIB, srcs):
        flags = [f for f in NVCC_FLAGS if not f.startswith("--use_fast_math")]
        cmd = [_nvcc(), *flags, "-shared", "-o", LIB, *srcs, "-lcudart"]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
        if verbose:
            print(res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
