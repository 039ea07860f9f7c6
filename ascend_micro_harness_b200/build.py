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

CUDA_SOURCES = ["tq_ingest.cu", "tq_ingest_umma.cu", "tq_ingest_umma256.cu", "tq_scatter.cu", "tq_decode.cu", "tq_routines.cu",
                "tq_lm.cu", "tq_nz.cu"]
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


def build_acl_shim(force: bool = False) -> str:
    """libtq_acl_shim.so: the ACL runtime surface of the reference harnesses over CUDA."""
    src = os.path.join(CSRC, "acl_shim.cpp")
    if force or _stale(ACL_LIB, [src]):
        cmd = [_nvcc(), "-O2", "-std=c++17", "-Xcompiler", "-fPIC", "-shared", "-o", ACL_LIB, src,
               "-lcudart"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    return ACL_LIB


# The reference's own device programs -- validation ladders, integration tests and benchmarks
# -- compiled from where they lie in a checkout of the reference against this library and the
# ACL shim. Outputs go to oracle/_ref/ only; nothing of the reference is copied into this tree.
REFERENCE_HARNESSES = [
    "tests/npu/validation/test_turboquant_a8_validation.cpp",
    "tests/npu/validation/test_turboquant_bf16_validation.cpp",
    "tests/npu/validation/test_turboquant_decode_splitk_aic_validation.cpp",
    "tests/npu/validation/test_turboquant_fused_decode_opt_npu.cpp",
    "tests/npu/bench/bench_turboquant_decode_splitk.cpp",
    "tests/npu/bench/bench_turboquant_reshape_and_cache.cpp",
    "kernels/ops/turboquant/vllm_integration_layer/tests/validation/test_integration_scatter.cpp",
    "kernels/ops/turboquant/vllm_integration_layer/tests/validation/test_integration_batch.cpp",
    "kernels/ops/turboquant/vllm_integration_layer/tests/benchmark/bench_integration_scatter.cpp",
]


def reference_root() -> str | None:
    """A checkout of fxslava/ascend-micro-harness: $TQ_REFERENCE_ROOT, else a directory named
    `reference` beside this repository. None when neither holds the reference's sources."""
    for cand in (os.environ.get("TQ_REFERENCE_ROOT"),
                 os.path.join(PKG, "..", "..", "reference")):
        if cand and os.path.exists(os.path.join(cand, REFERENCE_HARNESSES[0])):
            return os.path.abspath(cand)
    return None


def build_reference_harness(ref_root: str | None = None) -> list[str]:
    ref_root = ref_root or reference_root()
    if ref_root is None:
        return []
    build()
    build_acl_shim()
    out_dir = os.path.join(PKG, "..", "oracle", "_ref")
    os.makedirs(out_dir, exist_ok=True)
    cxx = shutil.which("g++") or "g++"
    built = []
    for rel in REFERENCE_HARNESSES:
        exe = os.path.join(out_dir, os.path.splitext(os.path.basename(rel))[0])
        cmd = [cxx, "-O2", "-std=c++17", f"-I{ref_root}/tests/host_stubs", f"-I{ref_root}",
               os.path.join(ref_root, rel), "-o", exe, f"-L{PKG}", "-ltq_b200", "-ltq_acl_shim",
               "-Wl,-rpath,$ORIGIN/../../ascend_micro_harness_b200", "-pthread"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"building {rel} failed:\n" + res.stdout + res.stderr)
        built.append(exe)
    return built


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    print(build_acl_shim(force="--force" in sys.argv))
    if "--harness" in sys.argv:
        print(build_reference_harness())
