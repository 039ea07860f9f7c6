"""The reference project's own device programs -- validation ladders, integration tests and
benchmarks -- built unmodified against libtq_b200.so and the ACL-over-CUDA shim (oracle/_ref/,
see build.py), must pass: they upload the reference fixture, call the launch_* symbols, and
compare every cache byte, every scale bit and every canary page
(tests/npu/turboquant_npu_common.hpp:519-651), every partial record
(tests/npu/turboquant_splitk_rigs.hpp:128-217) or every output word of the fused decoder
(tests/npu/validation/test_turboquant_fused_decode_opt_npu.cpp:264-306, budget 0 ulp) with the
reference's own oracle; the benchmarks validate before they time."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "..", "oracle", "_ref")


def run(name, *argv):
    exe = os.path.join(REF_DIR, name)
    if not os.path.exists(exe):
        pytest.skip(f"{name} not built (needs a checkout of the reference at build time)")
    res = subprocess.run([exe, *argv], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return res.stdout


def test_reference_a8_validation_ladder(cuda):
    out = run("test_turboquant_a8_validation")      # strips 1, 32, 33, 48, 64, 128
    assert "FAIL" not in out


def test_reference_bf16_validation_ladder(cuda):
    out = run("test_turboquant_bf16_validation")
    assert "FAIL" not in out


def test_reference_decode_splitk_aic_validation(cuda):
    out = run("test_turboquant_decode_splitk_aic_validation")
    assert "FAIL" not in out


def test_reference_fused_decode_opt_validation(cuda):
    """launch_fused_decode_opt over the NZ-tiled KV4 cache: every FP16 / BF16 output word equal to
    the correctly rounded FP64 oracle, canary pages, scale padding lanes and the workspace
    outside the live records untouched, the workspace untouched at one split."""
    out = run("test_turboquant_fused_decode_opt_npu")
    assert "PASS fused decode opt NPU validation" in out


@pytest.mark.parametrize("argv", [
    ("--context", "1024,4096", "--iters", "3", "--warmup", "1"),
    ("--context", "2048", "--splitk", "1,4", "--iters", "2", "--warmup", "1", "--pre-rotate", "off",
     "--post-rotate", "rotated"),
])
def test_reference_decode_benchmark_fused_entries(cuda, argv):
    """The reference's decode benchmark drives both fused entries through its rig, which
    validates every launch (tests/npu/turboquant_fused_decode_opt_rig.hpp:181-270). Output
    stages 1 and 2 of the raw-query entry cannot be validated by that rig at all: its
    reference_bits() refuses any expected value outside [1, 15]
    (tests/common/fused_decode_opt_fixture.hpp:47-55), which un-rotated and gated contexts leave;
    those stages are held to Fixture::expected_row in test_gpu_nz_inplace.py instead."""
    out = run("bench_turboquant_decode_splitk", *argv)
    assert "FAIL" not in out


def test_reference_ingest_benchmark(cuda):
    """The reference's own ingest protocol (device-event samples, warm and L2-pressure modes,
    tests/npu/bench/bench_turboquant_reshape_and_cache.cpp:114-143) over all three of its rows."""
    out = run("bench_turboquant_reshape_and_cache", "--warmups", "5", "--samples", "20", "--skip-native")
    assert "FAIL" not in out and "pressure" in out


@pytest.mark.parametrize("mode", ["canary", "zero", "sweep", "sequential"])
def test_reference_integration_scatter(cuda, mode):
    out = run("test_integration_scatter", "--mode", mode)
    assert "PASS" in out


def test_reference_integration_batch(cuda):
    out = run("test_integration_batch")
    assert "PASS turboquant_reshape_and_cache_bf16" in out


def test_reference_integration_scatter_benchmark(cuda):
    run("bench_integration_scatter", "5", "20")
