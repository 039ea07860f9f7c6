"""The reference project's own device validation programs, built unmodified against
libtq_b200.so and the ACL-over-CUDA shim (oracle/_ref/, see build.py), must pass: they
upload the reference fixture, call the launch_* symbols, and compare every cache byte,
every scale bit and every canary page (tests/npu/turboquant_npu_common.hpp:519-651) or
every partial record (tests/npu/turboquant_splitk_rigs.hpp:128-217) with the reference's
own oracle."""
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
