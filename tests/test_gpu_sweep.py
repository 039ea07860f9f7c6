"""Seeded sweeps over geometry on the GPU: odd head counts, every page size, 1..16 query rows
per KV head, explicit and planned split counts, contexts that end anywhere in a strip."""
import numpy as np
import pytest

from tests import helpers as hp
from tests.test_gpu_decode import assert_close, oracle_decode, run_decode
from tests.test_gpu_ingest import assert_identical, expect, run_device

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", range(10))
def test_decode_geometry_sweep(cuda, oracle, seed):
    rng = np.random.default_rng(1000 + seed)
    d = int(rng.choice([128, 256]))
    S = int(rng.choice([16, 32, 64, 128]))
    Hkv = int(rng.choice([1, 2, 3, 5]))
    G = int(rng.choice([1, 2, 3, 4, 6, 8, 12, 16]))
    B = int(rng.integers(1, 5))
    ctx = [int(rng.integers(0, 700)) for _ in range(B)]
    ctx[0] = max(ctx[0], 1)
    cache = hp.build_cache_from_gaussian(oracle, rng, ctx, Hkv, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((B, Hkv * G, d)).astype(np.float32))
    stage = int(rng.choice([0, 1, 2]))
    gate = rng.standard_normal((B, Hkv * G, d)).astype(np.float32) if stage == 2 else None
    scale = float(rng.choice([1.0 / np.sqrt(d), 0.05, 0.2]))
    want = oracle_decode(oracle, q, cache, Hkv * G, Hkv, d, S, stage, gate, scale)
    for splits in (0, int(rng.integers(1, 17))):
        got = run_decode(cuda, q, cache, Hkv * G, Hkv, d, S, splits, stage, gate, scale)
        assert np.isfinite(got).all()
        assert_close(got, want)


@pytest.mark.parametrize("seed", range(8))
def test_writer_geometry_sweep(cuda, oracle, seed):
    rng = np.random.default_rng(2000 + seed)
    d = int(rng.choice([128, 256]))
    S = int(rng.choice([16, 32, 64]))
    H = int(rng.choice([1, 3, 5, 8]))
    strips = int(rng.choice([1, 7, 8, 9, 70, 129]))
    dtype = rng.choice(["int8", "bf16"])
    if dtype == "int8":
        k, v = hp.int8_activations(rng, strips * 16, H, d)
    else:
        k, v = hp.gaussian_outlier_activations(rng, strips * 16, H, d, integer=True)
    per_page = S // 16
    P = (strips + per_page - 1) // per_page + 2
    pages = rng.permutation(P)
    where = rng.permutation(P * per_page)[:strips]
    slots = ((pages[where // per_page] * S + (where % per_page) * 16)[:, None] +
             np.arange(16)[None, :]).astype(np.int32).reshape(-1)
    signs = hp.random_signs(rng, d)
    got = run_device(cuda, k, v, slots, signs, H, d, S, P)
    assert_identical(got, expect(oracle, k, v, slots, signs, H, d, S, P))
