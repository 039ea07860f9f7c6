"""The routine oracles (Hadamard 16x16 tile, Lloyd-Max codec, ICDF int4 quantiser) and the
Lloyd-Max cache variant on the CPU: pinned to the reference's own golden models where the
reference checkout is present, and to committed vectors generated from them otherwise."""
import os

import numpy as np
import pytest

from oracle.bindings import Oracle, Reference, bf16_from_f32

GOLD = os.path.join(os.path.dirname(__file__), "golden", "routines.npz")


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD)


def test_lloydmax_codebook_and_codes_match_golden(oracle, gold):
    c, t = oracle.lloydmax4_tables()
    assert np.array_equal(c, gold["lm_centroids"]) and np.array_equal(t, gold["lm_thresholds"])
    packed, recon = oracle.lloydmax4_quantize(gold["lm_x"])
    assert np.array_equal(packed, gold["lm_packed"])
    codes = np.stack([packed & 15, packed >> 4], axis=1).reshape(-1)
    assert np.array_equal(recon, c[codes])


def test_lloydmax_threshold_ties_go_up(oracle):
    _, t = oracle.lloydmax4_tables()
    x = np.concatenate([t, np.nextafter(t, -np.inf, dtype=np.float32), np.float32([-0.0, 100, -100])])
    x = np.concatenate([x, np.zeros((-x.size) % 2, np.float32)])
    packed, _ = oracle.lloydmax4_quantize(x)
    codes = np.stack([packed & 15, packed >> 4], axis=1).reshape(-1)
    assert list(codes[:15]) == list(range(1, 16))        # x == t_i counts t_i
    assert list(codes[15:30]) == list(range(0, 15))      # just below it does not
    assert codes[30] == 8 and codes[31] == 15 and codes[32] == 0


def test_hadamard16_matches_golden_and_is_involutive(oracle, gold):
    y = oracle.hadamard16(gold["h16_x"])
    assert np.array_equal(y, gold["h16_y"])
    back = oracle.hadamard16(y.astype(np.float16).view(np.uint16))   # exact: dyadic, small
    x = gold["h16_x"].view(np.float16).astype(np.float32).reshape(-1, 16, 16)
    assert np.array_equal(back, 16 * x)


@pytest.mark.parametrize("bf16", [False, True])
def test_icdf_matches_golden(oracle, gold, bf16):
    tag = "bf16" if bf16 else "f16"
    assert np.array_equal(oracle.icdf_quantize(gold[f"icdf_{tag}_bits"], bf16), gold[f"icdf_{tag}_packed"])


@pytest.mark.skipif(not Reference.available(), reason="reference bridge not built")
def test_routines_against_the_reference_models(oracle):
    r = Reference()
    x = r.lloydmax_fixture(256, 16, True)
    assert np.array_equal(oracle.lloydmax4_quantize(x)[0], r.lloydmax4_pack(x))
    rng = np.random.default_rng(3)
    tiles = (rng.integers(-96, 97, size=(8, 16, 16)) / 16).astype(np.float16)
    y = oracle.hadamard16(tiles.view(np.uint16))
    for i in range(8):
        assert np.array_equal(y[i], r.hadamard16(tiles[i].view(np.uint16)))
    for bf in (False, True):
        bits, want = r.icdf_fixture(bf, 4)
        assert np.array_equal(oracle.icdf_quantize(bits, bf), want)


def test_lloydmax_cache_variant_round_trip(oracle):
    """Writer -> dequantise: the reconstruction error is the Lloyd-Max distortion (about
    0.0095 of the variance for 16 levels), the page layout is the strip layout, decode of a
    one-token context returns that token's dequantised value row."""
    rng = np.random.default_rng(1)
    H, d, S, T = 2, 128, 16, 32
    x = rng.standard_normal((2, T, H * d)).astype(np.float32)
    k, v = bf16_from_f32(x[0]), bf16_from_f32(x[1])
    slots = np.arange(T, dtype=np.int32)
    inv = float(np.float32(1) / np.sqrt(np.float32(d)))
    kc, vc, sc, bad = oracle.reshape_and_cache_lm(k, v, slots, H, d, S, 2, inv)
    assert bad == 0
    c, _ = oracle.lloydmax4_tables()
    # dequantise the key plane: token-major rows
    codes = np.stack([kc & 15, kc >> 4], axis=1).reshape(2, H, S, d)      # [page][head][tok][ch]
    scales = sc[: 2 * H * S].reshape(2, H, S)
    y_hat = c[codes]  * scales[..., None]                     # rotated, un-normalised / 4
    h16 = np.array([[(-1) ** bin(a & b).count("1") for b in range(16)] for a in range(16)], np.float32)
    xk = x[0].reshape(2, S, H, d).transpose(0, 2, 1, 3)                    # [page][head][tok][ch]
    xk = bf16_round(xk)
    y = (xk.reshape(2, H, S, d // 16, 16) @ h16).reshape(2, H, S, d) / 4
    rel = np.mean((y - y_hat) ** 2) / np.mean(y ** 2)
    assert 0.006 < rel < 0.014
    # value plane holds the same tokens channel-major inside the strip
    vcodes = np.stack([vc & 15, vc >> 4], axis=1).reshape(2, H, d, S)     # [page][head][ch][tok]
    xv = bf16_round(x[1].reshape(2, S, H, d).transpose(0, 2, 1, 3))
    yv = (xv.reshape(2, H, S, d // 16, 16) @ h16).reshape(2, H, S, d) / 4
    vs = sc[2 * H * S:].reshape(2, H, S)
    yv_hat = c[vcodes].transpose(0, 1, 3, 2) * vs[..., None]
    assert np.mean((yv - yv_hat) ** 2) / np.mean(yv ** 2) < 0.014


def bf16_round(a):
    from oracle.bindings import f32_from_bf16
    return f32_from_bf16(bf16_from_f32(np.ascontiguousarray(a, np.float32))).reshape(a.shape)


def test_lloydmax_decode_of_uniform_context(oracle):
    """A context whose tokens are all the same vector attends to that vector: the output,
    rotated back, is the dequantised value row."""
    rng = np.random.default_rng(2)
    H, d, S, T = 1, 128, 16, 48
    row = rng.standard_normal((1, H * d)).astype(np.float32)
    k = bf16_from_f32(np.repeat(row, T, 0))
    v = bf16_from_f32(np.repeat(rng.standard_normal((1, H * d)).astype(np.float32), T, 0))
    inv = float(np.float32(1) / np.sqrt(np.float32(d)))
    kc, vc, sc, _ = oracle.reshape_and_cache_lm(k, v, np.arange(T, dtype=np.int32), H, d, S, 3, inv)
    q = bf16_from_f32(rng.standard_normal((1, 4, d)).astype(np.float32))
    tables = np.array([[0, 1, 2]], np.int32)
    out = oracle.decode_lm(q, kc, vc, sc, tables, np.array([T], np.int32), 4, H, d, S, 3, 0.1, 1)
    c, _ = oracle.lloydmax4_tables()
    vcodes = np.stack([vc & 15, vc >> 4], axis=1).reshape(3, H, d, S)[0, 0, :, 0]
    y_hat = c[vcodes] * sc[3 * H * S]                                     # rotated basis
    h16 = np.array([[(-1) ** bin(a & b).count("1") for b in range(16)] for a in range(16)], np.float32)
    want = (y_hat.reshape(d // 16, 16) @ h16).reshape(d) / 4
    assert np.allclose(out[0], want[None, :], atol=2e-6, rtol=1e-5)
