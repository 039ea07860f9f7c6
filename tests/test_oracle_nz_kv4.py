"""The KV4/FP8 NZ-tiled cache of the reference's fused decoder on the CPU: the oracle's
addressing, import and FP64 decode pinned to the reference's own fixture
(tests/common/fused_decode_opt_fixture.hpp) -- live where the reference checkout is present,
through committed vectors generated from it otherwise."""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def nz_random_cache(rng, P, H, S):
    """A random NZ-tiled pool: arbitrary code bytes, positive non-power-of-two scales, NaN in
    the padding lanes of every scale record."""
    key = rng.integers(0, 256, P * S * H * 128, dtype=np.uint8)
    value = rng.integers(0, 256, P * S * H * 128, dtype=np.uint8)
    slot_floats = (2 * H + 7) // 8 * 8
    scales = np.full((P * S, slot_floats), np.nan, np.float32)
    scales[:, :2 * H] = rng.uniform(0.3, 0.9, (P * S, 2 * H)).astype(np.float32)
    return key, value, scales.reshape(-1)


@pytest.mark.parametrize("name", ["fused_kv4_s64", "fused_kv4_s128"])
def test_decode_oracle_reproduces_the_reference_fixture(oracle, name):
    g = np.load(os.path.join(GOLD, name + ".npz"))
    n, b, h, grp, S, pages, physical = [int(v) for v in g["dims"]]
    out = oracle.nz_kv4_decode(g["query"], g["key"], g["value"], g["scale_bits"].view(np.float32),
                               g["table"], g["lengths"], h * grp, h, S, gain=float(g["gain"]))
    want = g["expected"].reshape(out.shape)
    assert np.abs(out - want).max() <= 2e-6 * np.abs(want).max()
    for slot, head, col, H, at in g["nz_bytes"]:
        assert oracle.nz_tiled_packed_byte(int(slot), int(head), int(col), int(H)) == int(at)


@pytest.mark.parametrize("geom", [(64, 1, 1, 16, 128), (1000, 2, 4, 3, 128), (129, 3, 3, 1, 64),
                                  (63, 1, 2, 2, 64), (4096, 1, 1, 4, 128)])
def test_decode_oracle_against_the_live_reference_fixture(oracle, reference, geom):
    n, b, h, grp, S = geom
    fx = reference.fused_fixture(n, b, h, grp, S)
    table = fx.get("table")[:b * fx.pages].reshape(b, fx.pages)
    out = oracle.nz_kv4_decode(fx.get("query"), fx.get("key"), fx.get("value"), fx.get("scales"), table,
                               fx.get("lengths")[:b], h * grp, h, S, gain=reference.kv4_gain())
    want = fx.get("expected").reshape(out.shape)
    assert np.abs(out - want).max() <= 2e-6 * np.abs(want).max()
    rng = np.random.default_rng(n)
    for _ in range(200):
        H = int(rng.integers(1, 5))
        slot, head, col = int(rng.integers(0, 128)), int(rng.integers(0, H)), int(rng.integers(0, 128))
        assert oracle.nz_tiled_packed_byte(slot, head, col, H) == reference.nz_tiled_packed_byte(slot, head, col, H)


def native_codes(cache, P, H, S, value_plane):
    """[P][H][S][256] two's-complement codes out of a native-layout plane."""
    b = cache.reshape(P, H, -1)
    nib = np.stack([b & 15, b >> 4], -1).reshape(P, H, -1).astype(np.int32)
    nib = np.where(nib > 7, nib - 16, nib)
    if not value_plane:
        return nib.reshape(P, H, S, 256)
    return nib.reshape(P, H, S // 16, 256, 16).transpose(0, 1, 2, 4, 3).reshape(P, H, S, 256)


@pytest.mark.parametrize("H,S", [(1, 64), (2, 128), (3, 64), (4, 128)])
def test_import_moves_every_code_and_scale(oracle, H, S):
    rng = np.random.default_rng(H * 1000 + S)
    P = 3
    key, value, scales = nz_random_cache(rng, P, H, S)
    kc, vc, sc = oracle.nz_kv4_import(key, value, scales, H, S, P)
    got_k, got_v = native_codes(kc, P, H, S, False), native_codes(vc, P, H, S, True)
    slot_floats = (2 * H + 7) // 8 * 8
    gain = np.float32(oracle.KV4_GAIN)
    for _ in range(400):
        p, row, head, ch = (int(rng.integers(0, P)), int(rng.integers(0, S)), int(rng.integers(0, H)),
                            int(rng.integers(0, 256)))
        at = p * S * H * 128 + oracle.nz_tiled_packed_byte(row, head, ch % 128, H)
        for plane, src, got in ((0, key, got_k), (1, value, got_v)):
            nib = int(src[at]) >> (4 if ch >= 128 else 0) & 15
            assert got[p, head, row, ch] == (nib - 16 if nib > 7 else nib)
            want = scales[(p * S + row) * slot_floats + plane * H + head] / gain
            assert sc[((plane * P + p) * H + head) * S + row] == want


def test_pi_of_the_fused_decoder(oracle):
    """Pi = diag(s) H diag(s) / 16 is an involution and turns the fixture's rotated-basis rows into
    its un-rotated rows (golden vectors from RawQueryBasis::apply / Fixture::expected_row)."""
    g = np.load(os.path.join(GOLD, "fused_kv4_s64.npz"))
    s = g["pi_signs"]
    rows = g["expected"].reshape(-1, 256)
    un = oracle.signed_hadamard(rows, s)
    assert np.array_equal(un, g["expected_unrotated"])
    back = oracle.signed_hadamard(un, s)
    assert np.abs(back - rows).max() <= 1e-5 * np.abs(rows).max()


def test_pi_against_the_live_reference(oracle, reference):
    rng = np.random.default_rng(12)
    s = reference.fused_signs()
    for _ in range(5):
        x = rng.standard_normal(256).astype(np.float32)
        assert np.array_equal(oracle.signed_hadamard(x[None], s)[0], reference.fused_pi_apply(x))


def test_lloydmax_lut_table_is_the_reference_header_s(oracle, reference):
    """The 16 levels of the fused decoder's Lloyd-Max toggle, bit for bit as
    TurboQuantLloydMaxTraits<KV4_FP8> holds them; its thresholds are the midpoints and its gain is 1."""
    levels, thresholds, gain = reference.kv4_lloydmax_lut()
    ours = oracle.kv4_lloydmax_lut()
    assert np.array_equal(levels.view(np.uint32), ours.view(np.uint32))
    assert np.array_equal(thresholds, ((ours[1:].astype(np.float64) + ours[:-1]) / 2).astype(np.float32))
    assert gain == 1.0
    assert np.array_equal(ours, -ours[::-1]) and (np.diff(ours) > 0).all()


def test_levels_oracle_with_the_uniform_grid_is_the_mid_rise_oracle(oracle):
    """Levels (b - 7.5) at gain 1 must give exactly what the mid-rise decode gives: the two differ only in
    how a nibble becomes a value."""
    rng = np.random.default_rng(5)
    H, S, Hq = 2, 64, 4
    ctx = np.array([130, 9], np.int32)
    P = 5
    table = np.array([[4, 1, 0], [2, 0, 0]], np.int32)
    key, value, scales = nz_random_cache(rng, P, H, S)
    q = rng.standard_normal((2, Hq, 256)).astype(np.float32)
    a = oracle.nz_kv4_decode(q, key, value, scales, table, ctx, Hq, H, S, softmax_scale=0.07, gain=1.0)
    b = oracle.nz_kv4_decode_lut(q, key, value, scales, table, ctx, Hq, H, S, softmax_scale=0.07,
                                 levels=np.arange(16, dtype=np.float32) - 7.5)
    assert np.array_equal(a, b)
