"""Size-independent properties of the path, checked on the CPU oracle: the same probes the
reference runs on its own models (tests/cpu/test_reshape_and_cache_a8_probe.cpp:150-317,
tests/cpu/test_splitk_decode_probe.cpp:15-72)."""
import numpy as np
import pytest

from tests import helpers as hp


@pytest.mark.parametrize("d", [64, 128, 256])
def test_rotation_is_orthogonal_and_factored_equals_dense(oracle, d):
    rng = np.random.default_rng(d)
    signs = hp.random_signs(rng, d)
    M = np.stack([oracle.rotate_int(signs, np.eye(d, dtype=np.int64)[i], dense=True) for i in range(d)], 1)
    assert np.array_equal(M @ M.T, d * np.eye(d, dtype=np.int64))        # M M^T = d I
    x = rng.integers(-128, 128, d)
    assert np.array_equal(oracle.rotate_int(signs, x), M @ x)             # factored == dense
    # the FP32 cascade is the same matrix; its egress direction is the transpose
    xf = x.astype(np.float32)
    assert np.array_equal(oracle.butterfly_f32(signs, xf, ingress=True), (M @ x).astype(np.float32))
    assert np.array_equal(oracle.butterfly_f32(signs, xf, ingress=False), (M.T @ x).astype(np.float32))


def test_head_size_256_rotation_is_two_head_size_128_rotations_and_a_butterfly(oracle):
    """H_8 = H_2 (x) H_4: with M_h the 128 x 128 rotation over half h of the sign diagonal,
    M = [[M_0, M_1], [M_0, -M_1]] -- the two products and the add / subtract the head-size-256
    tensor-core writer computes."""
    rng = np.random.default_rng(256)
    signs = hp.random_signs(rng, 256)
    dense = lambda s, n: np.stack([oracle.rotate_int(s, np.eye(n, dtype=np.int64)[i], dense=True) for i in range(n)], 1)
    M, M0, M1 = dense(signs, 256), dense(signs[:128], 128), dense(signs[128:], 128)
    assert np.array_equal(M, np.block([[M0, M1], [M0, -M1]]))
    x = rng.integers(-128, 128, 256)
    a, b = M0 @ x[:128], M1 @ x[128:]
    assert np.array_equal(oracle.rotate_int(signs, x), np.concatenate([a + b, a - b]))


def test_resident_blocks_compose_to_the_matrix(oracle):
    """block parity(c1 & g)*G + g, row c0, column i  ==  M[c1*32+c0][g*32+i]."""
    d, G = 128, 4
    signs = oracle.writer_signs(d)
    t = oracle.build_tables_i8(signs).reshape(2 * G, 32, 32)
    M = np.stack([oracle.rotate_int(signs, np.eye(d, dtype=np.int64)[i], dense=True) for i in range(d)], 1)
    for c1 in range(G):
        for g in range(G):
            block = t[(bin(c1 & g).count("1") & 1) * G + g]
            assert np.array_equal(block, M[c1 * 32:(c1 + 1) * 32, g * 32:(g + 1) * 32])
    assert np.array_equal(np.sign(t[:G, :, 0].reshape(-1)), signs)    # column 0 carries the diagonal


def test_partition_owns_every_page_once(oracle):
    for pages in range(1, 130):
        for k in range(1, 17):
            seen = np.zeros(pages, int)
            for s in range(k):
                b, c = oracle.partition(pages, k, s)
                assert c <= (pages + k - 1) // k
                seen[b:b + c] += 1
            assert (seen == 1).all()


@pytest.mark.parametrize("S", [16, 64])
def test_split_merge_equals_full_context(oracle, S):
    """Per-split partials merged by log-sum-exp in shuffled order equal the full-context
    state, including empty splits (the neutral element) and an unaligned tail."""
    rng = np.random.default_rng(S)
    Hkv, d, ctx = 2, 128, 777
    cache = hp.build_cache_from_gaussian(oracle, rng, [ctx], Hkv, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((4, d)).astype(np.float32))
    q_rot = oracle.rotate_query_bf16(q, cache["signs"].astype(np.float32), hp.inv_sqrt_len(d))
    args = (cache["key_cache"], cache["value_cache"], cache["scale_cache"], cache["block_tables"][0],
            Hkv, 1, d, S, cache["num_blocks"], ctx)
    m, l, acc = oracle.decode_partial(q_rot, *args, 0, ctx, 0.1)
    pages = (ctx + S - 1) // S
    for k in (1, 2, 5, 16):
        parts = []
        for s in range(k):
            b, c = oracle.partition(pages, k, s)
            parts.append(oracle.decode_partial(q_rot, *args, b * S, (b + c) * S, 0.1))
        for row in range(4):
            order = rng.permutation(k)
            mm, ll, aa = oracle.lse_merge([(parts[s][0][row], parts[s][1][row], parts[s][2][row]) for s in order])
            assert mm == m[row]
            assert np.isclose(ll, l[row], rtol=1e-12) and np.allclose(aa, acc[row], rtol=1e-10, atol=1e-12)


def test_nibble_layouts_round_trip(oracle):
    """Key pages are token-major, value pages channel-major inside the strip, low nibble first."""
    rng = np.random.default_rng(3)
    H, d = 2, 128
    k, v = hp.int8_activations(rng, 16, H, d)
    signs = oracle.writer_signs(d)
    kc, vc, sc, _, _ = oracle.reshape_and_cache(k, v, np.arange(16, dtype=np.int32), signs, H, d, 16, 1,
                                               hp.inv_sqrt_len(d))
    def unpack(b):
        lo, hi = (b & 15).astype(np.int8), (b >> 4).astype(np.int8)
        q = np.stack([lo, hi], -1).reshape(-1)
        return np.where(q >= 8, q - 16, q)
    for head in range(H):
        kq = unpack(kc.reshape(H, -1)[head]).reshape(16, d)           # [token][channel]
        vq = unpack(vc.reshape(H, -1)[head]).reshape(d, 16).T         # [channel][token] -> [token][channel]
        for t in range(16):
            for plane, q, x in ((0, kq, k), (1, vq, v)):
                y = oracle.rotate_int(signs, x[t, head * d:(head + 1) * d].astype(np.int64))
                scale = sc.reshape(2, 1, H, 16)[plane, 0, head, t]
                e = int(np.floor(np.log2(max(1, np.abs(y).max()))))
                assert scale == np.float32(2.0 ** (e - 2)) * np.float32(hp.inv_sqrt_len(d))
                want = np.minimum(np.rint(y / 2.0 ** (e - 2)), 7)     # numpy rint is half-to-even
                assert np.array_equal(q[t], want)
