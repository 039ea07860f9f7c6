"""The CPU oracle (oracle/tq_oracle.cpp) against the committed golden vectors, which were
produced by the reference project's own golden models (tests/golden/make_golden.py), and
-- where oracle/_ref has been built -- against those models directly."""
import os

import numpy as np
import pytest

from tests import helpers as hp

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load(name):
    return np.load(os.path.join(GOLD, name + ".npz"))


@pytest.mark.parametrize("name", ["writer_h4_d256_t48", "writer_h1_d128_t16", "writer_h8_d128_t32"])
@pytest.mark.parametrize("as_bf16", [False, True])
def test_aligned_writer_golden(oracle, name, as_bf16):
    g = load(name)
    T, H, d, S, P = (int(x) for x in g["geometry"])
    key, value = g["key"], g["value"]
    if as_bf16:   # the same integers as bf16 must give byte-identical pages
        key, value = hp.bf16_from_f32(key.astype(np.float32)), hp.bf16_from_f32(value.astype(np.float32))
    assert np.array_equal(oracle.writer_signs(d), g["signs"])
    assert np.array_equal(oracle.build_tables_i8(g["signs"]), g["tables"])
    kc, vc, sc, pw, bad = oracle.reshape_and_cache(key, value, g["slots"], g["signs"], H, d, S, P,
                                                   hp.inv_sqrt_len(d), threads=2)
    assert bad == int(g["bad"][0]) == -1
    assert np.array_equal(kc, g["key_cache"]) and np.array_equal(vc, g["value_cache"])
    assert np.array_equal(sc.view(np.uint32), g["scale_bits"])
    assert np.array_equal(pw, g["page_written"])


def test_scatter_writer_golden(oracle):
    g = load("scatter_h2_d256")
    nreq, H, d, S, P = (int(x) for x in g["geometry"])
    kc, vc, sc = g["prior_key"].copy(), g["prior_value"].copy(), g["prior_scale"].copy()
    assert oracle.reshape_scatter(g["key"], g["value"], g["slots"], g["signs"], g["cu_seqlens"],
                                  nreq, H, d, S, P, hp.inv_sqrt_len(d), kc, vc, sc) == 0
    assert np.array_equal(kc, g["key_cache"]) and np.array_equal(vc, g["value_cache"])
    assert np.array_equal(sc.view(np.uint32), g["scale_bits"])
    assert int(g["zero_rows"][0]) > 0      # the absmax == 0 branch is in the fixture


@pytest.mark.parametrize("name", ["decode_aic_p2", "decode_aic_p2_tail"])
def test_decode_partials_golden(oracle, name):
    g = load(name)
    tokens, seq_len, pages, requests, heads, rows, pt = (int(x) for x in g["dims"])
    signs = g["signs"].astype(np.float32)
    q_rot = g["q_rot"].reshape(heads, rows, 256)
    # the query rotation is bit-exact
    assert np.array_equal(oracle.rotate_query_bf16(g["raw_q"].reshape(-1, 256), signs, 1 / 16.0).reshape(q_rot.shape), q_rot)
    scales = g["scale_bits"].view(np.float32)
    table = g["table"].astype(np.int32)
    for head in range(heads):
        for (b, c) in ((0, 2), (0, 1), (1, 1)):
            m, l, acc = oracle.decode_partial(q_rot[head], g["key"], g["value"], scales, table, heads,
                                              head, 256, pt, pages, seq_len, b * pt, (b + c) * pt)
            assert np.array_equal(m, g[f"m_h{head}_b{b}_c{c}"])
            assert np.allclose(l, g[f"l_h{head}_b{b}_c{c}"], rtol=1e-13, atol=0)
            assert np.allclose(acc, g[f"acc_h{head}_b{b}_c{c}"], rtol=1e-12, atol=1e-300)


def test_decode_full_context_golden(oracle):
    """Un-rotated, gated context of the reference's 6-row fixture (its FP32 `expected`)."""
    g = load("decode_full_p3")
    tokens, seq_len, pages, requests, heads, rows, pt = (int(x) for x in g["dims"])
    signs = g["signs"].astype(np.float32)
    q_rot = g["q_rot"].reshape(heads, rows, 256)
    raw = np.zeros_like(q_rot)
    for idx in np.ndindex(heads, rows):    # q = Pi^T q_rot is exact for this fixture
        raw[idx] = hp.bf16_from_f32(oracle.butterfly_f32(signs, hp.f32_from_bf16(q_rot[idx]),
                                                         ingress=False, scale=1 / 16.0))
    assert np.array_equal(oracle.rotate_query_bf16(raw, signs, 1 / 16.0).reshape(q_rot.shape), q_rot)
    out = oracle.decode(raw.reshape(1, heads * rows, 256), g["key"], g["value"],
                        g["scale_bits"].view(np.float32), g["table"].astype(np.int32)[None, :],
                        np.array([seq_len], np.int32), signs, heads * rows, heads, 256, pt, pages,
                        1 / 16.0, 1.0, 2, g["gate"], threads=2)
    assert np.abs(out.reshape(-1) - g["expected"]).max() < 2e-5


def test_contract_golden(oracle):
    g = load("contract")
    for p, k, s, b, c in g["partition"]:
        assert oracle.partition(int(p), int(k), int(s)) == (int(b), int(c))
    import ascend_micro_harness_b200 as tq
    # 3 requests x 4 KV heads x 8 splits of 16 rows x 272 floats
    assert int(g["workspace_floats"][0]) == 3 * 4 * 8 * 16 * 272
    # the engine's own sizing is the reference's record area plus its arrival counters
    # (one per request, KV head and 8-row tile)
    # and the two 64-bit words of its chunk schedule
    assert tq.decode_workspace_floats(3, 4 * 16, 4, 256, 8) == int(g["workspace_floats"][0]) + 3 * 4 * 2 + 4


# ------------------------------------------------- live against the reference models
@pytest.mark.parametrize("T,H,d", [(16, 4, 256), (528, 4, 256), (16, 1, 128), (128, 8, 128)])
def test_aligned_writer_vs_reference(oracle, reference, T, H, d):
    key, value, slots, P = reference.writer_fixture(T, H, d)
    signs = reference.writer_signs(d)
    want = reference.writer_reference(key, value, slots, H, d, 16, P)
    got = oracle.reshape_and_cache(key, value, slots, signs, H, d, 16, P, hp.inv_sqrt_len(d), threads=4)
    assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])
    assert np.array_equal(got[2].view(np.uint32), want[2].view(np.uint32))
    assert np.array_equal(got[3], want[3]) and got[4] == want[4] == -1


def test_reference_fixture_self_audit(reference):
    """The fixture properties that make a PASS meaningful (all 16 nibbles, the clamp,
    several exponents, distinct pages) hold at the geometries used here."""
    assert reference.writer_fixture_audit_ok(64, 4, 256)
    assert reference.writer_fixture_audit_ok(128, 8, 128)


@pytest.mark.parametrize("n,batch,heads,pt,live,fill", [(128, 1, 1, 128, -1, 1), (384, 2, 2, 128, 300, 2),
                                                      (64, 1, 2, 16, 50, 2), (128, 1, 1, 128, 1, 0)])
def test_decode_partials_vs_reference(oracle, reference, n, batch, heads, pt, live, fill):
    f = reference.decode_fixture(n, batch, heads, 16, pt, live, fill)
    q_rot = f.get("q_rot").reshape(batch, heads, 16, 256)
    signs = reference.decode_signs().astype(np.float32)
    assert np.array_equal(oracle.decode_signs(256), reference.decode_signs())
    assert np.array_equal(oracle.rotate_query_bf16(f.get("raw_q").reshape(-1, 256), signs, 1 / 16.0).reshape(q_rot.shape), q_rot)
    table = f.get("table").astype(np.int32).reshape(batch, f.pages)
    for req in range(batch):
        for head in range(heads):
            for (b, c) in ((0, f.pages), (f.pages - 1, 1)):
                m, l, acc = f.aic_partial(req, head, b, c)
                m2, l2, acc2 = oracle.decode_partial(q_rot[req, head], f.get("key"), f.get("value"),
                                                     f.get("scales"), table[req], heads, head, 256, pt,
                                                     batch * f.pages, f.seq_len, b * pt, (b + c) * pt)
                assert np.array_equal(m, m2)
                assert np.allclose(l, l2, rtol=1e-13) and np.allclose(acc, acc2, rtol=1e-12, atol=1e-300)
