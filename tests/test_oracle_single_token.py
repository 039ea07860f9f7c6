"""The reference's single-token decode fixture (6 query rows per KV head, head size 256,
tests/common/single_token_decode_oracle.hpp:165-220) and its golden model GoldenDecode
(:256-336), committed as tests/golden/single_token_p2.npz: the CPU oracle must reproduce the
golden state from the same cache bytes. Where the reference is checked out, the committed
vectors are also compared with a fresh run of the reference's own code."""
import os

import numpy as np

from tests import helpers as hp

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "single_token_p2.npz")
PAGES, HEADS, ROWS, D, S, P = 2, 4, 6, 256, 128, 9


def load():
    g = np.load(GOLD)
    return g, g["scale_bits"].view(np.float32)


def test_oracle_partials_match_the_golden_state(oracle):
    g, scales = load()
    for head in range(HEADS):
        q_rot = oracle.rotate_query_bf16(g["q"][head], g["signs"].astype(np.float32), 0.0625)
        # the rotated rows are exact in bf16, and equal the reference's Q_rot
        assert np.array_equal(hp.f32_from_bf16(q_rot), g[f"q_rot_h{head}"])
        m, l, acc = oracle.decode_partial(q_rot, g["key"], g["value"], scales, g["table"], HEADS, head, D, S, P,
                                          PAGES * S, 0, PAGES * S)
        gm, gl, ga = g[f"m_h{head}"], g[f"l_h{head}"], g[f"acc_h{head}"]
        assert np.array_equal(m.astype(np.float32), gm)      # maxima of exact scores are exact
        assert np.allclose(l, gl, rtol=2e-6, atol=0)
        assert (np.abs(acc - ga) <= 2e-6 * np.abs(ga).max(axis=1, keepdims=True) + 1e-7).all()


def test_oracle_decode_matches_the_golden_context(oracle):
    g, scales = load()
    q = g["q"].reshape(1, HEADS * ROWS, D)
    signs = g["signs"].astype(np.float32)
    for stage, name in ((1, "rotated"), (2, "context")):
        got = oracle.decode(q, g["key"], g["value"], scales, g["table"][None, :], np.array([PAGES * S], np.int32),
                            signs, HEADS * ROWS, HEADS, D, S, P, 0.0625, 1.0, stage, g["gate"].reshape(1, -1, D))
        want = np.stack([g[f"{name}_h{h}"] for h in range(HEADS)]).reshape(got.shape)
        # the reference's own budget is relative to the largest magnitude of the row
        assert (np.abs(got - want) <= 1e-5 * np.abs(want).max(axis=-1, keepdims=True)).all()


def test_committed_vectors_are_what_the_reference_computes(reference):
    g, scales = load()
    fx = reference.single_token_fixture(PAGES)
    assert np.array_equal(fx["q"], g["q"]) and np.array_equal(fx["key"], g["key"])
    assert np.array_equal(fx["value"], g["value"]) and np.array_equal(fx["table"], g["table"])
    assert np.array_equal(fx["scales"].view(np.uint32), g["scale_bits"])
    for head in range(HEADS):
        gold = reference.single_token_golden(head, PAGES)
        for k, v in gold.items():
            assert np.array_equal(v, g[f"{k}_h{head}"]), k


def test_fused_descriptor_mirrors_have_the_reference_layout(reference):
    """tq_fused_launch / tq_fused_buffers / tq_fused_raw_query_buffers of include/tq_b200.h
    against the reference's Launch / Buffers / RawQueryBuffers: sizes and every field offset
    (static_asserts in the bridge, which includes both headers)."""
    assert reference.fused_descriptor_layout_matches()
