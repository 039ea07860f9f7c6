"""Decode over the fused decoder's NZ-tiled KV4 pools where they lie (tq_decode_splitk_nz): no
import, no second pool. Held to three things: the partial records and outputs of import +
pre-rotated decode, bit for bit; the FP64 oracle that reads the NZ bytes directly; and the
reference's own fixture with its FP64 expected output, where the wider arithmetic must give the
correctly rounded 16-bit word of every channel (the budget of the reference's device ladder,
tests/npu/validation/test_turboquant_fused_decode_opt_npu.cpp:139)."""
import os

import numpy as np
import pytest

from tests.test_gpu_nz_kv4 import ABS_TOL, REL_TOL, dev, gpu_decode, gpu_import
from tests.test_oracle_nz_kv4 import GOLD, nz_random_cache

pytestmark = pytest.mark.gpu


def decode_in_place(cuda, q_rot, key, value, scales, table, lengths, Hq, H, S, splits, softmax_scale, ws=None,
                    out_dtype="f32", pi_signs=None, gate=None, stage=0, precise=False, P=0):
    import torch
    import ascend_micro_harness_b200 as tq
    B = q_rot.shape[0]
    n = splits if splits else tq.choose_splits(B, H, S, int(max(lengths.max(), 1)))
    if ws is None:
        ws = torch.full((max(1, tq.decode_workspace_floats(B, Hq, H, 256, n)),), float("nan"),
                        dtype=torch.float32, device=cuda)
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[out_dtype]
    out = torch.zeros((B, Hq, 256), dtype=tdt, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    tq.decode_splitk_nz(dev(cuda, q_rot), dev(cuda, key), dev(cuda, value), dev(cuda, scales), dev(cuda, table),
                        dev(cuda, lengths), out, num_heads=Hq, num_kv_heads=H, block_size=S, num_blocks=P,
                        softmax_scale=softmax_scale, splits=splits, max_context_hint=int(lengths.max()),
                        workspace=ws, pi_signs=None if pi_signs is None else dev(cuda, pi_signs), gate=gate,
                        output_stage=stage, precise=precise, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    return out, ws


def random_case(rng, H, S, ctx):
    B = len(ctx)
    pages = (ctx + S - 1) // S
    P = int(pages.sum()) + 3
    table = np.zeros((B, max(int(pages.max()), 1)), np.int32)
    perm, at = rng.permutation(P), 0
    for b in range(B):
        table[b, :pages[b]] = perm[at:at + pages[b]]
        at += int(pages[b])
    key, value, scales = nz_random_cache(rng, P, H, S)
    return P, table, key, value, scales


@pytest.mark.parametrize("H,G,S,splits", [(1, 16, 64, 1), (2, 4, 128, 4), (4, 3, 64, 2), (3, 1, 128, 7)])
def test_in_place_equals_import_then_decode_bit_for_bit(cuda, H, G, S, splits):
    import torch
    import ascend_micro_harness_b200 as tq
    from oracle.bindings import Oracle
    rng = np.random.default_rng(H * 31 + G)
    ctx = np.array([1, 63, 64, 65, 700, 129, 0, 2048], np.int32)
    P, table, key, value, scales = random_case(rng, H, S, ctx)
    Hq = H * G
    q_rot = rng.standard_normal((len(ctx), Hq, 256)).astype(np.float32)
    got, ws = decode_in_place(cuda, q_rot, key, value, scales, table, ctx, Hq, H, S, splits, 0.0625, P=P)
    kc, vc, sc = gpu_import(cuda, key, value, scales, H, S, P, Oracle.KV4_GAIN)
    ws2 = torch.full_like(ws, float("nan"))
    out2 = torch.zeros_like(got)
    tq.decode_splitk_prerotated(dev(cuda, q_rot), kc, vc, sc, dev(cuda, table), dev(cuda, ctx), out2, num_heads=Hq,
                                num_kv_heads=H, head_size=256, block_size=S, num_blocks=P, softmax_scale=0.0625,
                                splits=splits, max_context_hint=int(ctx.max()), workspace=ws2,
                                code_grid=tq.GRID_MIDRISE)
    torch.cuda.synchronize()
    assert torch.equal(got, out2)
    if splits > 1:      # the per-split partial records themselves (one split leaves the workspace alone)
        records = len(ctx) * H * splits * G * 272
        assert torch.equal(ws[:records], ws2[:records])
    else:
        assert torch.isnan(ws).all() and torch.isnan(ws2).all()


@pytest.mark.parametrize("H,G,S,splits", [(2, 4, 128, 0), (4, 16, 64, 0), (1, 8, 64, 3)])
def test_in_place_against_the_nz_oracle(cuda, oracle, H, G, S, splits):
    rng = np.random.default_rng(H * 7 + G + S)
    ctx = np.concatenate([rng.integers(1, 3000, size=10), [0, 64, 65, 5000]]).astype(np.int32)
    P, table, key, value, scales = random_case(rng, H, S, ctx)
    Hq = H * G
    q_rot = rng.standard_normal((len(ctx), Hq, 256)).astype(np.float32)
    want = oracle.nz_kv4_decode(q_rot, key, value, scales, table, ctx, Hq, H, S, softmax_scale=0.0625)
    got, _ = decode_in_place(cuda, q_rot, key, value, scales, table, ctx, Hq, H, S, splits, 0.0625)
    got = got.cpu().numpy()
    assert np.isfinite(got).all()
    err = np.abs(got - want)
    assert (err <= ABS_TOL + REL_TOL * np.abs(want)).all(), f"off by {(err / (ABS_TOL + REL_TOL * np.abs(want))).max():.2f}x"
    # the wider arithmetic on the same inputs: 1e-5 of the largest context magnitude
    fine, _ = decode_in_place(cuda, q_rot, key, value, scales, table, ctx, Hq, H, S, splits if splits else 4, 0.0625,
                              precise=True)
    assert (np.abs(fine.cpu().numpy() - want) <= 1e-5 * np.abs(want).max()).all()


def half_bits_rne(x32):
    """Correctly rounded FP16 words of FP32 values (numpy's conversion is round-to-nearest-even)."""
    return x32.astype(np.float16).view(np.uint16)


@pytest.mark.parametrize("name", ["fused_kv4_s64", "fused_kv4_s128"])
@pytest.mark.parametrize("splits", [1, 2, 5])
def test_reference_fixture_in_place_is_correctly_rounded(cuda, name, splits):
    """The reference's own fixture: FP16 output of the wider arithmetic equals the correctly
    rounded FP16 word of the FP64 expected value in every channel (0 ULP), and the native path
    stays inside the stated tolerance."""
    g = np.load(os.path.join(GOLD, name + ".npz"))
    n, b, h, grp, S, pages, physical = [int(v) for v in g["dims"]]
    q = g["query"].reshape(b, h * grp, 256)
    scales = g["scale_bits"].view(np.float32)
    got, _ = decode_in_place(cuda, q, g["key"], g["value"], scales, g["table"], g["lengths"], h * grp, h, S, splits,
                             0.0625, out_dtype="f16", precise=True)
    want = g["expected"].reshape(b, h * grp, 256)
    assert np.array_equal(got.cpu().numpy().view(np.uint16), half_bits_rne(want))
    fast, _ = decode_in_place(cuda, q, g["key"], g["value"], scales, g["table"], g["lengths"], h * grp, h, S, splits,
                              0.0625)
    assert (np.abs(fast.cpu().numpy() - want) <= ABS_TOL + REL_TOL * np.abs(want)).all()


@pytest.mark.parametrize("stage", [1, 2])
def test_reference_fixture_raw_query_stages_in_place(cuda, stage):
    """Raw query -> Pi -> in-place decode -> output stage 1 / 2, against Fixture::expected_row."""
    import torch
    import ascend_micro_harness_b200 as tq
    g = np.load(os.path.join(GOLD, "fused_kv4_s64.npz"))
    n, b, h, grp, S, pages, physical = [int(v) for v in g["dims"]]
    raw = torch.from_numpy(g["raw_query_f16_bits"].view(np.int16)).to(cuda).view(torch.float16)
    rot = torch.zeros(raw.numel(), dtype=torch.float32, device=cuda)
    tq.rotate_query_pi(raw, dev(cuda, g["pi_signs"]), rot, head_size=256)
    gate = torch.from_numpy(g["gate_f16_bits"].view(np.int16)).to(cuda).view(torch.float16)
    got, _ = decode_in_place(cuda, rot.cpu().numpy().reshape(b, h * grp, 256), g["key"], g["value"],
                             g["scale_bits"].view(np.float32), g["table"], g["lengths"], h * grp, h, S, 2, 0.0625,
                             pi_signs=g["pi_signs"], gate=gate if stage == 2 else None, stage=stage, precise=True)
    want = (g["expected_unrotated"] if stage == 1 else g["expected_gated"]).reshape(b, h * grp, 256)
    # the reference rig's budget for the restaged outputs is 8 FP16 ulps of a 256-term rotation
    assert (np.abs(got.cpu().numpy() - want) <= 8 * 2.0 ** -11 * np.maximum(np.abs(want), 1.0)).all()
