"""The fused decoder's KV4/FP8 cache written on its e4m3-rounded Lloyd-Max codebook (the
`kLloydMaxLut` toggle): same NZ-tiled storage, a stored nibble is the signed form of a bin
index, the bin's level times the scale is the value, gain 1. Read here through the import
(gain 1) and tq_decode_splitk_levels, against the FP64 oracle that reads the NZ bytes
directly; the table itself is pinned to the reference's header on the CPU side
(tests/test_oracle_nz_kv4.py)."""
import numpy as np
import pytest

from tests.test_gpu_nz_kv4 import ABS_TOL, REL_TOL, dev, gpu_import
from tests.test_gpu_nz_inplace import random_case

pytestmark = pytest.mark.gpu


def decode_levels(cuda, q_rot, levels, kc, vc, sc, table, lengths, Hq, H, S, P, splits, scale, pi_signs=None,
                  gate=None, stage=0, out_dtype="f32"):
    import torch
    import ascend_micro_harness_b200 as tq
    B = q_rot.shape[0]
    ws = torch.full((tq.decode_workspace_floats(B, Hq, H, 256, 16),), float("nan"), device=cuda)
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[out_dtype]
    out = torch.zeros((B, Hq, 256), dtype=tdt, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    tq.decode_splitk_levels(dev(cuda, q_rot), levels, kc, vc, sc, dev(cuda, table), dev(cuda, lengths), out,
                            num_heads=Hq, num_kv_heads=H, head_size=256, block_size=S, num_blocks=P,
                            softmax_scale=scale, splits=splits, max_context_hint=int(lengths.max()), workspace=ws,
                            pi_signs=None if pi_signs is None else dev(cuda, pi_signs), gate=gate,
                            output_stage=stage, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    return out


@pytest.mark.parametrize("H,G,S,splits", [(1, 8, 64, 1), (2, 4, 128, 4), (4, 3, 64, 0), (3, 1, 128, 16)])
def test_levels_decode_matches_the_oracle(cuda, oracle, H, G, S, splits):
    rng = np.random.default_rng(900 + H * 7 + G)
    ctx = np.array([1, 63, 64, 65, 700, 129, 0, 2048], np.int32)
    P, table, key, value, scales = random_case(rng, H, S, ctx)
    Hq = H * G
    q_rot = rng.standard_normal((len(ctx), Hq, 256)).astype(np.float32)
    levels = oracle.kv4_lloydmax_lut()
    want = oracle.nz_kv4_decode_lut(q_rot, key, value, scales, table, ctx, Hq, H, S, softmax_scale=0.0625)
    kc, vc, sc = gpu_import(cuda, key, value, scales, H, S, P, 1.0)
    got = decode_levels(cuda, q_rot, levels, kc, vc, sc, table, ctx, Hq, H, S, P, splits, 0.0625).cpu().numpy()
    assert np.isfinite(got).all()
    bad = np.abs(got - want) > ABS_TOL + REL_TOL * np.abs(want)
    assert not bad.any(), f"{bad.sum()} of {bad.size} beyond tolerance, worst {np.abs(got - want).max()}"
    assert np.all(got[ctx == 0] == 0.0)


def test_uniform_levels_reproduce_the_mid_rise_grid(cuda, oracle):
    """With levels (b - 7.5) the table decode is the uniform mid-rise grid: same answer as the oracle of the
    ordinary KV4 cache at gain 1 (the reference's kGatherLut leg: same instructions, the grid as the table)."""
    rng = np.random.default_rng(41)
    H, G, S = 2, 4, 64
    ctx = np.array([300, 17, 1025], np.int32)
    P, table, key, value, scales = random_case(rng, H, S, ctx)
    q_rot = rng.standard_normal((len(ctx), H * G, 256)).astype(np.float32)
    want = oracle.nz_kv4_decode(q_rot, key, value, scales, table, ctx, H * G, H, S, softmax_scale=0.0625, gain=1.0)
    kc, vc, sc = gpu_import(cuda, key, value, scales, H, S, P, 1.0)
    got = decode_levels(cuda, q_rot, np.arange(16) - 7.5, kc, vc, sc, table, ctx, H * G, H, S, P, 2,
                        0.0625).cpu().numpy()
    assert (np.abs(got - want) <= ABS_TOL + REL_TOL * np.abs(want)).all()


def test_levels_decode_output_stages(cuda, oracle):
    """Stage 1 applies Pi = diag(s) H diag(s) / 16 to the context, stage 2 also the gate, as the pre-rotated entry."""
    import torch
    rng = np.random.default_rng(43)
    H, G, S = 2, 2, 128
    ctx = np.array([513, 40], np.int32)
    P, table, key, value, scales = random_case(rng, H, S, ctx)
    Hq = H * G
    q_rot = rng.standard_normal((len(ctx), Hq, 256)).astype(np.float32)
    signs = np.where(rng.random(256) < 0.5, -1.0, 1.0).astype(np.float32)
    gate = rng.standard_normal((len(ctx), Hq, 256)).astype(np.float32)
    base = oracle.nz_kv4_decode_lut(q_rot, key, value, scales, table, ctx, Hq, H, S, softmax_scale=0.0625)
    unrot = oracle.signed_hadamard(base.reshape(-1, 256), signs).reshape(base.shape)
    kc, vc, sc = gpu_import(cuda, key, value, scales, H, S, P, 1.0)
    levels = oracle.kv4_lloydmax_lut()
    got1 = decode_levels(cuda, q_rot, levels, kc, vc, sc, table, ctx, Hq, H, S, P, 3, 0.0625, pi_signs=signs,
                         stage=1).cpu().numpy()
    got2 = decode_levels(cuda, q_rot, levels, kc, vc, sc, table, ctx, Hq, H, S, P, 3, 0.0625, pi_signs=signs,
                         gate=torch.from_numpy(gate).to(cuda), stage=2).cpu().numpy()
    assert (np.abs(got1 - unrot) <= ABS_TOL + REL_TOL * np.abs(unrot)).all()
    gated = unrot / (1.0 + np.exp(-gate.astype(np.float64)))
    assert (np.abs(got2 - gated) <= ABS_TOL + REL_TOL * np.abs(gated)).all()


def test_levels_decode_refusals(cuda):
    import torch
    import ascend_micro_harness_b200 as tq
    z8 = torch.zeros(64 * 128, dtype=torch.uint8, device=cuda)
    sc = torch.ones(2 * 64, dtype=torch.float32, device=cuda)
    q = torch.zeros((1, 9, 256), dtype=torch.float32, device=cuda)
    out = torch.zeros((1, 9, 256), dtype=torch.float32, device=cuda)
    tab = torch.zeros((1, 1), dtype=torch.int32, device=cuda)
    lens = torch.ones(1, dtype=torch.int32, device=cuda)
    ws = torch.zeros(tq.decode_workspace_floats(1, 9, 1, 256, 16), device=cuda)
    with pytest.raises(tq.TqError) as e:      # nine query heads on one KV head: beyond the table kernel's eight rows
        tq.decode_splitk_levels(q, np.zeros(16), z8, z8, sc, tab, lens, out, num_heads=9, num_kv_heads=1,
                                head_size=256, block_size=64, num_blocks=1, splits=1, workspace=ws)
    assert e.value.status == 1
