"""A KV4/FP8 NZ-tiled cache of the reference's fused decoder on the GPU: the import kernel
bit for bit against the oracle, and import + pre-rotated mid-rise decode against the FP64
oracle that reads the NZ-tiled cache directly and against the reference's own fixture."""
import os

import numpy as np
import pytest

from tests.test_oracle_nz_kv4 import GOLD, nz_random_cache

pytestmark = pytest.mark.gpu

ABS_TOL, REL_TOL = 1e-3, 2e-3


def dev(cuda, a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def gpu_import(cuda, key, value, scales, H, S, P, gain):
    import torch
    import ascend_micro_harness_b200 as tq
    kc = torch.full((P * H * S * 128,), 0x5A, dtype=torch.uint8, device=cuda)
    vc = torch.full_like(kc, 0x5A)
    sc = torch.full((2 * P * H * S,), float("nan"), dtype=torch.float32, device=cuda)
    tq.nz_kv4_import(dev(cuda, key), dev(cuda, value), dev(cuda, scales), kc, vc, sc, num_kv_heads=H,
                     block_size=S, num_blocks=P, gain=gain)
    torch.cuda.synchronize()
    return kc, vc, sc


def gpu_decode(cuda, q_rot, kc, vc, sc, table, lengths, Hq, H, S, P, splits, softmax_scale, code_grid=1,
               out_dtype="f32", pi_signs=None, gate=None, stage=0):
    import torch
    import ascend_micro_harness_b200 as tq
    B = q_rot.shape[0]
    n_splits = splits if splits else tq.choose_splits(B, H, S, int(max(lengths.max(), 1)))
    ws = torch.full((max(1, tq.decode_workspace_floats(B, Hq, H, 256, max(n_splits, 1))),), float("nan"),
                    dtype=torch.float32, device=cuda)
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[out_dtype]
    out = torch.zeros((B, Hq, 256), dtype=tdt, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    tq.decode_splitk_prerotated(dev(cuda, q_rot), kc, vc, sc, dev(cuda, table), dev(cuda, lengths), out,
                                num_heads=Hq, num_kv_heads=H, head_size=256, block_size=S, num_blocks=P,
                                softmax_scale=softmax_scale, splits=splits,
                                max_context_hint=int(lengths.max()), workspace=ws, code_grid=code_grid,
                                pi_signs=None if pi_signs is None else dev(cuda, pi_signs),
                                gate=gate, output_stage=stage, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    return out.float().cpu().numpy()


@pytest.mark.parametrize("H,S,P", [(1, 64, 5), (2, 128, 3), (3, 64, 4), (4, 128, 7)])
def test_import_is_bit_exact(cuda, oracle, H, S, P):
    rng = np.random.default_rng(H * 100 + S)
    key, value, scales = nz_random_cache(rng, P, H, S)
    kc, vc, sc = gpu_import(cuda, key, value, scales, H, S, P, oracle.KV4_GAIN)
    ekc, evc, esc = oracle.nz_kv4_import(key, value, scales, H, S, P)
    assert np.array_equal(kc.cpu().numpy(), ekc)
    assert np.array_equal(vc.cpu().numpy(), evc)
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), esc.view(np.uint32))


@pytest.mark.parametrize("H,G,S,splits", [(1, 16, 64, 1), (2, 4, 128, 4), (4, 3, 64, 0), (3, 1, 128, 2)])
def test_imported_cache_decodes_like_the_nz_oracle(cuda, oracle, H, G, S, splits):
    rng = np.random.default_rng(H * 31 + G)
    ctx = np.array([1, 63, 64, 65, 700, 129, 0, 2048], np.int32)
    B = len(ctx)
    pages = (ctx + S - 1) // S
    P = int(pages.sum()) + 3
    table = np.zeros((B, max(int(pages.max()), 1)), np.int32)
    perm, at = rng.permutation(P), 0
    for b in range(B):
        table[b, :pages[b]] = perm[at:at + pages[b]]
        at += int(pages[b])
    key, value, scales = nz_random_cache(rng, P, H, S)
    Hq = H * G
    q_rot = rng.standard_normal((B, Hq, 256)).astype(np.float32)
    want = oracle.nz_kv4_decode(q_rot, key, value, scales, table, ctx, Hq, H, S, softmax_scale=0.0625)
    kc, vc, sc = gpu_import(cuda, key, value, scales, H, S, P, oracle.KV4_GAIN)
    got = gpu_decode(cuda, q_rot, kc, vc, sc, table, ctx, Hq, H, S, P, splits, 0.0625)
    assert np.isfinite(got).all()
    err = np.abs(got - want)
    assert (err <= ABS_TOL + REL_TOL * np.abs(want)).all(), f"off by {(err / (ABS_TOL + REL_TOL * np.abs(want))).max():.2f}x"


@pytest.mark.parametrize("name", ["fused_kv4_s64", "fused_kv4_s128"])
@pytest.mark.parametrize("out_dtype", ["f32", "f16"])
def test_reference_fixture_through_import_and_decode(cuda, name, out_dtype):
    """The reference's own fixture (FP32 pre-rotated queries, NZ-tiled KV4 cache, ragged
    context, poisoned unmapped pages) against its FP64 expected output."""
    g = np.load(os.path.join(GOLD, name + ".npz"))
    n, b, h, grp, S, pages, physical = [int(v) for v in g["dims"]]
    kc, vc, sc = gpu_import(cuda, g["key"], g["value"], g["scale_bits"].view(np.float32), h, S, physical,
                            float(g["gain"]))
    q = g["query"].reshape(b, h * grp, 256)
    got = gpu_decode(cuda, q, kc, vc, sc, g["table"], g["lengths"], h * grp, h, S, physical, 2, 0.0625,
                     out_dtype=out_dtype)
    want = g["expected"].reshape(got.shape)
    tol = ABS_TOL + REL_TOL * np.abs(want) + (2.0 ** -11 * np.abs(want) if out_dtype == "f16" else 0.0)
    assert (np.abs(got - want) <= tol).all()


def test_prerotated_integer_grid_equals_the_rotating_entry(cuda, oracle):
    """code_grid 0 with the bf16-rounded rotated query reproduces tq_decode_splitk's rotated
    output: same fixed-point query, same cache, same kernel path."""
    import torch
    import ascend_micro_harness_b200 as tq
    from tests import helpers as hp
    rng = np.random.default_rng(77)
    Hq, H, d, S = 8, 2, 256, 64
    cache = hp.build_cache_from_gaussian(oracle, rng, [500, 64, 1], H, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((3, Hq, d)).astype(np.float32))
    signs = torch.from_numpy(cache["signs"].astype(np.float32)).to(cuda)
    qd = torch.from_numpy(q.view(np.int16)).to(cuda).view(torch.bfloat16)
    q_rot = torch.zeros_like(qd)
    tq.rotate_query(qd, signs, q_rot, head_size=d, inv_sqrt_len=hp.inv_sqrt_len(d))
    kc, vc, sc = (dev(cuda, cache[k]) for k in ("key_cache", "value_cache", "scale_cache"))
    tab, ctx = dev(cuda, cache["block_tables"]), dev(cuda, cache["context_lens"])
    P = cache["num_blocks"]
    ws = torch.zeros(tq.decode_workspace_floats(3, Hq, H, d, 2), dtype=torch.float32, device=cuda)
    a = torch.zeros((3, Hq, d), dtype=torch.float32, device=cuda)
    b = torch.zeros_like(a)
    tq.decode_splitk(qd, kc, vc, sc, tab, ctx, signs, a, num_heads=Hq, num_kv_heads=H, head_size=d,
                     block_size=S, num_blocks=P, inv_sqrt_len=hp.inv_sqrt_len(d), softmax_scale=0.0625,
                     splits=2, workspace=ws)
    tq.decode_splitk_prerotated(q_rot.float().contiguous(), kc, vc, sc, tab, ctx, b, num_heads=Hq,
                                num_kv_heads=H, head_size=d, block_size=S, num_blocks=P,
                                softmax_scale=0.0625, splits=2, workspace=ws, code_grid=tq.GRID_INTEGER)
    torch.cuda.synchronize()
    assert torch.equal(a, b)


@pytest.mark.parametrize("d,grid", [(128, 1), (128, 0), (256, 0)])
def test_prerotated_decode_against_a_numpy_reference(cuda, d, grid):
    """Both code grids at both head sizes against an FP64 attention written out in numpy over the
    native planes (key token-major, value channel-major per 16-token strip, planar scales)."""
    import torch
    import ascend_micro_harness_b200 as tq
    rng = np.random.default_rng(d + grid)
    Hq, H, S = 8, 2, 16
    ctx = np.array([37, 300, 16, 1], np.int32)
    B = len(ctx)
    pages = (ctx + S - 1) // S
    P = int(pages.sum()) + 2
    table = np.zeros((B, int(pages.max())), np.int32)
    perm, at = rng.permutation(P), 0
    for b in range(B):
        table[b, :pages[b]] = perm[at:at + pages[b]]
        at += int(pages[b])
    kc = rng.integers(0, 256, P * H * S * d // 2, dtype=np.uint8)
    vc = rng.integers(0, 256, P * H * S * d // 2, dtype=np.uint8)
    sc = rng.uniform(0.05, 0.2, 2 * P * H * S).astype(np.float32)
    q = rng.standard_normal((B, Hq, d)).astype(np.float32)

    def codes(cache, value_plane):
        b = cache.reshape(P, H, -1)
        nib = np.stack([b & 15, b >> 4], -1).reshape(P, H, -1).astype(np.int32)
        nib = np.where(nib > 7, nib - 16, nib)
        if not value_plane:
            return nib.reshape(P, H, S, d)
        return nib.reshape(P, H, S // 16, d, 16).transpose(0, 1, 2, 4, 3).reshape(P, H, S, d)
    K, V = codes(kc, False) + 0.5 * grid, codes(vc, True) + 0.5 * grid
    scp = sc.reshape(2, P, H, S).astype(np.float64)
    want = np.zeros((B, Hq, d))
    for b in range(B):
        for h in range(Hq):
            kv = h // (Hq // H)
            pg, tk = table[b, np.arange(ctx[b]) // S], np.arange(ctx[b]) % S
            logits = (K[pg, kv, tk] @ q[b, h].astype(np.float64)) * scp[0, pg, kv, tk] * 0.3
            p = np.exp(logits - logits.max())
            want[b, h] = (p * scp[1, pg, kv, tk]) @ V[pg, kv, tk] / p.sum()
    dkc, dvc, dsc = (torch.from_numpy(a).to(cuda) for a in (kc, vc, sc))
    ws = torch.zeros(tq.decode_workspace_floats(B, Hq, H, d, 2), dtype=torch.float32, device=cuda)
    out = torch.zeros((B, Hq, d), dtype=torch.float32, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    tq.decode_splitk_prerotated(torch.from_numpy(q).to(cuda), dkc, dvc, dsc, torch.from_numpy(table).to(cuda),
                                torch.from_numpy(ctx).to(cuda), out, num_heads=Hq, num_kv_heads=H, head_size=d,
                                block_size=S, num_blocks=P, softmax_scale=0.3, splits=2, workspace=ws,
                                code_grid=grid, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    got = out.cpu().numpy()
    assert (np.abs(got - want) <= ABS_TOL + REL_TOL * np.abs(want)).all()


@pytest.mark.parametrize("stage", [1, 2])
def test_reference_fixture_unrotated_and_gated(cuda, stage):
    """Output stages 1 and 2 of the fused decoder's raw-query entry on its own fixture: the context
    rotated back by Pi, then gated by the fixture's FP16 gate logits (Fixture::expected_row)."""
    import torch
    g = np.load(os.path.join(GOLD, "fused_kv4_s64.npz"))
    n, b, h, grp, S, pages, physical = [int(v) for v in g["dims"]]
    kc, vc, sc = gpu_import(cuda, g["key"], g["value"], g["scale_bits"].view(np.float32), h, S, physical,
                            float(g["gain"]))
    q = g["query"].reshape(b, h * grp, 256)
    gate = torch.from_numpy(g["gate_f16_bits"].view(np.int16)).to(cuda).view(torch.float16)
    got = gpu_decode(cuda, q, kc, vc, sc, g["table"], g["lengths"], h * grp, h, S, physical, 2, 0.0625,
                     pi_signs=g["pi_signs"], gate=gate if stage == 2 else None, stage=stage)
    want = (g["expected_unrotated"] if stage == 1 else g["expected_gated"]).reshape(got.shape)
    # the rotated rows hold values of 1..15; Pi mixes 256 of them, so the error bound of a row is
    # carried through the rotation: sqrt(256) / 16 = 1 times the per-element bound of the largest
    bound = ABS_TOL + REL_TOL * 15.0
    assert (np.abs(got - want) <= bound).all()


def test_raw_query_rotation_reproduces_the_fixture_query(cuda):
    """Pi(raw query) is the fixture's pre-rotated FP32 query bit for bit (its entries are small
    dyadic numbers, exact in any summation order)."""
    import torch
    import ascend_micro_harness_b200 as tq
    g = np.load(os.path.join(GOLD, "fused_kv4_s64.npz"))
    raw = torch.from_numpy(g["raw_query_f16_bits"].view(np.int16)).to(cuda).view(torch.float16)
    rot = torch.zeros(raw.numel(), dtype=torch.float32, device=cuda)
    tq.rotate_query_pi(raw, dev(cuda, g["pi_signs"]), rot, head_size=256)
    torch.cuda.synchronize()
    assert np.array_equal(rot.cpu().numpy(), g["query"])
