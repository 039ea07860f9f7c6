"""tq_decode_splitk_static: the decode entry point for callers that cannot allocate device
memory when they launch (their process gave all HBM to a cache pool at start-up, or they
may not call their host runtime's allocator from the launch path). Its split-K partials
live in a fixed array inside the library instead of a caller workspace.

Checked here through the C ABI: its output equals that of tq_decode_splitk (same kernels,
same arithmetic, only the workspace differs) on two calls in a row with different inputs --
the second call finds the first call's records in the shared array and must not be disturbed
by them -- and a launch that needs more than the array holds is refused with a clear status.
This file sorts last on purpose, so a run that stops at the first failure has already run
every other test; it also passes when run alone in a fresh process."""
import numpy as np
import pytest

from tests import helpers as hp

pytestmark = pytest.mark.gpu


def _dev(cuda, a):
    import torch
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(cuda).view(torch.bfloat16)
    return torch.from_numpy(a).to(cuda)


def _decode_both(cuda, oracle, seed, ctx, splits, d=128):
    import torch
    import ascend_micro_harness_b200 as tq
    rng = np.random.default_rng(seed)
    Hq, Hkv, S = 16, 4, 16
    cache = hp.build_cache_from_gaussian(oracle, rng, ctx, Hkv, d, S)
    B = len(ctx)
    q = _dev(cuda, hp.bf16_from_f32(rng.standard_normal((B, Hq, d)).astype(np.float32)))
    args = [q] + [_dev(cuda, cache[k]) for k in ("key_cache", "value_cache", "scale_cache",
                                                  "block_tables", "context_lens")]
    args.append(_dev(cuda, cache["signs"].astype(np.float32)))
    kw = dict(num_heads=Hq, num_kv_heads=Hkv, head_size=d, block_size=S,
              num_blocks=cache["num_blocks"], inv_sqrt_len=hp.inv_sqrt_len(d), softmax_scale=0.1,
              splits=splits, max_context_hint=int(max(ctx)), output_stage=tq.OUT_UNROTATED)
    use = splits or tq.choose_splits(B, Hkv, S, int(max(ctx)))
    ws = torch.zeros(tq.decode_workspace_floats(B, Hq, Hkv, d, use), dtype=torch.float32, device=cuda)
    want = torch.zeros((B, Hq, d), dtype=torch.float32, device=cuda)
    got = torch.full((B, Hq, d), float("nan"), dtype=torch.float32, device=cuda)
    tq.decode_splitk(*args, want, workspace=ws, **kw)
    tq.decode_splitk_static(*args, got, **kw)
    torch.cuda.synchronize()
    return got.cpu().numpy(), want.cpu().numpy()


def test_static_workspace_matches_caller_workspace_twice(cuda, oracle):
    # two calls in a row, different batches and split counts: the second reuses the array
    for seed, ctx, splits in ((1, [700, 33, 2048], 4), (2, [1500, 16, 0, 999, 64], 0)):
        got, want = _decode_both(cuda, oracle, seed, ctx, splits)
        assert np.isfinite(got).all()
        # same kernels on the same inputs: identical, and in any case within the decode tolerance
        assert np.array_equal(got, want) or (np.abs(got - want) <= 1e-3 + 2e-3 * np.abs(want)).all()
        assert np.abs(got - want).max() <= 1e-6 * max(1.0, np.abs(want).max())


def test_launch_beyond_the_array_is_refused(cuda):
    import torch
    import ascend_micro_harness_b200 as tq
    B, Hq, Hkv, d = 512, 128, 8, 128          # 512 * 8 * 16 * 16 * 144 floats >> 2 Mi
    z = torch.zeros(16, dtype=torch.bfloat16, device=cuda)
    zi = torch.zeros((B, 4), dtype=torch.int32, device=cuda)
    out = torch.zeros((B, Hq, d), dtype=torch.bfloat16, device=cuda)
    q = torch.zeros((B, Hq, d), dtype=torch.bfloat16, device=cuda)
    with pytest.raises(tq.TqError) as e:
        tq.decode_splitk_static(q, z.view(torch.uint8), z.view(torch.uint8), z.float(), zi,
                                zi[:, 0].contiguous(), z.float(), out, num_heads=Hq, num_kv_heads=Hkv,
                                head_size=d, block_size=16, num_blocks=8, inv_sqrt_len=0.1, splits=16)
    assert e.value.status == 5
    assert "workspace" in str(e.value)


def test_head_size_256_twice(cuda, oracle):
    for seed, ctx, splits in ((3, [900, 40], 0), (4, [65, 1300, 7], 2)):
        got, want = _decode_both(cuda, oracle, seed, ctx, splits, d=256)
        assert np.isfinite(got).all()
        assert np.abs(got - want).max() <= 1e-6 * max(1.0, np.abs(want).max())


def test_the_limit_is_exact(cuda):
    """The largest batch whose records and counters fit the array runs; one sequence more is
    refused, also when the split count is left to the launcher; nonsense geometry is refused as
    nonsense, not as too large."""
    import torch
    import ascend_micro_harness_b200 as tq
    Hq = Hkv = 1
    d, S, splits = 128, 16, 16
    fits = 1
    while tq.decode_workspace_floats(fits + 1, Hq, Hkv, d, splits) <= tq.STATIC_WORKSPACE_FLOATS:
        fits += 1
    assert tq.decode_workspace_floats(fits, Hq, Hkv, d, splits) <= tq.STATIC_WORKSPACE_FLOATS
    assert tq.decode_workspace_floats(fits + 1, Hq, Hkv, d, splits) > tq.STATIC_WORKSPACE_FLOATS

    def call(batch, n_splits, heads=Hq, hint=0):
        P = 4
        kc = torch.zeros(P * Hkv * S * d // 2, dtype=torch.uint8, device=cuda)
        sc = torch.ones(2 * P * Hkv * S, dtype=torch.float32, device=cuda)
        tables = torch.zeros((batch, 2), dtype=torch.int32, device=cuda)
        lens = torch.full((batch,), 20, dtype=torch.int32, device=cuda)
        q = torch.ones((batch, heads, d), dtype=torch.bfloat16, device=cuda)
        out = torch.full((batch, heads, d), float("nan"), dtype=torch.float32, device=cuda)
        tq.decode_splitk_static(q, kc, kc, sc, tables, lens, torch.ones(d, device=cuda), out, num_heads=heads,
                                num_kv_heads=Hkv, head_size=d, block_size=S, num_blocks=P, inv_sqrt_len=0.088,
                                splits=n_splits, max_context_hint=hint)
        torch.cuda.synchronize()
        return out

    assert torch.isfinite(call(fits, splits)).all()
    with pytest.raises(tq.TqError) as e:
        call(fits + 1, splits)
    assert e.value.status == 5
    # splits = 0 with a hint that makes the launcher pick at least as many splits: the same limit applies
    assert tq.choose_splits(fits + 1, Hkv, S, 1 << 20) >= splits
    with pytest.raises(tq.TqError) as e:
        call(fits + 1, 0, hint=1 << 20)
    assert e.value.status == 5
    with pytest.raises(tq.TqError) as e:      # 17 query rows per KV head: invalid, whatever its size
        call(1 << 16, splits, heads=17)
    assert e.value.status == 1
