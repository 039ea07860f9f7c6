"""The persistent decode grid (tq_decode_splitk_persistent: the batch's tiles cut into chunks
that one resident wave of CTAs takes, first statically and then off an atomic ticket; the last
CTA to finish a head merges its records and writes the output) against the FP64 oracle and
against the classic grid, on batches chosen for what can break it: heads that straddle several
chunks, heads that fit inside one, empty and one-token sequences, two row tiles per KV head,
counter and ticket words that start as garbage, and the split plan of the classic grid with
several query tokens per request."""
import numpy as np
import pytest

from tests import helpers as hp
from tests.test_gpu_decode import assert_close, dev, oracle_decode

pytestmark = pytest.mark.gpu


def launch(cuda, q, cache, Hq, Hkv, d, S, ws, stage=0, gate=None, scale=0.1, out_dtype=None, splits=0, hint=None,
           persistent=True):
    import torch
    import ascend_micro_harness_b200 as tq
    out = torch.full((q.shape[0], Hq, d), 7.0, dtype=out_dtype or torch.float32, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    tq.decode_splitk(dev(cuda, q), dev(cuda, cache["key_cache"]), dev(cuda, cache["value_cache"]),
                     dev(cuda, cache["scale_cache"]), dev(cuda, cache["block_tables"]),
                     dev(cuda, cache["context_lens"]), dev(cuda, cache["signs"].astype(np.float32)), out,
                     num_heads=Hq, num_kv_heads=Hkv, head_size=d, block_size=S, num_blocks=cache["num_blocks"],
                     inv_sqrt_len=hp.inv_sqrt_len(d), softmax_scale=scale, splits=splits,
                     max_context_hint=int(cache["context_lens"].max()) if hint is None else hint, workspace=ws,
                     gate=None if gate is None else dev(cuda, gate), output_stage=stage, status=st,
                     persistent=persistent)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    return out.float().cpu().numpy()


def workspace(cuda, B, Hq, Hkv, d, S, max_ctx, fill, n=None):
    """A workspace for `n` record slots per head (default: all 32), every word set to `fill`."""
    import torch
    import ascend_micro_harness_b200 as tq
    n = n or tq.MAX_SPLITS
    ws = torch.empty(tq.decode_workspace_floats(B, Hq, Hkv, d, n), dtype=torch.float32, device=cuda)
    ws.view(torch.int32).fill_(fill)
    return ws, n


@pytest.mark.parametrize("d,Hq,Hkv,S", [(128, 32, 8, 16), (256, 16, 4, 16), (128, 8, 2, 64), (256, 32, 2, 128)])
def test_ragged_batch_against_the_oracle(cuda, oracle, d, Hq, Hkv, S):
    rng = np.random.default_rng(d + S)
    ctx = [int(c) for c in rng.integers(1, 5000, size=20)] + [0, 1, 16, 17, 4097, 9000]
    cache = hp.build_cache_from_gaussian(oracle, rng, ctx, Hkv, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((len(ctx), Hq, d)).astype(np.float32))
    want = oracle_decode(oracle, q, cache, Hq, Hkv, d, S, softmax_scale=0.1)
    # counters that start as 0xFFFFFFFF, as zeros, and as whatever the previous launch left
    ws, n = workspace(cuda, len(ctx), Hq, Hkv, d, S, max(ctx), -1)
    first = launch(cuda, q, cache, Hq, Hkv, d, S, ws)
    again = launch(cuda, q, cache, Hq, Hkv, d, S, ws)
    ws0, _ = workspace(cuda, len(ctx), Hq, Hkv, d, S, max(ctx), 0)
    zeroed = launch(cuda, q, cache, Hq, Hkv, d, S, ws0)
    assert np.isfinite(first).all()
    assert_close(first, want)
    # the shares and the order in which records merge are fixed by the batch, so a relaunch
    # reproduces every bit whichever CTA happens to arrive last
    assert np.array_equal(first, again) and np.array_equal(first, zeroed)
    assert (first[20] == 0).all()       # the empty sequence
    # the classic grid (a split count fixed by the caller) agrees within the tolerance
    import torch
    import ascend_micro_harness_b200 as tq
    wsc = torch.full((tq.decode_workspace_floats(len(ctx), Hq, Hkv, d, 3),), float("nan"), device=cuda)
    assert_close(launch(cuda, q, cache, Hq, Hkv, d, S, wsc, splits=3, persistent=False), want)
    # few record slots: the chunks stay wide enough that no head needs more than the workspace holds
    ws4, _ = workspace(cuda, len(ctx), Hq, Hkv, d, S, max(ctx), -1, n=4)
    assert_close(launch(cuda, q, cache, Hq, Hkv, d, S, ws4, splits=4), want)


def test_counter_words_that_look_like_counts_of_another_launch(cuda, oracle):
    """Counter words holding small numbers (a plausible stale count under a foreign tag) must
    not be taken for arrivals of this launch."""
    import torch
    rng = np.random.default_rng(5)
    Hq, Hkv, d, S = 16, 4, 128, 16
    ctx = [3000, 2500, 40, 7000]
    cache = hp.build_cache_from_gaussian(oracle, rng, ctx, Hkv, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((len(ctx), Hq, d)).astype(np.float32))
    want = oracle_decode(oracle, q, cache, Hq, Hkv, d, S, softmax_scale=0.1)
    for fill in (1, 2, 0x00000101, 0x7FC0BEEF):
        ws, _ = workspace(cuda, len(ctx), Hq, Hkv, d, S, max(ctx), fill)
        assert_close(launch(cuda, q, cache, Hq, Hkv, d, S, ws), want)


@pytest.mark.parametrize("stage,out", [(1, "f32"), (2, "bf16"), (2, "f16")])
def test_output_stages_and_narrow_outputs(cuda, oracle, stage, out):
    import torch
    rng = np.random.default_rng(stage * 7 + len(out))
    Hq, Hkv, d, S = 16, 4, 128, 16
    ctx = [2222, 5, 800, 3100]
    cache = hp.build_cache_from_gaussian(oracle, rng, ctx, Hkv, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((len(ctx), Hq, d)).astype(np.float32))
    gate = rng.standard_normal((len(ctx), Hq, d)).astype(np.float32)
    want = oracle_decode(oracle, q, cache, Hq, Hkv, d, S, stage, gate, 0.09)
    ws, _ = workspace(cuda, len(ctx), Hq, Hkv, d, S, max(ctx), -1)
    f32 = launch(cuda, q, cache, Hq, Hkv, d, S, ws, stage, gate, 0.09)
    assert_close(f32, want)
    if out != "f32":
        tdt = torch.bfloat16 if out == "bf16" else torch.float16
        narrow = launch(cuda, q, cache, Hq, Hkv, d, S, ws, stage, gate, 0.09, out_dtype=tdt)
        assert np.array_equal(narrow, torch.from_numpy(f32).to(tdt).float().numpy())


@pytest.mark.parametrize("d", [128, 256])
def test_sixteen_rows_per_kv_head_use_two_row_tiles(cuda, oracle, d):
    rng = np.random.default_rng(d)
    Hkv, G, S = 2, 16, 16
    ctx = [1500, 2600, 333]
    cache = hp.build_cache_from_gaussian(oracle, rng, ctx, Hkv, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((len(ctx), Hkv * G, d)).astype(np.float32))
    want = oracle_decode(oracle, q, cache, Hkv * G, Hkv, d, S, 1, None, 0.1)
    ws, _ = workspace(cuda, len(ctx), Hkv * G, Hkv, d, S, max(ctx), -1)
    assert_close(launch(cuda, q, cache, Hkv * G, Hkv, d, S, ws, stage=1), want)


def test_several_query_tokens_per_request(cuda, oracle):
    """tokens_per_req = 3 with the split plan left to the library: query token t sees the context
    without its last 2 - t tokens (the oracle is the ordinary decode run once per query token)."""
    import torch
    import ascend_micro_harness_b200 as tq
    rng = np.random.default_rng(77)
    Hq, Hkv, d, S, T = 8, 2, 128, 16, 3
    ctx = [2000, 950, 4100]
    cache = hp.build_cache_from_gaussian(oracle, rng, ctx, Hkv, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((len(ctx) * T, Hq, d)).astype(np.float32))
    want = np.zeros((len(ctx) * T, Hq, d))
    for t in range(T):
        c2 = dict(cache)
        c2["context_lens"] = (cache["context_lens"] - (T - 1 - t)).astype(np.int32)
        want[t::T] = oracle_decode(oracle, q[t::T], c2, Hq, Hkv, d, S, softmax_scale=0.1)
    n = tq.choose_splits(len(ctx), Hkv, S, max(ctx))
    ws = torch.full((tq.decode_workspace_floats(len(ctx), Hq * T, Hkv, d, n),), float("nan"), device=cuda)
    out = torch.zeros((len(ctx) * T, Hq, d), dtype=torch.float32, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    tq.decode_splitk_mtp(dev(cuda, q), dev(cuda, cache["key_cache"]), dev(cuda, cache["value_cache"]),
                         dev(cuda, cache["scale_cache"]), dev(cuda, cache["block_tables"]),
                         dev(cuda, cache["context_lens"]), dev(cuda, cache["signs"].astype(np.float32)), out,
                         tokens_per_req=T, num_heads=Hq, num_kv_heads=Hkv, head_size=d, block_size=S,
                         num_blocks=cache["num_blocks"], inv_sqrt_len=hp.inv_sqrt_len(d), softmax_scale=0.1,
                         splits=0, max_context_hint=max(ctx), workspace=ws, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert_close(out.cpu().numpy(), want)


def test_one_split_writes_the_output_without_a_workspace(cuda, oracle):
    """splits = 1: every CTA holds a head's whole state and finishes it itself. No workspace
    is passed at all, and a poisoned one that is passed comes back untouched."""
    import torch
    import ascend_micro_harness_b200 as tq
    rng = np.random.default_rng(9)
    Hq, Hkv, d, S = 8, 2, 128, 16
    ctx = [700, 0, 33]
    cache = hp.build_cache_from_gaussian(oracle, rng, ctx, Hkv, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((len(ctx), Hq, d)).astype(np.float32))
    want = oracle_decode(oracle, q, cache, Hq, Hkv, d, S, 1, None, 0.1)
    got = launch(cuda, q, cache, Hq, Hkv, d, S, None, stage=1, splits=1, persistent=False)
    assert_close(got, want)
    assert (got[1] == 0).all()
    ws = torch.full((tq.decode_workspace_floats(len(ctx), Hq, Hkv, d, 1),), float("nan"), device=cuda)
    assert np.array_equal(launch(cuda, q, cache, Hq, Hkv, d, S, ws, stage=1, splits=1, persistent=False), got)
    assert torch.isnan(ws).all()


def test_precise_entry_scales_with_the_values(cuda, oracle):
    """The wider arithmetic: values 64 times larger move the output 64 times, the error bound
    does not grow with them (held to 1e-5 of the largest value magnitude here)."""
    import torch
    import ascend_micro_harness_b200 as tq
    rng = np.random.default_rng(4)
    Hq, Hkv, d, S = 8, 2, 128, 16
    ctx = [1200, 300]
    cache = hp.build_cache_from_gaussian(oracle, rng, ctx, Hkv, d, S)
    P = cache["num_blocks"]
    cache["scale_cache"][P * Hkv * S:] *= 64.0     # the value plane
    q = hp.bf16_from_f32(rng.standard_normal((len(ctx), Hq, d)).astype(np.float32))
    want = oracle_decode(oracle, q, cache, Hq, Hkv, d, S, softmax_scale=0.1)
    ws = torch.full((tq.decode_workspace_floats(len(ctx), Hq, Hkv, d, 4),), float("nan"), device=cuda)
    out = torch.zeros((len(ctx), Hq, d), dtype=torch.float32, device=cuda)
    tq.decode_splitk(dev(cuda, q), dev(cuda, cache["key_cache"]), dev(cuda, cache["value_cache"]),
                     dev(cuda, cache["scale_cache"]), dev(cuda, cache["block_tables"]),
                     dev(cuda, cache["context_lens"]), dev(cuda, cache["signs"].astype(np.float32)), out,
                     num_heads=Hq, num_kv_heads=Hkv, head_size=d, block_size=S, num_blocks=P,
                     inv_sqrt_len=hp.inv_sqrt_len(d), softmax_scale=0.1, splits=4, workspace=ws, precise=True)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert (np.abs(got - want) <= 1e-5 * np.abs(want).max()).all()
