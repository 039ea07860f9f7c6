"""The fused decode step as one unit: the scatter writer puts the new token of every sequence
into the paged cache, then the decode on the same stream must see it. Checked on a ragged batch
of the benchmark's shape (scaled down) against the oracle run over the oracle-written cache,
and by the difference the new token makes: decoding one token less gives another answer."""
import numpy as np
import pytest

from tests import helpers as hp
from tests.test_gpu_decode import assert_close, dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("splits", [0, 3])
def test_scatter_then_decode_sees_the_new_token(cuda, oracle, splits):
    import torch
    import ascend_micro_harness_b200 as tq
    rng = np.random.default_rng(31 + splits)
    Hq, Hkv, d, S = 32, 8, 128, 16
    ctx = rng.integers(512, 6000, size=12).astype(np.int64)
    ctx[0], ctx[1], ctx[2] = 1024, 1039, 527        # new token opens a page / closes a strip / mid-strip
    cache = hp.build_cache_from_gaussian(oracle, rng, list(ctx + 1), Hkv, d, S)   # room for the new token
    P, tables = cache["num_blocks"], cache["block_tables"]
    signs = cache["signs"].astype(np.float32)
    new_k = hp.bf16_from_f32(rng.standard_normal((len(ctx), Hkv * d)).astype(np.float32) * 3.0)
    new_v = hp.bf16_from_f32(rng.standard_normal((len(ctx), Hkv * d)).astype(np.float32) * 3.0)
    slots = np.array([tables[b, ctx[b] // S] * S + ctx[b] % S for b in range(len(ctx))], np.int32)
    q = hp.bf16_from_f32(rng.standard_normal((len(ctx), Hq, d)).astype(np.float32))
    # oracle: scatter into a copy of the cache, decode ctx + 1 tokens
    ekc, evc, esc = cache["key_cache"].copy(), cache["value_cache"].copy(), cache["scale_cache"].copy()
    oracle.reshape_scatter(new_k, new_v, slots, signs, None, len(ctx), Hkv, d, S, P, hp.inv_sqrt_len(d), ekc, evc, esc)
    lens = (ctx + 1).astype(np.int32)
    want = oracle.decode(q, ekc, evc, esc, tables, lens, signs, Hq, Hkv, d, S, P, hp.inv_sqrt_len(d), 0.09, 1, None,
                         threads=8)
    stale = oracle.decode(q, ekc, evc, esc, tables, ctx.astype(np.int32), signs, Hq, Hkv, d, S, P,
                          hp.inv_sqrt_len(d), 0.09, 1, None, threads=8)
    # device: both launches on one stream, no synchronisation in between
    kc, vc, sc = dev(cuda, cache["key_cache"]), dev(cuda, cache["value_cache"]), dev(cuda, cache["scale_cache"])
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    n = splits if splits else tq.choose_splits(len(ctx), Hkv, S, int(lens.max()))
    ws = torch.full((tq.decode_workspace_floats(len(ctx), Hq, Hkv, d, n),), float("nan"), device=cuda)
    out = torch.zeros((len(ctx), Hq, d), dtype=torch.float32, device=cuda)
    dsigns = dev(cuda, signs)
    tq.reshape_scatter(dev(cuda, new_k), dev(cuda, new_v), kc, vc, sc, dev(cuda, slots), dsigns, None,
                       num_requests=len(ctx), num_kv_heads=Hkv, head_size=d, block_size=S, num_blocks=P,
                       inv_sqrt_len=hp.inv_sqrt_len(d), status=st)
    tq.decode_splitk(dev(cuda, q), kc, vc, sc, dev(cuda, tables), dev(cuda, lens), dsigns, out, num_heads=Hq,
                     num_kv_heads=Hkv, head_size=d, block_size=S, num_blocks=P, inv_sqrt_len=hp.inv_sqrt_len(d),
                     softmax_scale=0.09, splits=splits, max_context_hint=int(lens.max()), workspace=ws,
                     output_stage=tq.OUT_UNROTATED, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert np.array_equal(kc.cpu().numpy(), ekc) and np.array_equal(vc.cpu().numpy(), evc)
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), esc.view(np.uint32))
    got = out.cpu().numpy()
    assert_close(got, want)
    # the new token matters: the answer without it lies outside the tolerance somewhere in every sequence
    miss = np.abs(stale - want) > 2 * (1e-3 + 2e-3 * np.abs(want))
    assert miss.reshape(len(ctx), -1).any(axis=1).all()


@pytest.mark.parametrize("splits", [0, 1, 5])
def test_decode_step_as_one_call(cuda, oracle, splits):
    """tq_decode_step: the same step as one call of the library, the decode scheduled under the writer.
    Two steps back to back on one stream (the second appends a second token): cache bytes and both
    outputs must match the oracle, so no CTA of a decode read a page before its writer was done."""
    import torch
    import ascend_micro_harness_b200 as tq
    rng = np.random.default_rng(77 + splits)
    Hq, Hkv, d, S = 32, 8, 128, 16
    B = 10
    ctx = rng.integers(300, 5000, size=B).astype(np.int64)
    ctx[0], ctx[1] = 1023, 2047                      # the first new token closes a strip, the second opens a page
    cache = hp.build_cache_from_gaussian(oracle, rng, list(ctx + 2), Hkv, d, S)
    P, tables = cache["num_blocks"], cache["block_tables"]
    signs = cache["signs"].astype(np.float32)
    ekc, evc, esc = cache["key_cache"].copy(), cache["value_cache"].copy(), cache["scale_cache"].copy()
    kc, vc, sc = dev(cuda, ekc), dev(cuda, evc), dev(cuda, esc)
    dsigns, dtab = dev(cuda, signs), dev(cuda, tables)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    n = splits if splits else tq.choose_splits(B, Hkv, S, int(ctx.max()) + 2)
    ws = torch.full((tq.decode_workspace_floats(B, Hq, Hkv, d, n),), float("nan"), device=cuda)
    steps = []
    for t in range(2):
        at = ctx + t
        new_k = hp.bf16_from_f32(rng.standard_normal((B, Hkv * d)).astype(np.float32) * 3.0)
        new_v = hp.bf16_from_f32(rng.standard_normal((B, Hkv * d)).astype(np.float32) * 3.0)
        slots = np.array([tables[b, at[b] // S] * S + at[b] % S for b in range(B)], np.int32)
        q = hp.bf16_from_f32(rng.standard_normal((B, Hq, d)).astype(np.float32))
        lens = (at + 1).astype(np.int32)
        oracle.reshape_scatter(new_k, new_v, slots, signs, None, B, Hkv, d, S, P, hp.inv_sqrt_len(d), ekc, evc, esc)
        want = oracle.decode(q, ekc, evc, esc, tables, lens, signs, Hq, Hkv, d, S, P, hp.inv_sqrt_len(d), 0.09, 1,
                             None, threads=8)
        out = torch.zeros((B, Hq, d), dtype=torch.float32, device=cuda)
        steps.append((dev(cuda, new_k), dev(cuda, new_v), dev(cuda, slots), dev(cuda, q), dev(cuda, lens), out, want))
    for nk, nv, sl, q, lens, out, _ in steps:          # no synchronisation between the two steps
        tq.decode_step(nk, nv, sl, q, kc, vc, sc, dtab, lens, dsigns, out, num_heads=Hq, num_kv_heads=Hkv,
                       head_size=d, block_size=S, num_blocks=P, inv_sqrt_len=hp.inv_sqrt_len(d), softmax_scale=0.09,
                       splits=splits, max_context_hint=int(ctx.max()) + 2, workspace=ws,
                       output_stage=tq.OUT_UNROTATED, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    assert np.array_equal(kc.cpu().numpy(), ekc) and np.array_equal(vc.cpu().numpy(), evc)
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), esc.view(np.uint32))
    for *_, out, want in steps:
        assert_close(out.cpu().numpy(), want)


def test_decode_step_refuses_before_it_writes(cuda):
    """A step whose decode would be refused (17 query rows per KV head) leaves the cache untouched."""
    import torch
    import ascend_micro_harness_b200 as tq
    B, Hkv, d, S, P = 2, 1, 128, 16, 8
    kc = torch.full((P * Hkv * S * d // 2,), 0xAA, dtype=torch.uint8, device=cuda)
    vc = torch.full_like(kc, 0xAA)
    sc = torch.ones(2 * P * Hkv * S, dtype=torch.float32, device=cuda)
    nk = torch.ones((B, Hkv * d), dtype=torch.bfloat16, device=cuda)
    q = torch.ones((B, 17, d), dtype=torch.bfloat16, device=cuda)
    out = torch.zeros((B, 17, d), dtype=torch.float32, device=cuda)
    tab = torch.zeros((B, 2), dtype=torch.int32, device=cuda)
    lens = torch.full((B,), 5, dtype=torch.int32, device=cuda)
    slots = torch.tensor([4, 20], dtype=torch.int32, device=cuda)
    ws = torch.zeros(1 << 16, device=cuda)
    with pytest.raises(tq.TqError) as e:
        tq.decode_step(nk, nk, slots, q, kc, vc, sc, tab, lens, torch.ones(d, device=cuda), out, num_heads=17,
                       num_kv_heads=Hkv, head_size=d, block_size=S, num_blocks=P, inv_sqrt_len=0.088, splits=1,
                       workspace=ws)
    assert e.value.status == 1
    torch.cuda.synchronize()
    assert (kc == 0xAA).all() and (vc == 0xAA).all()
