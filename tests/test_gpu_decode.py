"""Paged split-K decode on the GPU through the C ABI vs the FP64 CPU oracle."""
import numpy as np
import pytest

from tests import helpers as hp

pytestmark = pytest.mark.gpu

ABS_TOL, REL_TOL = 1e-3, 2e-3   # the stated tolerance of the decode output against the FP64 reference


def dev(cuda, a):
    import torch
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(cuda).view(torch.bfloat16)
    if a.dtype == np.uint32:
        return torch.from_numpy(a.view(np.int32)).to(cuda)
    return torch.from_numpy(a).to(cuda)


def run_decode(cuda, q, cache, Hq, Hkv, d, S, splits, stage=0, gate=None, softmax_scale=1.0,
               out_dtype="f32"):
    import torch
    import ascend_micro_harness_b200 as tq
    B = q.shape[0]
    use_splits = splits if splits else tq.choose_splits(B, Hkv, S, int(cache["context_lens"].max()))
    ws = torch.full((max(1, tq.decode_workspace_floats(B, Hq, Hkv, d, max(use_splits, 1))),),
                    float("nan"), dtype=torch.float32, device=cuda)
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[out_dtype]
    out = torch.zeros((B, Hq, d), dtype=tdt, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    tq.decode_splitk(dev(cuda, q), dev(cuda, cache["key_cache"]), dev(cuda, cache["value_cache"]),
                     dev(cuda, cache["scale_cache"]), dev(cuda, cache["block_tables"]),
                     dev(cuda, cache["context_lens"]), dev(cuda, cache["signs"].astype(np.float32)),
                     out, num_heads=Hq, num_kv_heads=Hkv, head_size=d, block_size=S,
                     num_blocks=cache["num_blocks"], inv_sqrt_len=hp.inv_sqrt_len(d),
                     softmax_scale=softmax_scale, splits=splits,
                     max_context_hint=int(cache["context_lens"].max()), workspace=ws,
                     gate=None if gate is None else dev(cuda, gate), output_stage=stage, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    return out.float().cpu().numpy()


def oracle_decode(oracle, q, cache, Hq, Hkv, d, S, stage=0, gate=None, softmax_scale=1.0):
    return oracle.decode(q, cache["key_cache"], cache["value_cache"], cache["scale_cache"],
                         cache["block_tables"], cache["context_lens"],
                         cache["signs"].astype(np.float32), Hq, Hkv, d, S, cache["num_blocks"],
                         hp.inv_sqrt_len(d), softmax_scale, stage, gate, threads=8)


def assert_close(got, want):
    err = np.abs(got - want)
    bound = ABS_TOL + REL_TOL * np.abs(want)
    worst = (err / bound).max()
    assert worst <= 1.0, f"decode output off by {worst:.2f}x the tolerance"


@pytest.mark.parametrize("splits", [1, 2, 4, 8, 16, 0])
def test_config3_batch1_ctx4096(cuda, oracle, splits):
    """The single-sequence benchmark configuration: batch 1, 32 q / 8 KV heads, d=128, ctx 4096, shuffled table."""
    rng = np.random.default_rng(33)
    Hq, Hkv, d, S = 32, 8, 128, 16
    cache = hp.build_cache_from_gaussian(oracle, rng, [4096], Hkv, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((1, Hq, d)).astype(np.float32))
    scale = 1.0 / np.sqrt(d)
    want = oracle_decode(oracle, q, cache, Hq, Hkv, d, S, softmax_scale=scale)
    got = run_decode(cuda, q, cache, Hq, Hkv, d, S, splits, softmax_scale=scale)
    assert_close(got, want)


@pytest.mark.parametrize("S", [16, 64, 128])
@pytest.mark.parametrize("d", [128, 256])
def test_ragged_batch_with_tails(cuda, oracle, S, d):
    """Ragged contexts including lengths that end inside a strip; the dead slots of the
    last page hold NaN scales and 0xAA codes, which must not reach the output."""
    rng = np.random.default_rng(S * 1000 + d)
    Hq, Hkv = 8, 2
    ctx = [1, 15, 16, 17, 79, 257, 1023, 300, 0, 513]
    cache = hp.build_cache_from_gaussian(oracle, rng, ctx, Hkv, d, S)
    # poison everything past each sequence's live length inside its last page
    for b, c in enumerate(ctx):
        if c % S:
            page = cache["block_tables"][b, c // S]
            for h in range(Hkv):
                for kv in range(2):
                    base = ((kv * cache["num_blocks"] + page) * Hkv + h) * S
                    cache["scale_cache"][base + c % S: base + S] = np.nan
    q = hp.bf16_from_f32(rng.standard_normal((len(ctx), Hq, d)).astype(np.float32))
    for splits in (1, 3, 0):
        want = oracle_decode(oracle, q, cache, Hq, Hkv, d, S, softmax_scale=0.1)
        got = run_decode(cuda, q, cache, Hq, Hkv, d, S, splits, softmax_scale=0.1)
        assert np.isfinite(got).all()
        assert_close(got, want)
        assert (got[8] == 0).all()      # the empty sequence


def test_narrow_outputs_are_the_rounded_fp32_output(cuda, oracle):
    """bf16 / f16 outputs are the FP32 result narrowed once, round-to-nearest-even."""
    import torch
    rng = np.random.default_rng(12)
    Hq, Hkv, d, S = 8, 2, 128, 16
    cache = hp.build_cache_from_gaussian(oracle, rng, [333, 64], Hkv, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((2, Hq, d)).astype(np.float32))
    f32 = run_decode(cuda, q, cache, Hq, Hkv, d, S, 2, softmax_scale=0.1)
    bf = run_decode(cuda, q, cache, Hq, Hkv, d, S, 2, softmax_scale=0.1, out_dtype="bf16")
    fh = run_decode(cuda, q, cache, Hq, Hkv, d, S, 2, softmax_scale=0.1, out_dtype="f16")
    t = torch.from_numpy(f32)
    assert np.array_equal(bf, t.to(torch.bfloat16).float().numpy())
    assert np.array_equal(fh, t.to(torch.float16).float().numpy())


@pytest.mark.parametrize("stage", [1, 2])
def test_output_stages(cuda, oracle, stage):
    rng = np.random.default_rng(stage)
    Hq, Hkv, d, S = 16, 4, 128, 16
    cache = hp.build_cache_from_gaussian(oracle, rng, [200, 777], Hkv, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((2, Hq, d)).astype(np.float32))
    gate = rng.standard_normal((2, Hq, d)).astype(np.float32)
    want = oracle_decode(oracle, q, cache, Hq, Hkv, d, S, stage, gate, 0.09)
    got = run_decode(cuda, q, cache, Hq, Hkv, d, S, 2, stage, gate, 0.09)
    assert_close(got, want)


@pytest.mark.parametrize("elem", ["bf16", "f16"])
@pytest.mark.parametrize("stage", [0, 2])
def test_element_typed_entry(cuda, oracle, elem, stage):
    """Query, gate and output in one 16-bit type (the fused decoder's raw-query form). The
    output is the FP32 result narrowed once, so it is held to the tolerance plus half an ulp
    of the element type."""
    import torch
    import ascend_micro_harness_b200 as tq
    rng = np.random.default_rng(41 + stage)
    Hq, Hkv, d, S = 16, 4, 128, 16
    cache = hp.build_cache_from_gaussian(oracle, rng, [333, 1500, 64], Hkv, d, S)
    tdt = torch.bfloat16 if elem == "bf16" else torch.float16
    qt = torch.from_numpy(rng.standard_normal((3, Hq, d)).astype(np.float32)).to(tdt)
    gt = torch.from_numpy(rng.standard_normal((3, Hq, d)).astype(np.float32)).to(tdt)
    q_bits = qt.view(torch.int16).numpy().view(np.uint16)
    want = oracle.decode(q_bits, cache["key_cache"], cache["value_cache"], cache["scale_cache"],
                         cache["block_tables"], cache["context_lens"], cache["signs"].astype(np.float32),
                         Hq, Hkv, d, S, cache["num_blocks"], hp.inv_sqrt_len(d), 0.09, stage,
                         gt.float().numpy() if stage == 2 else None, threads=8, q_f16=(elem == "f16"))
    splits = 3
    ws = torch.full((tq.decode_workspace_floats(3, Hq, Hkv, d, splits),), float("nan"), device=cuda)
    out = torch.zeros((3, Hq, d), dtype=tdt, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    tq.decode_splitk_elem(qt.to(cuda), dev(cuda, cache["key_cache"]), dev(cuda, cache["value_cache"]),
                          dev(cuda, cache["scale_cache"]), dev(cuda, cache["block_tables"]),
                          dev(cuda, cache["context_lens"]), dev(cuda, cache["signs"].astype(np.float32)), out,
                          num_heads=Hq, num_kv_heads=Hkv, head_size=d, block_size=S,
                          num_blocks=cache["num_blocks"], inv_sqrt_len=hp.inv_sqrt_len(d), softmax_scale=0.09,
                          splits=splits, workspace=ws, gate=gt.to(cuda) if stage == 2 else None,
                          output_stage=stage, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    got = out.float().cpu().numpy()
    half_ulp = (2.0 ** -9 if elem == "bf16" else 2.0 ** -12) * np.abs(want)
    err = np.abs(got - want)
    assert (err <= ABS_TOL + REL_TOL * np.abs(want) + half_ulp).all()


@pytest.mark.parametrize("tpr,G,d", [(2, 6, 128), (3, 4, 128), (4, 4, 256), (2, 8, 256), (2, 1, 128)])
def test_several_query_tokens_per_request(cuda, oracle, tpr, G, d):
    """Speculative rows: token t of a request attends to the context without its last
    tpr - 1 - t tokens; all tpr * G rows of a KV head share one pass over the pages. The
    oracle is the ordinary decode run once per query token with that token's length."""
    import torch
    import ascend_micro_harness_b200 as tq
    rng = np.random.default_rng(tpr * 100 + G)
    Hkv, S = 2, 16
    Hq = Hkv * G
    ctx = [tpr, 16, 17 + tpr, 333, 1]          # includes a context shorter than the token count
    B = len(ctx)
    cache = hp.build_cache_from_gaussian(oracle, rng, ctx, Hkv, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((B, tpr, Hq, d)).astype(np.float32))
    gate = rng.standard_normal((B, tpr, Hq, d)).astype(np.float32)
    scale = float(1 / np.sqrt(d))
    want = np.zeros((B, tpr, Hq, d))
    for t in range(tpr):
        lens = np.maximum(np.array(ctx) - (tpr - 1 - t), 0).astype(np.int32)
        c2 = dict(cache, context_lens=lens)
        want[:, t] = oracle_decode(oracle, np.ascontiguousarray(q[:, t]), c2, Hq, Hkv, d, S, 2,
                                   np.ascontiguousarray(gate[:, t]), scale)
    for splits in (1, 3, 0):
        use = splits if splits else tq.choose_splits(B, Hkv, S, max(ctx))
        ws = torch.full((tq.decode_workspace_floats(B, Hq * tpr, Hkv, d, use),), float("nan"), device=cuda)
        out = torch.zeros((B * tpr, Hq, d), dtype=torch.float32, device=cuda)
        st = torch.zeros(1, dtype=torch.int32, device=cuda)
        tq.decode_splitk_mtp(dev(cuda, q.reshape(B * tpr, Hq, d)), dev(cuda, cache["key_cache"]),
                             dev(cuda, cache["value_cache"]), dev(cuda, cache["scale_cache"]),
                             dev(cuda, cache["block_tables"]), dev(cuda, cache["context_lens"]),
                             dev(cuda, cache["signs"].astype(np.float32)), out, tokens_per_req=tpr,
                             num_heads=Hq, num_kv_heads=Hkv, head_size=d, block_size=S,
                             num_blocks=cache["num_blocks"], inv_sqrt_len=hp.inv_sqrt_len(d),
                             softmax_scale=scale, splits=splits, max_context_hint=max(ctx), workspace=ws,
                             gate=dev(cuda, gate.reshape(B * tpr, Hq, d)), output_stage=2, status=st)
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        got = out.cpu().numpy().reshape(B, tpr, Hq, d)
        assert np.isfinite(got).all()
        assert_close(got, want)


def test_peaked_softmax_without_scale(cuda, oracle):
    """No softmax scale (the AIC decoder's convention): scores of std ~ sqrt(d)."""
    rng = np.random.default_rng(9)
    Hq, Hkv, d, S = 8, 2, 128, 16
    cache = hp.build_cache_from_gaussian(oracle, rng, [2048], Hkv, d, S, outliers=True)
    q = hp.bf16_from_f32(rng.standard_normal((1, Hq, d)).astype(np.float32))
    want = oracle_decode(oracle, q, cache, Hq, Hkv, d, S)
    got = run_decode(cuda, q, cache, Hq, Hkv, d, S, 4)
    assert_close(got, want)


def test_value_amplitude_scales_the_output(cuda, oracle):
    """The tolerance is stated for unit-variance values. Values 64 times larger (a power of
    two: same codes, scales shifted by six exponents) give 64 times the output, and the error
    bound scales with them."""
    rng = np.random.default_rng(21)
    Hq, Hkv, d, S = 8, 2, 128, 16
    cache = hp.build_cache_from_gaussian(oracle, rng, [700, 33], Hkv, d, S)
    q = hp.bf16_from_f32(rng.standard_normal((2, Hq, d)).astype(np.float32))
    base = run_decode(cuda, q, cache, Hq, Hkv, d, S, 2, softmax_scale=0.1)
    loud = dict(cache)
    sc = cache["scale_cache"].copy().reshape(2, -1)
    sc[1] *= np.float32(64.0)   # the value plane of the planar scale cache
    loud["scale_cache"] = sc.reshape(-1)
    got = run_decode(cuda, q, loud, Hq, Hkv, d, S, 2, softmax_scale=0.1)
    want = oracle_decode(oracle, q, loud, Hq, Hkv, d, S, softmax_scale=0.1)
    err = np.abs(got - want)
    assert (err <= 64.0 * ABS_TOL + REL_TOL * np.abs(want)).all()
    assert np.allclose(got, 64.0 * base, rtol=1e-5, atol=64.0 * 1e-5)


def run_partials(cuda, fx, splits, begin, count, seq_len, table_bf16):
    """The reference AIC contract: 16 rows, d=256, records of 272 floats."""
    import torch
    import ascend_micro_harness_b200 as tq
    R, Hd = fx["requests"], fx["heads"]
    ws = torch.empty(R * Hd * splits * 16 * 272, dtype=torch.float32, device=cuda)
    ws.view(torch.int32).fill_(0x7FC0BEEF)
    qrot = torch.full((R * Hd * splits * 16 * 256,), -21846, dtype=torch.int16, device=cuda)  # 0xAAAA
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    tq.decode_splitk_partials(
        dev(cuda, fx["raw_q"]), dev(cuda, table_bf16), dev(cuda, fx["key"]), dev(cuda, fx["value"]),
        dev(cuda, fx["scales"]), dev(cuda, fx["table"]), qrot.view(torch.bfloat16), ws,
        requests=R, heads=Hd, rows=16, head_size=256, block_size=fx["page_tokens"],
        cache_pages=R * fx["pages"], seq_pages=fx["pages"], splits=splits, page_begin=begin,
        page_count=count, seq_len=seq_len, inv_sqrt_len=1.0 / 16, sign_source=tq.SIGNS_TABLES_BF16,
        status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    return (ws.cpu().numpy().reshape(R * Hd, splits, 16, 272),
            qrot.cpu().numpy().view(np.uint16).reshape(R * Hd, splits, 16, 256))


def check_partials(oracle, fx, ws, qrot, splits, begin, count):
    """The tolerances of the reference rig (tests/npu/turboquant_splitk_rigs.hpp:144-215)."""
    R, Hd, pt = fx["requests"], fx["heads"], fx["page_tokens"]
    table = fx["table"].astype(np.int32).reshape(R, fx["pages"])
    q_rot_ref = fx["q_rot"].reshape(R * Hd, 16, 256)
    worst = 0.0
    for item in range(R * Hd):
        req, head = divmod(item, Hd)
        for k in range(splits):
            rb, rc = oracle.partition(count, splits, k)
            m, l, acc = oracle.decode_partial(
                q_rot_ref[item], fx["key"], fx["value"], fx["scales"], table[req], Hd, head, 256,
                pt, R * fx["pages"], fx["seq_len"], (begin + rb) * pt, (begin + rb + rc) * pt)
            rec = ws[item, k]
            live = min((begin + rb + rc) * pt, fx["seq_len"]) > (begin + rb) * pt
            for row in range(16):
                gm, gl, gacc = rec[row, 0], rec[row, 8], rec[row, 16:]
                assert (rec[row, :8] == gm).all() and (rec[row, 8:16] == gl).all()  # not torn
                if not live:
                    assert gm == np.float32(-3e38) and gl == 0 and (gacc == 0).all()
                    continue
                assert abs(gm - m[row]) <= 2e-6 * max(1.0, abs(m[row]))
                assert abs(gl - l[row]) <= 1e-4 * max(1.0, l[row])
                tol = 2e-4 * np.abs(acc[row]).max() + 1e-5 * l[row] + 1e-6
                worst = max(worst, (np.abs(gacc - acc[row]) / tol).max())
            if rc:
                assert np.array_equal(qrot[item, k], q_rot_ref[item]), "q_rot not bit-exact"
            else:
                assert (qrot[item, k] == 0xAAAA).all()
    assert worst <= 1.0, f"accumulator off by {worst:.2f}x the reference rig tolerance"


def load_fixture(reference, n, batch, heads, pt, live=-1, fill=1):
    f = reference.decode_fixture(n, batch, heads, 16, pt, live, fill)
    fx = {k: f.get(k) for k in ("q_rot", "raw_q", "key", "value", "scales", "table")}
    fx.update(requests=batch, heads=heads, pages=f.pages, page_tokens=pt, seq_len=f.seq_len)
    return fx


@pytest.mark.parametrize("pages", [1, 3, 4, 8])
def test_reference_aic_fixture_ladder(cuda, oracle, reference, pages):
    """The reference's own split-K fixture (2 requests x 2 heads, 128-token pages, 16 rows,
    d=256), partitions K=1,2,4,8, whole range and a window that drops the first page."""
    fx = load_fixture(reference, pages * 128, 2, 2, 128)
    table_bf16 = reference.rotation_table_bf16()
    for splits in (1, 2, 4, 8):
        for begin in ((0, 1) if pages > 1 else (0,)):
            count = pages - begin
            ws, qrot = run_partials(cuda, fx, splits, begin, count, fx["seq_len"], table_bf16)
            check_partials(oracle, fx, ws, qrot, splits, begin, count)


@pytest.mark.parametrize("dead,fill", [(1, 2), (15, 2), (127, 2), (40, 1), (40, 0)])
def test_reference_aic_fixture_tails(cuda, oracle, reference, dead, fill):
    """Unaligned contexts: dead slots flooded with zero / adversarial garbage / NaN canaries."""
    pages = 2
    fx = load_fixture(reference, pages * 128, 1, 2, 128, live=pages * 128 - dead, fill=fill)
    table_bf16 = reference.rotation_table_bf16()
    for splits in (1, 2, 4):
        ws, qrot = run_partials(cuda, fx, splits, 0, pages, fx["seq_len"], table_bf16)
        check_partials(oracle, fx, ws, qrot, splits, 0, pages)


@pytest.mark.parametrize("d,Hkv,G", [(128, 8, 4), (256, 4, 4)])
@pytest.mark.parametrize("hint", ["exact", "too_small", "far_too_large", "none"])
def test_the_library_s_own_plan_under_any_hint(cuda, oracle, d, Hkv, G, hint):
    """splits = 0: the launcher cuts every sequence at launch-constant page offsets derived from the
    caller's max_context_hint, graded by head size. The hint is only a hint: whatever it says, every token of
    every sequence must be read exactly once: a hint that is too small leaves the last piece to take the rest,
    one that is far too large leaves all but the first piece empty. Contexts of many lengths around page and
    piece boundaries, next to empty and one-token sequences."""
    import torch
    import ascend_micro_harness_b200 as tq
    rng = np.random.default_rng(d + len(hint))
    S, Hq = 16, Hkv * G
    ctx = [1536, 1535, 1, 0, 345, 346, 344, 691, 1008, 1200, 17, 768, 769, 1537 - 1, 256, 1296]
    cache = hp.build_cache_from_gaussian(oracle, rng, ctx, Hkv, d, S)
    B = len(ctx)
    q = hp.bf16_from_f32(rng.standard_normal((B, Hq, d)).astype(np.float32))
    want = oracle_decode(oracle, q, cache, Hq, Hkv, d, S, softmax_scale=0.1)
    max_blocks = cache["block_tables"].shape[1]
    h = {"exact": max(ctx), "too_small": 300, "far_too_large": 1 << 20, "none": 0}[hint]
    plan_ctx = h if h else max_blocks * S
    n = tq.choose_splits(B, Hkv, S, plan_ctx)
    assert n >= 2 or hint == "too_small"
    ws = torch.full((tq.decode_workspace_floats(B, Hq, Hkv, d, n),), float("nan"), device=cuda)
    out = torch.full((B, Hq, d), float("nan"), dtype=torch.float32, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    tq.decode_splitk(dev(cuda, q), dev(cuda, cache["key_cache"]), dev(cuda, cache["value_cache"]),
                     dev(cuda, cache["scale_cache"]), dev(cuda, cache["block_tables"]),
                     dev(cuda, cache["context_lens"]), dev(cuda, cache["signs"].astype(np.float32)), out,
                     num_heads=Hq, num_kv_heads=Hkv, head_size=d, block_size=S, num_blocks=cache["num_blocks"],
                     inv_sqrt_len=hp.inv_sqrt_len(d), softmax_scale=0.1, splits=0, max_context_hint=h,
                     workspace=ws, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    assert_close(got, want)
