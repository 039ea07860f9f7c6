"""reshape_and_cache (aligned writer) on the GPU through the C ABI vs the CPU oracle:
packed nibbles and FP32 scale bits must be identical, unowned pages untouched."""
import numpy as np
import pytest

from tests import helpers as hp

pytestmark = pytest.mark.gpu

CANARY = 0xAA
WARP_MMA = False
TCGEN05 = False


@pytest.fixture(params=["auto", "tcgen05", "warp_mma"], autouse=True)
def ingest_kernel(request):
    """Every case runs three times: on the kernel the library picks, and on the tcgen05 kernels
    and the warp-MMA kernel forced through their own entry points (any head size, either type)."""
    global WARP_MMA, TCGEN05
    WARP_MMA = request.param == "warp_mma"
    TCGEN05 = request.param == "tcgen05"
    yield


def run_device(cuda, key, value, slots, signs, H, d, S, P, sign_source="f32", status=False):
    import torch
    import ascend_micro_harness_b200 as tq
    tdt = torch.int8 if key.dtype == np.int8 else torch.bfloat16
    k = torch.from_numpy(key.view(np.int8 if key.dtype == np.int8 else np.int16)).to(cuda)
    v = torch.from_numpy(value.view(np.int8 if key.dtype == np.int8 else np.int16)).to(cuda)
    if tdt == torch.bfloat16:
        k, v = k.view(torch.bfloat16), v.view(torch.bfloat16)
    kc = torch.full((P * H * S * d // 2,), CANARY, dtype=torch.uint8, device=cuda)
    vc = torch.full_like(kc, CANARY)
    sc = torch.full((2 * P * H * S,), float("nan"), dtype=torch.float32, device=cuda)
    sc.view(torch.int32).fill_(0x7FC0BEEF)
    sl = torch.from_numpy(slots).to(cuda)
    if sign_source == "f32":
        sg = torch.from_numpy(signs.astype(np.float32)).to(cuda)
        src = tq.SIGNS_F32
    else:
        from oracle.bindings import Oracle
        tables = Oracle().build_tables_i8(signs)
        if sign_source == "tables_i8":
            sg = torch.from_numpy(tables).to(cuda)
            src = tq.SIGNS_TABLES_I8
        else:
            sg = torch.from_numpy(tables.astype(np.float32)).to(cuda).to(torch.bfloat16)
            src = tq.SIGNS_TABLES_BF16
    st = torch.zeros(1, dtype=torch.int32, device=cuda) if status else None
    tq.reshape_and_cache(k, v, kc, vc, sc, sl, sg, num_kv_heads=H, head_size=d, block_size=S,
                         num_blocks=P, inv_sqrt_len=hp.inv_sqrt_len(d), sign_source=src, status=st,
                         warp_mma=WARP_MMA, tcgen05=TCGEN05)
    torch.cuda.synchronize()
    out = kc.cpu().numpy(), vc.cpu().numpy(), sc.cpu().numpy()
    return out + ((int(st.item()),) if status else ())


def expect(oracle, key, value, slots, signs, H, d, S, P):
    kc = np.full(P * H * S * d // 2, CANARY, np.uint8)
    vc = np.full_like(kc, CANARY)
    sc = np.zeros(2 * P * H * S, np.float32)
    sc.view(np.uint32)[:] = 0x7FC0BEEF
    _, _, _, pw, bad = oracle.reshape_and_cache(key, value, slots, signs, H, d, S, P,
                                                hp.inv_sqrt_len(d), kc, vc, sc, threads=8)
    return kc, vc, sc, pw, bad


def assert_identical(got, want):
    kc, vc, sc = got[:3]
    ekc, evc, esc = want[:3]
    assert np.array_equal(kc, ekc), f"key cache differs in {(kc != ekc).sum()} bytes"
    assert np.array_equal(vc, evc), f"value cache differs in {(vc != evc).sum()} bytes"
    assert np.array_equal(sc.view(np.uint32), esc.view(np.uint32)), "scale bits differ"


def test_config1_a8_single_strip(cuda, oracle):
    """The single-strip benchmark configuration: 16 tokens, 1 KV head, d=128, int8 U[-127,127], identity slots."""
    rng = np.random.default_rng(0x7151)
    k, v = hp.int8_activations(rng, 16, 1, 128)
    slots = np.arange(16, dtype=np.int32)
    signs = oracle.writer_signs(128)
    for src in ("f32", "tables_i8"):
        got = run_device(cuda, k, v, slots, signs, 1, 128, 16, 1, src)
        assert_identical(got, expect(oracle, k, v, slots, signs, 1, 128, 16, 1))


@pytest.mark.parametrize("strips", [1, 33, 148, 149, 600])
@pytest.mark.parametrize("dtype", ["int8", "bf16"])
def test_reference_geometry_ladder(cuda, oracle, strips, dtype):
    """The reference harness geometry (4 heads x 256) on fragmented pages 2s+1, over a
    ladder chosen around the SM count instead of the 32 AI cores."""
    H, d = 4, 256
    rng = np.random.default_rng(strips)
    k, v = hp.int8_activations(rng, strips * 16, H, d)
    k[0, 0], k[1, 1], v[0, 0], v[1, 1] = -128, 127, 127, -128
    slots, P = hp.fragmented_slots(strips)
    signs = oracle.writer_signs(d)
    want = expect(oracle, k, v, slots, signs, H, d, 16, P)
    if dtype == "bf16":
        k, v = hp.bf16_from_f32(k.astype(np.float32)), hp.bf16_from_f32(v.astype(np.float32))
        src = "tables_bf16"
    else:
        src = "tables_i8"
    got = run_device(cuda, k, v, slots, signs, H, d, 16, P, src)
    assert_identical(got, want)
    # every page no strip owns still holds its canary
    kc = got[0].reshape(P, -1)
    assert (kc[0::2] == CANARY).all()


@pytest.mark.parametrize("S", [64, 128])
@pytest.mark.parametrize("d", [128, 256])
def test_large_pages_strips_at_in_page_offsets(cuda, oracle, S, d):
    """Pages of 64 and 128 tokens (a serving stack's page sizes): strips land at every
    in-page offset, pages are scattered, some pages stay partly unwritten."""
    rng = np.random.default_rng(S + d)
    H, strips = 2, 150
    k, v = hp.gaussian_outlier_activations(rng, strips * 16, H, d, integer=True)
    per_page = S // 16
    P = (strips + per_page - 1) // per_page + 3
    pages = rng.permutation(P)
    where = rng.permutation(P * per_page)[:strips]            # (page, in-page strip) per strip
    slots = ((pages[where // per_page] * S + (where % per_page) * 16)[:, None] +
             np.arange(16)[None, :]).astype(np.int32).reshape(-1)
    signs = hp.random_signs(rng, d)
    got = run_device(cuda, k, v, slots, signs, H, d, S, P)
    assert_identical(got, expect(oracle, k, v, slots, signs, H, d, S, P))


def test_config2_bf16_integer_valued(cuda, oracle):
    """The bf16 prefill benchmark configuration, bit-exact leg: 1024 tokens x 8 heads x 128, integer-valued bf16,
    seeded page permutation of 64 pages."""
    rng = np.random.default_rng(2)
    H, d, T = 8, 128, 1024
    k, v = hp.gaussian_outlier_activations(rng, T, H, d, integer=True)
    slots, P = hp.page_permutation_slots(rng, T // 16)
    signs = hp.random_signs(rng, d)
    got = run_device(cuda, k, v, slots, signs, H, d, 16, P)
    assert_identical(got, expect(oracle, k, v, slots, signs, H, d, 16, P))


def test_config2_bf16_gaussian_outliers(cuda, oracle):
    """The bf16 prefill benchmark configuration as stated (non-integer bf16): the FP32 accumulation order is
    free, so codes may differ from the FP64-rotated oracle only at rounding ties."""
    rng = np.random.default_rng(3)
    H, d, T = 8, 128, 1024
    k, v = hp.gaussian_outlier_activations(rng, T, H, d)
    slots, P = hp.page_permutation_slots(rng, T // 16)
    signs = hp.random_signs(rng, d)
    kc, vc, sc = run_device(cuda, k, v, slots, signs, H, d, 16, P)
    ekc, evc, esc, _, _ = expect(oracle, k, v, slots, signs, H, d, 16, P)
    assert np.array_equal(sc.view(np.uint32), esc.view(np.uint32))
    for a, b in ((kc, ekc), (vc, evc)):
        lo = (a & 15).astype(np.int16) - (b & 15).astype(np.int16)
        hi = (a >> 4).astype(np.int16) - (b >> 4).astype(np.int16)
        diff = np.concatenate([lo, hi])
        diff = np.where(diff > 8, diff - 16, np.where(diff < -8, diff + 16, diff))
        assert np.abs(diff).max() <= 1
        assert (diff != 0).mean() < 1e-4


def test_zero_rows_and_extremes(cuda, oracle):
    """All-zero tokens take the absmax floor (scale 2^-2/sqrt(d)); +-128/127 saturate."""
    H, d = 2, 128
    k = np.zeros((32, H * d), np.int8)
    v = np.zeros((32, H * d), np.int8)
    k[3, :] = -128
    v[4, :] = 127
    k[5, 7] = 1
    slots, P = hp.fragmented_slots(2)
    signs = oracle.writer_signs(d)
    got = run_device(cuda, k, v, slots, signs, H, d, 16, P)
    assert_identical(got, expect(oracle, k, v, slots, signs, H, d, 16, P))


def test_bad_slot_run_is_skipped_and_reported(cuda, oracle):
    """A strip whose slots are not one aligned run writes nothing and sets the status."""
    import ascend_micro_harness_b200 as tq
    rng = np.random.default_rng(5)
    H, d = 1, 128
    k, v = hp.int8_activations(rng, 48, H, d)
    slots, P = hp.fragmented_slots(3)
    slots[16 + 5] += 1          # strip 1: broken run
    signs = oracle.writer_signs(d)
    want = expect(oracle, k, v, slots, signs, H, d, 16, P)
    assert want[4] == 1
    got = run_device(cuda, k, v, slots, signs, H, d, 16, P, status=True)
    assert_identical(got, want)
    assert got[3] & tq.STATUS_BAD_SLOT


@pytest.mark.parametrize("d", [128, 256])
@pytest.mark.parametrize("dtype", ["int8", "bf16"])
def test_wait_that_runs_out_is_reported_and_nothing_is_stored(cuda, oracle, dtype, d):
    """tcgen05 writers: with a wait budget of zero every wait on a tile fetch gives up at once. The
    launch must set STATUS_WAIT_EXPIRED, store nothing, let its fetches land and return; the next
    launch with the default budget, in the same context, is exact again."""
    import ascend_micro_harness_b200 as tq
    if WARP_MMA:
        pytest.skip("the warp-MMA writer has no barrier waits")
    rng = np.random.default_rng(77)
    H, strips = 4, 2400                   # more (tile, head) items than resident groups
    k, v = hp.int8_activations(rng, strips * 16, H, d)
    slots, P = hp.fragmented_slots(strips)
    signs = oracle.writer_signs(d)
    want = expect(oracle, k, v, slots, signs, H, d, 16, P)
    if dtype == "bf16":
        k, v = hp.bf16_from_f32(k.astype(np.float32)), hp.bf16_from_f32(v.astype(np.float32))
    tq.set_ingest_wait_budget(0)
    try:
        kc, vc, sc, status = run_device(cuda, k, v, slots, signs, H, d, 16, P, status=True)
    finally:
        tq.set_ingest_wait_budget(-1)
    assert status & tq.STATUS_WAIT_EXPIRED
    assert (kc == CANARY).all() and (vc == CANARY).all()
    assert (sc.view(np.uint32) == 0x7FC0BEEF).all()
    got = run_device(cuda, k, v, slots, signs, H, d, 16, P, status=True)
    assert_identical(got, want)
    assert got[3] == 0


@pytest.mark.parametrize("d", [128, 256])
def test_int8_rows_at_the_accumulator_extremes(cuda, oracle, d):
    """int8 rows whose rotated sums reach +-128 * d (a row of -128s against a sign row of all
    ones or of all minus ones, and its mirror), next to rows of zeros and of single +-1 entries:
    the absmax read from the low halves of the accumulators must still be exact. At d = 256 the
    sum +32768 does not fit a signed 16-bit lane."""
    rng = np.random.default_rng(404)
    H, strips = 2, 9
    k, v = hp.int8_activations(rng, strips * 16, H, d)
    signs = np.ones(d, np.float32)
    k[0, :], k[1, :], k[2, :] = -128, 127, 0
    v[0, :], v[1, :], v[2, :] = 127, -128, 0
    k[3, :], v[3, :] = 0, 0
    k[3, 5], v[3, 77] = 1, -1
    k[4, :d] = -128                      # head 0 only
    v[5, d:] = -128                      # head 1 only
    slots, P = hp.fragmented_slots(strips)
    for sg in (signs, -signs, oracle.writer_signs(d)):
        got = run_device(cuda, k, v, slots, sg, H, d, 16, P)
        assert_identical(got, expect(oracle, k, v, slots, sg, H, d, 16, P))


def test_partial_strip_is_refused(cuda):
    import torch
    import ascend_micro_harness_b200 as tq
    z = torch.zeros(24 * 128, dtype=torch.int8, device=cuda)
    c = torch.zeros(4096, dtype=torch.uint8, device=cuda)
    s = torch.zeros(256, dtype=torch.float32, device=cuda)
    sl = torch.zeros(24, dtype=torch.int32, device=cuda)
    sg = torch.ones(128, dtype=torch.float32, device=cuda)
    with pytest.raises(tq.TqError) as e:
        tq.reshape_and_cache(z, z, c, c, s, sl, sg, num_kv_heads=1, head_size=128, block_size=16,
                             num_blocks=2, inv_sqrt_len=0.1)
    assert e.value.status == 2


@pytest.mark.parametrize("d,S", [(128, 16), (128, 64), (256, 128)])
def test_ragged_requests_with_tail_strips(cuda, oracle, d, S):
    """The aligned writer over requests of any length: strips are cut per request, a short
    last strip writes its own key rows and scales only and the whole value strip with zeros
    for the missing tokens; everything else keeps its canary."""
    import torch
    import ascend_micro_harness_b200 as tq
    if WARP_MMA or TCGEN05:
        pytest.skip("one kernel serves this entry")
    rng = np.random.default_rng(d + S)
    H = 2
    lens = [1, 15, 16, 17, 79, 257, 33, 160]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    T = int(cu[-1])
    k, v = hp.gaussian_outlier_activations(rng, T, H, d, integer=True)
    per_page = S // 16
    strips = [(n + 15) // 16 for n in lens]
    # every request starts on a fresh page; its strips fill consecutive in-page positions
    pages_needed = sum((s + per_page - 1) // per_page for s in strips)
    P = pages_needed + 3
    perm = rng.permutation(P)
    slots = np.zeros(T, np.int32)
    at = 0
    for b, n in enumerate(lens):
        for t in range(n):
            page = perm[at + t // S]
            slots[cu[b] + t] = page * S + t % S
        at += (strips[b] + per_page - 1) // per_page
    signs = hp.random_signs(rng, d)
    kc = torch.full((P * H * S * d // 2,), CANARY, dtype=torch.uint8, device=cuda)
    vc = torch.full_like(kc, CANARY)
    sc = torch.zeros(2 * P * H * S, dtype=torch.float32, device=cuda)
    sc.view(torch.int32).fill_(0x7FC0BEEF)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    kd = torch.from_numpy(k.view(np.int16)).to(cuda).view(torch.bfloat16)
    vd = torch.from_numpy(v.view(np.int16)).to(cuda).view(torch.bfloat16)
    tq.reshape_and_cache_varlen(kd, vd, kc, vc, sc, torch.from_numpy(slots).to(cuda),
                                torch.from_numpy(signs.astype(np.float32)).to(cuda), cu, num_kv_heads=H,
                                head_size=d, block_size=S, num_blocks=P, inv_sqrt_len=hp.inv_sqrt_len(d),
                                status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    ekc = np.full(P * H * S * d // 2, CANARY, np.uint8)
    evc = np.full_like(ekc, CANARY)
    esc = np.zeros(2 * P * H * S, np.float32)
    esc.view(np.uint32)[:] = 0x7FC0BEEF
    assert oracle.reshape_and_cache_varlen(k, v, slots, signs, cu, H, d, S, P, hp.inv_sqrt_len(d), ekc, evc,
                                           esc) == 0
    assert_identical((kc.cpu().numpy(), vc.cpu().numpy(), sc.cpu().numpy()), (ekc, evc, esc))
