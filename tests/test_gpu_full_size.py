"""The benchmark-sized workloads on the GPU. The FP64 / integer oracles are too slow to check
every output at these sizes, so the cases combine
  * size-independent properties (the two aligned-writer kernels agree byte for byte; the
    decode result does not depend on the split count, on how pages are scattered through the
    pool, or on what lies in dead slots), with
  * the oracle on a sample of the same launch (a few hundred strips, a few sequences)."""
import numpy as np
import pytest

from tests import helpers as hp

pytestmark = pytest.mark.gpu

ABS_TOL, REL_TOL = 1e-3, 2e-3


def _bf16_dev(cuda, a):
    import torch
    return torch.from_numpy(a.view(np.int16)).to(cuda).view(torch.bfloat16)


def test_prefill_262144_tokens_both_kernels_and_sampled_oracle(cuda, oracle):
    """bf16 prefill at the benchmark's size (262 144 tokens x 8 KV heads x 128, 1.4 GB moved),
    integer-valued so that every byte is pinned."""
    import torch
    import ascend_micro_harness_b200 as tq
    T, H, d, S = 262144, 8, 128, 16
    g = torch.Generator(device=cuda)
    g.manual_seed(7)
    k = torch.randint(-127, 128, (T, H * d), device=cuda, generator=g).to(torch.bfloat16)
    v = torch.randint(-127, 128, (T, H * d), device=cuda, generator=g).to(torch.bfloat16)
    P = T // S + 5
    perm = torch.randperm(P, device=cuda, generator=g)[: T // S]
    slots = (perm[:, None] * S + torch.arange(S, device=cuda)[None, :]).reshape(-1).int().contiguous()
    rng = np.random.default_rng(7)
    signs_np = hp.random_signs(rng, d)
    signs = torch.from_numpy(signs_np.astype(np.float32)).to(cuda)
    out = []
    for warp_mma, tcgen05 in ((False, False), (True, False), (False, True)):
        kc = torch.full((P * H * S * d // 2,), 0xAA, dtype=torch.uint8, device=cuda)
        vc = torch.full_like(kc, 0xAA)
        sc = torch.full((2 * P * H * S,), float("nan"), dtype=torch.float32, device=cuda)
        st = torch.zeros(1, dtype=torch.int32, device=cuda)
        tq.reshape_and_cache(k, v, kc, vc, sc, slots, signs, num_kv_heads=H, head_size=d,
                             block_size=S, num_blocks=P, inv_sqrt_len=hp.inv_sqrt_len(d), status=st,
                             warp_mma=warp_mma, tcgen05=tcgen05)
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        out.append((kc, vc, sc))
    assert torch.equal(out[0][0], out[1][0]) and torch.equal(out[0][1], out[1][1])
    assert torch.equal(out[0][0], out[2][0]) and torch.equal(out[0][1], out[2][1])
    assert torch.equal(out[0][2].view(torch.int32), out[1][2].view(torch.int32))
    # the five pages no strip owns keep their canaries
    owned = torch.zeros(P, dtype=torch.bool, device=cuda)
    owned[perm] = True
    free = (~owned).nonzero().flatten()
    page_bytes = H * S * d // 2
    for pg in free.tolist():
        assert bool((out[0][0][pg * page_bytes:(pg + 1) * page_bytes] == 0xAA).all())
    # oracle on 256 sampled strips, written into a private small pool
    pick = np.sort(rng.choice(T // S, size=256, replace=False))
    rows = (pick[:, None] * S + np.arange(S)[None, :]).reshape(-1)
    rows_t = torch.from_numpy(rows).to(cuda)
    ks = k[rows_t].view(torch.int16).cpu().numpy().view(np.uint16)
    vs = v[rows_t].view(torch.int16).cpu().numpy().view(np.uint16)
    small_slots = np.arange(256 * S, dtype=np.int32)
    ekc = np.zeros(256 * H * S * d // 2, np.uint8)
    evc = np.zeros_like(ekc)
    esc = np.zeros(2 * 256 * H * S, np.float32)
    oracle.reshape_and_cache(ks, vs, small_slots, signs_np, H, d, S, 256, hp.inv_sqrt_len(d), ekc, evc,
                             esc, threads=8)
    pages = perm[torch.from_numpy(pick).to(cuda)]
    idx = (pages[:, None] * page_bytes + torch.arange(page_bytes, device=cuda)[None, :]).reshape(-1)
    assert np.array_equal(out[0][0][idx].cpu().numpy(), ekc)
    assert np.array_equal(out[0][1][idx].cpu().numpy(), evc)
    sidx = (pages[:, None] * (H * S) + torch.arange(H * S, device=cuda)[None, :]).reshape(-1)
    got_ks = out[0][2][sidx].cpu().numpy()
    got_vs = out[0][2][P * H * S + sidx].cpu().numpy()
    assert np.array_equal(got_ks.view(np.uint32), esc[:256 * H * S].view(np.uint32))
    assert np.array_equal(got_vs.view(np.uint32), esc[256 * H * S:].view(np.uint32))


def _random_cache(torch, cuda, ctx, Hkv, d, S, seed, spare=16):
    """A quantised cache generated directly on the device, pages scattered through the pool."""
    B = len(ctx)
    pages_per_seq = (ctx + S - 1) // S
    P = int(pages_per_seq.sum()) + spare
    rng = np.random.default_rng(seed)
    perm = rng.permutation(P)
    tables = np.zeros((B, int(pages_per_seq.max())), np.int32)
    at = 0
    for b in range(B):
        n = int(pages_per_seq[b])
        tables[b, :n] = perm[at:at + n]
        at += n
    g = torch.Generator(device=cuda)
    g.manual_seed(seed)
    nbytes = P * Hkv * S * d // 2
    kc = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device=cuda, generator=g)
    vc = torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device=cuda, generator=g)
    e = torch.randint(0, 3, (2 * P * Hkv * S,), device=cuda, generator=g)
    sc = (torch.ldexp(torch.ones_like(e, dtype=torch.float32), e - 2) * hp.inv_sqrt_len(d)).contiguous()
    return dict(P=P, tables=tables, kc=kc, vc=vc, sc=sc, perm=perm)


def _decode(torch, tq, cuda, q, c, ctx, Hq, Hkv, d, S, splits):
    B = len(ctx)
    use = splits if splits else tq.choose_splits(B, Hkv, S, int(ctx.max()))
    ws = torch.full((tq.decode_workspace_floats(B, Hq, Hkv, d, use),), float("nan"), device=cuda)
    out = torch.zeros((B, Hq, d), dtype=torch.float32, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    tq.decode_splitk(q, c["kc"], c["vc"], c["sc"], torch.from_numpy(c["tables"]).to(cuda),
                     torch.from_numpy(ctx.astype(np.int32)).to(cuda), c["signs"], out, num_heads=Hq,
                     num_kv_heads=Hkv, head_size=d, block_size=S, num_blocks=c["P"],
                     inv_sqrt_len=hp.inv_sqrt_len(d), softmax_scale=float(1 / np.sqrt(d)), splits=splits,
                     max_context_hint=int(ctx.max()), workspace=ws, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    return out


def _oracle_subset(oracle, torch, q, c, ctx, pick, Hq, Hkv, d, S):
    """FP64 oracle for the sequences in `pick`, on a private copy of just their pages."""
    page_bytes = Hkv * S * d // 2
    tables, remap, at = c["tables"], [], 0
    sub_tables = np.zeros((len(pick), tables.shape[1]), np.int32)
    for i, b in enumerate(pick):
        n = int((ctx[b] + S - 1) // S)
        remap.extend(tables[b, :n].tolist())
        sub_tables[i, :n] = np.arange(at, at + n)
        at += n
    pages = torch.tensor(remap, device=c["kc"].device)
    idx = (pages[:, None] * page_bytes + torch.arange(page_bytes, device=pages.device)[None, :]).reshape(-1)
    kc, vc = c["kc"][idx].cpu().numpy(), c["vc"][idx].cpu().numpy()
    sidx = (pages[:, None] * (Hkv * S) + torch.arange(Hkv * S, device=pages.device)[None, :]).reshape(-1)
    sc = torch.cat([c["sc"][sidx], c["sc"][c["P"] * Hkv * S + sidx]]).cpu().numpy()
    qs = q[torch.tensor(pick, device=q.device)].view(torch.int16).cpu().numpy().view(np.uint16)
    return oracle.decode(qs, kc, vc, sc, sub_tables, ctx[pick].astype(np.int32),
                         c["signs"].cpu().numpy(), Hq, Hkv, d, S, at, hp.inv_sqrt_len(d),
                         float(1 / np.sqrt(d)), 0, None, threads=8)


def _close(got, want):
    err = np.abs(got - want)
    return float((err / (ABS_TOL + REL_TOL * np.abs(want))).max())


def test_ragged_batch_64_sequences_to_32768_tokens(cuda, oracle):
    """The benchmark batch (64 sequences, 512..32768 tokens, 32 q / 8 KV heads, d = 128):
    the library's plan, one fixed split count and no splitting agree; a re-scattered copy of
    the cache gives the same output bit for bit; sampled sequences match the FP64 oracle."""
    import torch
    import ascend_micro_harness_b200 as tq
    Hq, Hkv, d, S = 32, 8, 128, 16
    rng = np.random.default_rng(4)
    ctx = rng.integers(512, 32769, size=64)
    c = _random_cache(torch, cuda, ctx, Hkv, d, S, seed=4)
    c["signs"] = torch.from_numpy(hp.random_signs(rng, d).astype(np.float32)).to(cuda)
    g = torch.Generator(device=cuda)
    g.manual_seed(5)
    q = torch.randn((64, Hq, d), device=cuda, generator=g).bfloat16()
    auto = _decode(torch, tq, cuda, q, c, ctx, Hq, Hkv, d, S, 0).cpu().numpy()
    fixed = _decode(torch, tq, cuda, q, c, ctx, Hq, Hkv, d, S, 16).cpu().numpy()
    single = _decode(torch, tq, cuda, q, c, ctx, Hq, Hkv, d, S, 1).cpu().numpy()
    assert _close(fixed, auto) <= 1.0 and _close(single, auto) <= 1.0
    # the same logical cache with every page moved elsewhere in a bigger pool
    P2 = c["P"] + 1000
    move = torch.from_numpy(np.random.default_rng(9).permutation(P2)[: c["P"]]).to(cuda)
    page_bytes = Hkv * S * d // 2
    c2 = dict(P=P2, signs=c["signs"])
    c2["kc"] = torch.full((P2 * page_bytes,), 0xAA, dtype=torch.uint8, device=cuda)
    c2["vc"] = torch.full_like(c2["kc"], 0xAA)
    c2["kc"].view(P2, page_bytes)[move] = c["kc"].view(c["P"], page_bytes)
    c2["vc"].view(P2, page_bytes)[move] = c["vc"].view(c["P"], page_bytes)
    sc2 = torch.full((2, P2, Hkv * S), float("nan"), device=cuda)
    sc2[:, move] = c["sc"].view(2, c["P"], Hkv * S)
    c2["sc"] = sc2.reshape(-1).contiguous()
    c2["tables"] = move.cpu().numpy()[c["tables"]].astype(np.int32)
    moved = _decode(torch, tq, cuda, q, c2, ctx, Hq, Hkv, d, S, 0).cpu().numpy()
    assert np.array_equal(moved, auto)
    pick = [int(np.argmin(ctx)), int(np.argmax(ctx)), 17]
    want = _oracle_subset(oracle, torch, q, c, ctx, pick, Hq, Hkv, d, S)
    assert _close(auto[pick], want) <= 1.0


def test_long_context_share_16_sequences_of_65536_tokens(cuda, oracle):
    """One GPU's share of the 128 x 65 536-token configuration on 8 GPUs (1.1 GB of cache):
    dead slots poisoned, split counts agree, two sequences checked against the FP64 oracle."""
    import torch
    import ascend_micro_harness_b200 as tq
    Hq, Hkv, d, S = 32, 8, 128, 16
    ctx = np.full(16, 65536) - np.array([0, 1, 15, 16, 17, 100, 0, 0, 3, 0, 0, 7, 0, 0, 0, 9])
    c = _random_cache(torch, cuda, ctx, Hkv, d, S, seed=11)
    rng = np.random.default_rng(11)
    c["signs"] = torch.from_numpy(hp.random_signs(rng, d).astype(np.float32)).to(cuda)
    # NaN scales in every slot past a sequence's last token
    sc = c["sc"].view(2, c["P"], Hkv, S)
    for b, n in enumerate(ctx):
        if n % S:
            sc[:, int(c["tables"][b, n // S]), :, n % S:] = float("nan")
    g = torch.Generator(device=cuda)
    g.manual_seed(12)
    q = torch.randn((16, Hq, d), device=cuda, generator=g).bfloat16()
    auto = _decode(torch, tq, cuda, q, c, ctx, Hq, Hkv, d, S, 0).cpu().numpy()
    assert np.isfinite(auto).all()
    eight = _decode(torch, tq, cuda, q, c, ctx, Hq, Hkv, d, S, 8).cpu().numpy()
    assert _close(eight, auto) <= 1.0
    pick = [2, 5]
    want = _oracle_subset(oracle, torch, q, c, ctx, pick, Hq, Hkv, d, S)
    assert _close(auto[pick], want) <= 1.0
