"""The torch.library registration: schemas and FakeTensor tracing on the CPU, the ops
themselves against the oracle on the GPU."""
import numpy as np
import pytest

from tests import helpers as hp


def test_ops_are_registered_with_meta_kernels():
    import torch
    import ascend_micro_harness_b200.torch_ops  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode
    ns = torch.ops.tq_b200
    for name in ("reshape_aligned", "reshape_scatter", "rotate_q_batch", "paged_decode", "decode_combine",
                 "decode_workspace_size"):
        assert hasattr(ns, name)
    assert ns.decode_workspace_size(64, 32, 8, 128, 4) == 64 * 8 * 4 * 4 * (16 + 128) + 64 * 8 + 4
    with FakeTensorMode():
        H, d, S, P, T = 8, 128, 16, 4, 32
        k = torch.empty(T, H * d, dtype=torch.bfloat16, device="cuda")
        kc = torch.empty(P * H * S * d // 2, dtype=torch.uint8, device="cuda")
        vc = torch.empty_like(kc)
        sc = torch.empty(2 * P * H * S, dtype=torch.float32, device="cuda")
        sl = torch.empty(T, dtype=torch.int32, device="cuda")
        sg = torch.empty(d, dtype=torch.float32, device="cuda")
        ns.reshape_aligned(k, k, kc, vc, sc, sl, sg, H, d, S)
        ns.reshape_aligned(k, k, kc, vc, sc, sl, sg, H, d, S, [0, 20, 32])
        ns.reshape_scatter(k[:2], k[:2], kc, vc, sc, sl[:2], sg, H, d, S)
        q = torch.empty(2, 32, d, dtype=torch.bfloat16, device="cuda")
        ns.rotate_q_batch(q, sg, torch.empty_like(q), d)
        ws = torch.empty(ns.decode_workspace_size(2, 32, H, d, 2), dtype=torch.float32, device="cuda")
        out = torch.empty(2, 32, d, dtype=torch.float32, device="cuda")
        bt = torch.empty(2, 2, dtype=torch.int32, device="cuda")
        ns.paged_decode(q, None, kc, vc, sc, bt, sl[:2], sg, ws, 32, H, S, 2, 0.1, 0, out)
        ns.decode_combine(ws, None, sg, 32, H, 2, 1, out)


@pytest.mark.gpu
def test_ops_on_the_gpu_match_the_oracle(cuda, oracle):
    import torch
    import ascend_micro_harness_b200.torch_ops  # noqa: F401
    ns = torch.ops.tq_b200
    rng = np.random.default_rng(8)
    H, Hq, d, S = 2, 8, 128, 16
    lens = [40, 16, 7]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    T = int(cu[-1])
    k, v = hp.gaussian_outlier_activations(rng, T, H, d, integer=True)
    pages_per = [(n + S - 1) // S for n in lens]
    P = sum(pages_per) + 2
    perm = rng.permutation(P)
    tables = np.zeros((3, max(pages_per)), np.int32)
    slots = np.zeros(T, np.int32)
    at = 0
    for b, n in enumerate(lens):
        tables[b, :pages_per[b]] = perm[at:at + pages_per[b]]
        at += pages_per[b]
        for t in range(n):
            slots[cu[b] + t] = tables[b, t // S] * S + t % S
    signs = hp.random_signs(rng, d)

    def bf(a):
        return torch.from_numpy(a.view(np.int16)).to(cuda).view(torch.bfloat16)

    kc = torch.zeros(P * H * S * d // 2, dtype=torch.uint8, device=cuda)
    vc = torch.zeros_like(kc)
    sc = torch.ones(2 * P * H * S, dtype=torch.float32, device=cuda)
    sg = torch.from_numpy(signs.astype(np.float32)).to(cuda)
    ns.reshape_aligned(bf(k), bf(v), kc, vc, sc, torch.from_numpy(slots).to(cuda), sg, H, d, S, cu.tolist())
    ekc = np.zeros(P * H * S * d // 2, np.uint8)
    evc = np.zeros_like(ekc)
    esc = np.ones(2 * P * H * S, np.float32)
    oracle.reshape_and_cache_varlen(k, v, slots, signs, cu, H, d, S, P, hp.inv_sqrt_len(d), ekc, evc, esc)
    torch.cuda.synchronize()
    assert np.array_equal(kc.cpu().numpy(), ekc) and np.array_equal(vc.cpu().numpy(), evc)
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), esc.view(np.uint32))

    # one more token per request through the scatter op, then decode through the ops
    k1, v1 = hp.gaussian_outlier_activations(rng, 3, H, d)
    new_slots = np.array([tables[b, lens[b] // S] * S + lens[b] % S for b in range(3)], np.int32)
    ns.reshape_scatter(bf(k1), bf(v1), kc, vc, sc, torch.from_numpy(new_slots).to(cuda), sg, H, d, S)
    oracle.reshape_scatter(k1, v1, new_slots, signs.astype(np.float32), None, 3, H, d, S, P,
                           hp.inv_sqrt_len(d), ekc, evc, esc)
    torch.cuda.synchronize()
    assert np.array_equal(kc.cpu().numpy(), ekc) and np.array_equal(vc.cpu().numpy(), evc)

    q = hp.bf16_from_f32(rng.standard_normal((3, Hq, d)).astype(np.float32))
    q_rot = torch.zeros((3, Hq, d), dtype=torch.bfloat16, device=cuda)
    ns.rotate_q_batch(bf(q), sg, q_rot, d)
    want_rot = oracle.rotate_query_bf16(q.reshape(-1, d), signs.astype(np.float32), hp.inv_sqrt_len(d))
    assert np.array_equal(q_rot.view(torch.int16).cpu().numpy().view(np.uint16).reshape(-1, d),
                          np.asarray(want_rot).reshape(-1, d))

    ctx = np.array([n + 1 for n in lens], np.int32)
    splits = 2
    ws = torch.full((ns.decode_workspace_size(3, Hq, H, d, splits),), float("nan"), device=cuda)
    out = torch.zeros((3, Hq, d), dtype=torch.float32, device=cuda)
    ns.paged_decode(bf(q), None, kc, vc, sc, torch.from_numpy(tables).to(cuda), torch.from_numpy(ctx).to(cuda),
                    sg, ws, Hq, H, S, splits, 0.1, 1, out)
    torch.cuda.synchronize()
    want = oracle.decode(q, ekc, evc, esc, tables, ctx, signs.astype(np.float32), Hq, H, d, S, P,
                         hp.inv_sqrt_len(d), 0.1, 1, None, threads=4)
    got = out.cpu().numpy()
    # the activations of this case are integers of scale 16 (so that the writers can be checked
    # bit for bit): the absolute part of the decode tolerance scales with them
    assert (np.abs(got - want) <= 16 * 1e-3 + 2e-3 * np.abs(want)).all()
    out2 = torch.zeros_like(out)
    ns.decode_combine(ws, None, sg, Hq, H, splits, 1, out2)
    torch.cuda.synchronize()
    assert torch.equal(out, out2)
