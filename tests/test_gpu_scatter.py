"""reshape_scatter (1..16-token writer, value-strip read-modify-write) vs the CPU oracle."""
import numpy as np
import pytest

from tests import helpers as hp

pytestmark = pytest.mark.gpu


def run_scatter(cuda, kb, vb, slots, signs, cu, nreq, H, d, S, P, kc, vc, sc):
    import torch
    import ascend_micro_harness_b200 as tq

    def t(a):
        if a.dtype == np.uint16:
            return torch.from_numpy(a.view(np.int16)).to(cuda).view(torch.bfloat16)
        return torch.from_numpy(a).to(cuda)
    dk, dv, ds = t(kc), t(vc), t(sc)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    tq.reshape_scatter(t(kb), t(vb), dk, dv, ds, t(slots), t(signs.astype(np.float32)),
                       None if cu is None else t(np.asarray(cu, np.int32)), num_requests=nreq,
                       num_kv_heads=H, head_size=d, block_size=S, num_blocks=P,
                       inv_sqrt_len=hp.inv_sqrt_len(d), status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    return dk.cpu().numpy(), dv.cpu().numpy(), ds.cpu().numpy()


@pytest.mark.parametrize("d", [128, 256])
@pytest.mark.parametrize("S", [16, 64])
@pytest.mark.parametrize("integer", [True, False])
def test_scatter_matches_oracle(cuda, oracle, d, S, integer):
    rng = np.random.default_rng(d + S + integer)
    H, P = 3, 12
    cu = [0, 1, 4, 4, 12, 13]          # 1, 3, 0, 8, 1 tokens
    nreq, T = len(cu) - 1, cu[-1]
    x = rng.standard_normal((2, T, H * d)).astype(np.float32) * 3
    if integer:
        x = np.clip(np.rint(x * 8), -127, 127)
    x[:, 2, :] = 0.0                    # an all-zero token: the absmax == 0 branch
    kb, vb = hp.bf16_from_f32(x[0]), hp.bf16_from_f32(x[1])
    slots = np.array([5, 20, 21, 22, 100, 101, 102, -1, 110, 111, 112, 113, S * 11 + S - 1],
                     np.int32)
    slots = np.minimum(slots, P * S - 1).astype(np.int32)
    slots[7] = -1
    signs = hp.random_signs(rng, d)
    kc = rng.integers(0, 256, P * H * S * d // 2, dtype=np.uint8)
    vc = rng.integers(0, 256, P * H * S * d // 2, dtype=np.uint8)
    sc = rng.standard_normal(2 * P * H * S).astype(np.float32)
    ekc, evc, esc = kc.copy(), vc.copy(), sc.copy()
    assert oracle.reshape_scatter(kb, vb, slots, signs, cu, nreq, H, d, S, P, hp.inv_sqrt_len(d),
                                  ekc, evc, esc) == 0
    gkc, gvc, gsc = run_scatter(cuda, kb, vb, slots, signs, cu, nreq, H, d, S, P, kc, vc, sc)
    assert np.array_equal(gkc, ekc)
    assert np.array_equal(gvc, evc)       # includes every preserved neighbour nibble
    assert np.array_equal(gsc.view(np.uint32), esc.view(np.uint32))


def test_scatter_reference_fixture(cuda, oracle, reference):
    """The reference's own scatter fixture (d=256) including its zero-token row."""
    H, S, P = 4, 16, 8
    rng = np.random.default_rng(1)
    cu = [0, 3, 8]
    slots = np.array([32, 33, 34, 70, 71, 72, -1, 90], np.int32)
    kc = rng.integers(0, 256, P * H * S * 128, dtype=np.uint8)
    vc = rng.integers(0, 256, P * H * S * 128, dtype=np.uint8)
    sc = rng.standard_normal(2 * P * H * S).astype(np.float32)
    ekc, evc, esc = kc.copy(), vc.copy(), sc.copy()
    zero_rows, kb, vb = reference.scatter_reference(2, H, S, P, slots, cu, 1, ekc, evc, esc)
    assert zero_rows > 0
    signs = reference.writer_signs(256)
    gkc, gvc, gsc = run_scatter(cuda, kb, vb, slots, signs, cu, 2, H, 256, S, P, kc, vc, sc)
    assert np.array_equal(gkc, ekc) and np.array_equal(gvc, evc)
    assert np.array_equal(gsc.view(np.uint32), esc.view(np.uint32))
