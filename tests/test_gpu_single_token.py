"""The reference's single-token decode fixture on the GPU: 6 query rows per KV head (the row
count the vector-only score routine routines/routine_vector_decode_gemv.hpp:183-253 serves),
head size 256, 128-token pages, a block table that is not the identity. The partial records of
tq_decode_splitk_partials and the gated context of tq_decode_splitk are held to the golden
model of tests/common/single_token_decode_oracle.hpp:256-336 (tests/golden/single_token_p2.npz)
with the tolerances the reference's own rig uses for partial records
(tests/npu/turboquant_splitk_rigs.hpp:144-215)."""
import numpy as np
import pytest

from tests.test_oracle_single_token import D, HEADS, P, PAGES, ROWS, S, load

pytestmark = pytest.mark.gpu


def dev(cuda, a):
    import torch
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(cuda).view(torch.bfloat16)
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


@pytest.mark.parametrize("rows", [1, 3, 6])
@pytest.mark.parametrize("splits", [1, 2])
def test_partial_records_match_the_golden_state(cuda, rows, splits):
    import torch
    import ascend_micro_harness_b200 as tq
    g, scales = load()
    q = np.ascontiguousarray(g["q"][:, :rows, :])
    ws = torch.full((HEADS * splits * 16 * (16 + D),), float("nan"), dtype=torch.float32, device=cuda)
    q_rot = torch.zeros((HEADS * splits, 16, D), dtype=torch.bfloat16, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    tq.decode_splitk_partials(dev(cuda, q), dev(cuda, g["signs"].astype(np.float32)), dev(cuda, g["key"]),
                              dev(cuda, g["value"]), dev(cuda, scales), dev(cuda, g["table"]), q_rot, ws,
                              requests=1, heads=HEADS, rows=rows, head_size=D, block_size=S, cache_pages=P,
                              seq_pages=PAGES, splits=splits, page_begin=0, page_count=PAGES, seq_len=0,
                              inv_sqrt_len=0.0625, softmax_scale=1.0, status=st)
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    rec = ws.cpu().numpy().reshape(HEADS, splits, 16, 16 + D).astype(np.float64)
    rot = q_rot.float().cpu().numpy().reshape(HEADS, splits, 16, D)
    for head in range(HEADS):
        gm, gl, ga = (g[f"{k}_h{head}"][:rows].astype(np.float64) for k in ("m", "l", "acc"))
        assert np.array_equal(rot[head, 0, :rows], g[f"q_rot_h{head}"][:rows])     # bit-exact rotation
        # log-sum-exp merge of the split records in FP64 (one page per split at splits = 2)
        m = rec[head, :, :rows, 0].max(axis=0)
        w = np.exp(rec[head, :, :rows, 0] - m[None, :])
        l = (rec[head, :, :rows, 8] * w).sum(axis=0)
        acc = (rec[head, :, :rows, 16:] * w[:, :, None]).sum(axis=0)
        assert (rec[head, :, :rows, 0:8] == rec[head, :, :rows, 0:1]).all()          # replicated lanes, not torn
        assert (rec[head, :, :rows, 8:16] == rec[head, :, :rows, 8:9]).all()
        assert (np.abs(m - gm) <= 2e-6 * np.maximum(1.0, np.abs(gm))).all()
        assert (np.abs(l - gl) <= 1e-4 * np.maximum(1.0, gl)).all()
        bound = 2e-4 * np.abs(ga).max(axis=1, keepdims=True) + 1e-5 * gl[:, None] + 1e-6
        assert (np.abs(acc - ga) <= bound).all()


@pytest.mark.parametrize("splits", [1, 2, 0])
def test_gated_context_matches_the_golden_model(cuda, splits):
    import torch
    import ascend_micro_harness_b200 as tq
    g, scales = load()
    q = g["q"].reshape(1, HEADS * ROWS, D)
    use = splits if splits else tq.choose_splits(1, HEADS, S, PAGES * S)
    ws = torch.full((tq.decode_workspace_floats(1, HEADS * ROWS, HEADS, D, use),), float("nan"),
                    dtype=torch.float32, device=cuda)
    out = torch.zeros((1, HEADS * ROWS, D), dtype=torch.float32, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    for stage, name in ((1, "rotated"), (2, "context")):
        tq.decode_splitk(dev(cuda, q), dev(cuda, g["key"]), dev(cuda, g["value"]), dev(cuda, scales),
                         dev(cuda, g["table"][None, :].copy()), dev(cuda, np.array([PAGES * S], np.int32)),
                         dev(cuda, g["signs"].astype(np.float32)), out, num_heads=HEADS * ROWS, num_kv_heads=HEADS,
                         head_size=D, block_size=S, num_blocks=P, inv_sqrt_len=0.0625, softmax_scale=1.0,
                         splits=splits, max_context_hint=PAGES * S, workspace=ws,
                         gate=dev(cuda, g["gate"].reshape(1, -1, D)), output_stage=stage, status=st)
        torch.cuda.synchronize()
        assert int(st.item()) == 0
        got = out.cpu().numpy()
        want = np.stack([g[f"{name}_h{h}"] for h in range(HEADS)]).reshape(got.shape)
        # tolerance-grade path: 2e-3 relative / 1e-3 absolute, taken against the row's largest magnitude
        assert (np.abs(got - want) <= 1e-3 + 2e-3 * np.abs(want).max(axis=-1, keepdims=True)).all()
