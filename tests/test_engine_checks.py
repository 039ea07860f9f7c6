"""The Python host layer refuses operands the library would misread: tensors that are not on a
GPU, on different GPUs, of an element type the kernel does not assume, or a workspace smaller
than the launch's records. The device-free cases run everywhere; the rest need a GPU."""
import numpy as np
import pytest


def test_cpu_tensors_are_refused_before_the_library_is_called():
    import torch
    import ascend_micro_harness_b200 as tq
    t = torch.zeros(16, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA tensor"):
        tq.rotate_query(t, torch.zeros(128), t.clone(), head_size=128, inv_sqrt_len=0.1)
    with pytest.raises(ValueError, match="CUDA tensor"):
        tq.reshape_and_cache(t, t, t, t, t, t, t, num_kv_heads=1, head_size=128, block_size=16, num_blocks=1,
                             inv_sqrt_len=0.1)


def test_workspace_size_operator_counts_records_and_counters():
    from ascend_micro_harness_b200 import torch_ops
    import ascend_micro_harness_b200 as tq
    for (b, hq, hkv, d, k) in ((64, 32, 8, 128, 9), (3, 64, 4, 256, 2), (1, 8, 8, 128, 16)):
        assert torch_ops._workspace_size(b, hq, hkv, d, k) == tq.decode_workspace_floats(b, hq, hkv, d, k)
    # splits left to the launch: sized for the most it can pick
    assert torch_ops._workspace_size(5, 32, 8, 128, 0) == tq.decode_workspace_floats(5, 32, 8, 128, 32)


@pytest.mark.gpu
def test_wrong_element_types_and_short_workspaces_are_refused(cuda):
    import torch
    import ascend_micro_harness_b200 as tq
    Hq, Hkv, d, S, P, B = 8, 2, 128, 16, 8, 2
    kc = torch.zeros(P * Hkv * S * d // 2, dtype=torch.uint8, device=cuda)
    sc = torch.ones(2 * P * Hkv * S, dtype=torch.float32, device=cuda)
    tables = torch.zeros((B, 4), dtype=torch.int32, device=cuda)
    lens = torch.full((B,), 40, dtype=torch.int32, device=cuda)
    signs = torch.ones(d, device=cuda)
    q = torch.zeros((B, Hq, d), dtype=torch.bfloat16, device=cuda)
    out = torch.zeros((B, Hq, d), dtype=torch.float32, device=cuda)
    geom = dict(num_heads=Hq, num_kv_heads=Hkv, head_size=d, block_size=S, num_blocks=P, inv_sqrt_len=0.088)
    ws = torch.zeros(tq.decode_workspace_floats(B, Hq, Hkv, d, 2), device=cuda)
    with pytest.raises(ValueError, match="block_tables must be int32"):
        tq.decode_splitk(q, kc, kc, sc, tables.long(), lens, signs, out, splits=2, workspace=ws, **geom)
    with pytest.raises(ValueError, match="context_lens must be int32"):
        tq.decode_splitk(q, kc, kc, sc, tables, lens.long(), signs, out, splits=2, workspace=ws, **geom)
    with pytest.raises(ValueError, match="query must be bfloat16"):
        tq.decode_splitk(q.half(), kc, kc, sc, tables, lens, signs, out, splits=2, workspace=ws, **geom)
    with pytest.raises(ValueError, match="workspace holds"):
        tq.decode_splitk(q, kc, kc, sc, tables, lens, signs, out, splits=4, workspace=ws, **geom)
    with pytest.raises(ValueError, match="workspace is required"):
        tq.decode_splitk(q, kc, kc, sc, tables, lens, signs, out, splits=2, workspace=None, **geom)
    with pytest.raises(ValueError, match="slot_mapping must be int32"):
        tq.reshape_scatter(q.view(B, -1)[:, :Hkv * d].contiguous(), q.view(B, -1)[:, :Hkv * d].contiguous(), kc, kc,
                           sc, torch.zeros(B, dtype=torch.int64, device=cuda), signs, None, num_requests=B,
                           num_kv_heads=Hkv, head_size=d, block_size=S, num_blocks=P, inv_sqrt_len=0.088)
    # softmax_scale must be positive and finite: refused by the library on the host
    for bad in (0.0, -1.0, float("nan"), float("inf")):
        with pytest.raises(tq.TqError):
            tq.decode_splitk(q, kc, kc, sc, tables, lens, signs, out, splits=2, workspace=ws, softmax_scale=bad, **geom)
    # a float16 query through the operator layer goes to the one-element-type entry, not the bf16 one
    from ascend_micro_harness_b200 import torch_ops  # noqa: F401
    outh = torch.zeros((B, Hq, d), dtype=torch.float16, device=cuda)
    torch.ops.tq_b200.paged_decode(q.half(), None, kc, kc, sc, tables, lens, signs, ws, Hq, Hkv, S, 2, 0.1, 0, outh)
    torch.cuda.synchronize()
    if torch.cuda.device_count() > 1:
        other = torch.zeros_like(q, device="cuda:1")
        with pytest.raises(ValueError, match="is on cuda:1"):
            tq.decode_splitk(q, kc, kc, sc, tables, lens, signs, other.float(), splits=2, workspace=ws, **geom)


@pytest.mark.gpu
def test_negative_table_entry_inside_the_live_range_is_reported(cuda):
    """A negative block-table entry under live tokens sets TQ_STATUS_BAD_PAGE (page 0 is read
    instead); the launch completes and the context stays usable."""
    import torch
    import ascend_micro_harness_b200 as tq
    Hq, Hkv, d, S, P = 8, 2, 128, 16, 8
    kc = torch.zeros(P * Hkv * S * d // 2, dtype=torch.uint8, device=cuda)
    sc = torch.ones(2 * P * Hkv * S, dtype=torch.float32, device=cuda)
    tables = torch.tensor([[1, -3, 2, 0]], dtype=torch.int32, device=cuda)
    lens = torch.tensor([60], dtype=torch.int32, device=cuda)
    q = torch.ones((1, Hq, d), dtype=torch.bfloat16, device=cuda)
    out = torch.zeros((1, Hq, d), dtype=torch.float32, device=cuda)
    st = torch.zeros(1, dtype=torch.int32, device=cuda)
    for splits in (1, 2):
        st.zero_()
        ws = torch.zeros(tq.decode_workspace_floats(1, Hq, Hkv, d, splits), device=cuda)
        tq.decode_splitk(q, kc, kc, sc, tables, lens, torch.ones(d, device=cuda), out, num_heads=Hq, num_kv_heads=Hkv,
                         head_size=d, block_size=S, num_blocks=P, inv_sqrt_len=0.088, splits=splits, workspace=ws,
                         status=st)
        torch.cuda.synchronize()
        assert int(st.item()) & tq.STATUS_BAD_PAGE
        assert torch.isfinite(out).all()
