"""torch.library registration of the engine's operators under the `tq_b200` namespace.

The schemas follow the operator list the reference project drafts for its serving
integration (reports/qwen35_turboquant_rfc.md:253-340): an aligned writer, a sub-strip
scatter writer, a batched query rotation, a GQA paged decode, a cross-split combine and a
workspace-size query. Differences from that draft, all because of how this engine is built:
  * the rotation needs only the sign diagonal, so there is no `tables` operand;
  * `paged_decode` takes the raw query and rotates it in the kernel (the stand-alone
    `rotate_q_batch` exists for callers that want the rotated operand);
  * the egress offsets / signs operands are the same sign diagonal and are not repeated.
Every mutating op has a Meta registration that does nothing, so FakeTensor tracing and
torch.export see the ops without a GPU. Importing this module does not load the CUDA library;
calling an op on CUDA tensors does.
"""
from __future__ import annotations

import torch

from . import engine

NAMESPACE = "tq_b200"
_lib = torch.library.Library(NAMESPACE, "DEF")

_lib.define("reshape_aligned(Tensor key, Tensor value, Tensor(a!) key_cache, Tensor(b!) value_cache, "
            "Tensor(c!) scale_cache, Tensor slot_mapping, Tensor pi_signs, int num_kv_heads, int head_size, "
            "int block_size, int[]? cu_seqlens=None) -> ()")
_lib.define("reshape_scatter(Tensor key, Tensor value, Tensor(a!) key_cache, Tensor(b!) value_cache, "
            "Tensor(c!) scale_cache, Tensor slot_mapping, Tensor pi_signs, int num_kv_heads, int head_size, "
            "int block_size, Tensor? cu_seqlens=None) -> ()")
_lib.define("rotate_q_batch(Tensor query, Tensor pi_signs, Tensor(a!) query_rot, int head_size) -> ()")
_lib.define("paged_decode(Tensor query, Tensor? gate, Tensor key_cache, Tensor value_cache, Tensor scale_cache, "
            "Tensor block_tables, Tensor seq_lens, Tensor pi_signs, Tensor(a!) workspace, int num_heads, "
            "int num_kv_heads, int block_size, int temporal_splits, float scale_value, int output_stage, "
            "Tensor(b!) out) -> ()")
_lib.define("decode_combine(Tensor workspace, Tensor? gate, Tensor pi_signs, int num_heads, int num_kv_heads, "
            "int temporal_splits, int output_stage, Tensor(a!) out) -> ()")
_lib.define("decode_workspace_size(int num_reqs, int num_heads, int num_kv_heads, int head_size, "
            "int temporal_splits) -> int")


def _inv_sqrt(head_size: int) -> float:
    import numpy as np
    return float(np.float32(1.0) / np.sqrt(np.float32(head_size)))


def _num_blocks(cache: torch.Tensor, num_kv_heads: int, head_size: int, block_size: int) -> int:
    return cache.numel() // (num_kv_heads * block_size * head_size // 2)


def _reshape_aligned(key, value, key_cache, value_cache, scale_cache, slot_mapping, pi_signs, num_kv_heads,
                     head_size, block_size, cu_seqlens=None):
    geom = dict(num_kv_heads=num_kv_heads, head_size=head_size, block_size=block_size,
                num_blocks=_num_blocks(key_cache, num_kv_heads, head_size, block_size),
                inv_sqrt_len=_inv_sqrt(head_size))
    if cu_seqlens is None:
        engine.reshape_and_cache(key, value, key_cache, value_cache, scale_cache, slot_mapping, pi_signs, **geom)
    else:
        engine.reshape_and_cache_varlen(key, value, key_cache, value_cache, scale_cache, slot_mapping,
                                        pi_signs, cu_seqlens, **geom)


def _reshape_scatter(key, value, key_cache, value_cache, scale_cache, slot_mapping, pi_signs, num_kv_heads,
                     head_size, block_size, cu_seqlens=None):
    requests = key.numel() // (num_kv_heads * head_size) if cu_seqlens is None else cu_seqlens.numel() - 1
    engine.reshape_scatter(key, value, key_cache, value_cache, scale_cache, slot_mapping, pi_signs, cu_seqlens,
                           num_requests=requests, num_kv_heads=num_kv_heads, head_size=head_size,
                           block_size=block_size,
                           num_blocks=_num_blocks(key_cache, num_kv_heads, head_size, block_size),
                           inv_sqrt_len=_inv_sqrt(head_size))


def _rotate_q_batch(query, pi_signs, query_rot, head_size):
    engine.rotate_query(query, pi_signs, query_rot, head_size=head_size, inv_sqrt_len=_inv_sqrt(head_size))


def _paged_decode(query, gate, key_cache, value_cache, scale_cache, block_tables, seq_lens, pi_signs, workspace,
                  num_heads, num_kv_heads, block_size, temporal_splits, scale_value, output_stage, out):
    head_size = query.shape[-1]
    kwargs = dict(num_heads=num_heads, num_kv_heads=num_kv_heads, head_size=head_size, block_size=block_size,
                  num_blocks=_num_blocks(key_cache, num_kv_heads, head_size, block_size),
                  inv_sqrt_len=_inv_sqrt(head_size), softmax_scale=scale_value, splits=temporal_splits,
                  workspace=workspace, gate=gate, output_stage=output_stage)
    # route by the query's element type: float16 queries, and bfloat16 queries whose gate shares
    # the element type, take the one-element-type entry; bfloat16 with an FP32 gate (or none)
    # the plain one
    if query.dtype == torch.float16 or (gate is not None and gate.dtype != torch.float32):
        engine.decode_splitk_elem(query, key_cache, value_cache, scale_cache, block_tables, seq_lens, pi_signs,
                                  out, **kwargs)
    else:
        engine.decode_splitk(query, key_cache, value_cache, scale_cache, block_tables, seq_lens, pi_signs, out,
                             **kwargs)


def _decode_combine(workspace, gate, pi_signs, num_heads, num_kv_heads, temporal_splits, output_stage, out):
    head_size = out.shape[-1]
    rows = num_heads // num_kv_heads
    items = out.numel() // (rows * head_size)
    engine.splitk_combine(workspace, pi_signs, gate, out, items=items, rows=rows, rows_stride=rows,
                          head_size=head_size, splits=temporal_splits, output_stage=output_stage,
                          inv_sqrt_len=_inv_sqrt(head_size))


def _workspace_size(num_reqs, num_heads, num_kv_heads, head_size, temporal_splits):
    """Floats of workspace (tq_decode_workspace_floats): the records of every split, one arrival
    counter per (request, KV head, 8-row tile) and, 8-byte aligned behind them, two 64-bit
    schedule words. temporal_splits 0 leaves the choice to the launch, which never takes more
    than 32 splits: sized for that."""
    rows = num_heads // num_kv_heads
    splits = temporal_splits if temporal_splits else 32
    words = (num_reqs * num_kv_heads * splits * rows * (16 + head_size)
             + num_reqs * num_kv_heads * ((rows + 7) // 8))
    return (words + 1) // 2 * 2 + 4


for _name, _fn in (("reshape_aligned", _reshape_aligned), ("reshape_scatter", _reshape_scatter),
                   ("rotate_q_batch", _rotate_q_batch), ("paged_decode", _paged_decode),
                   ("decode_combine", _decode_combine)):
    _lib.impl(_name, _fn, "CUDA")
    _lib.impl(_name, lambda *a, **k: None, "Meta")
_lib.impl("decode_workspace_size", _workspace_size, "CompositeExplicitAutograd")
