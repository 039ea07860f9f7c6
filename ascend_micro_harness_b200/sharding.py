"""Sharding of a decode batch over GPUs. Sequences (and KV heads) are independent
units of the path -- the grid axes of the reference decoder
(kernels/ops/turboquant/turboquant_paged_decode_attention.cpp:1598-1603) -- so a batch
shards by sequence with no collective on the data path; only the timing is reduced."""
from __future__ import annotations

from typing import List, Sequence


def partition_sequences(context_lens: Sequence[int], world: int, policy: str = "lpt") -> List[List[int]]:
    """Sequence indices owned by each rank.
    'round_robin' suits uniform lengths; 'lpt' (longest processing time first) balances the
    KV bytes of a ragged batch: sequences in decreasing length, each to the lightest rank;
    'lpt_equal' does the same but no rank takes more than ceil(n / world) sequences, for
    engines whose launch geometry is sized for a fixed batch per GPU."""
    if world <= 0:
        raise ValueError("world must be positive")
    shards: List[List[int]] = [[] for _ in range(world)]
    if policy == "round_robin":
        for i in range(len(context_lens)):
            shards[i % world].append(i)
        return shards
    if policy not in ("lpt", "lpt_equal"):
        raise ValueError(f"unknown policy {policy!r}")
    cap = -(-len(context_lens) // world) if policy == "lpt_equal" else len(context_lens)
    load = [0] * world
    for i in sorted(range(len(context_lens)), key=lambda j: (-int(context_lens[j]), j)):
        r = min((k for k in range(world) if len(shards[k]) < cap), key=lambda k: (load[k], k))
        shards[r].append(i)
        load[r] += int(context_lens[i])
    for s in shards:
        s.sort()
    return shards


def kv_bytes(context_lens: Sequence[int], num_kv_heads: int, head_size: int) -> int:
    """Packed K + packed V + both scale planes: ctx * H_kv * (d + 8) bytes per sequence
    (the reference's accounting, tests/npu/bench/bench_turboquant_decode_splitk.cpp:569)."""
    return int(sum(int(c) * num_kv_heads * (head_size + 8) for c in context_lens))


def aggregate(ms_local: float, bytes_local: int, dist=None, device=None):
    """(max step time over ranks, total bytes over ranks). dist is torch.distributed or None."""
    if dist is None or not dist.is_initialized() or dist.get_world_size() == 1:
        return float(ms_local), int(bytes_local)
    import torch
    t = torch.tensor([ms_local], dtype=torch.float64, device=device)
    b = torch.tensor([float(bytes_local)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.all_reduce(b, op=dist.ReduceOp.SUM)
    return float(t.item()), int(b.item())
