"""The multi-GPU path is 'shard the sequences, reduce only the timing'; its host logic is
exercised here with world_size-2 gloo ranks on CPU."""
import os
import socket

import numpy as np
import pytest


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ctx, out):
    import torch.distributed as dist
    from ascend_micro_harness_b200.sharding import aggregate, kv_bytes, partition_sequences
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    mine = partition_sequences(ctx, world)[rank]
    local_bytes = kv_bytes([ctx[i] for i in mine], 8, 128)
    ms, total = aggregate(10.0 + rank, local_bytes, dist)   # rank 1 is the slow one
    out[rank] = (ms, total, mine)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_sharding_and_timing_reduce():
    import torch.multiprocessing as mp
    rng = np.random.default_rng(4)
    ctx = [int(c) for c in rng.integers(512, 32769, 64)]
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(2, _free_port(), ctx, out), nprocs=2, join=True)
        r0, r1 = out[0], out[1]
    from ascend_micro_harness_b200.sharding import kv_bytes
    assert r0[0] == r1[0] == 11.0                                   # max over ranks
    assert r0[1] == r1[1] == kv_bytes(ctx, 8, 128)                  # bytes add up
    assert sorted(r0[2] + r1[2]) == list(range(64))                 # every sequence once


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_lpt_balances_a_ragged_batch(world):
    from ascend_micro_harness_b200.sharding import partition_sequences
    rng = np.random.default_rng(world)
    ctx = [int(c) for c in rng.integers(512, 32769, 64)]
    shards = partition_sequences(ctx, world)
    assert sorted(i for s in shards for i in s) == list(range(64))
    loads = [sum(ctx[i] for i in s) for s in shards]
    assert max(loads) - min(loads) <= max(ctx)                      # LPT bound
    rr = partition_sequences(ctx, world, "round_robin")
    assert all(len(s) in (64 // world, 64 // world + (64 % world > 0)) for s in rr)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_equal_count_lpt_keeps_the_batch_per_rank(world):
    """The benchmark's dealing of 64 sequences per GPU: equal counts, loads within a few percent."""
    from ascend_micro_harness_b200.sharding import partition_sequences
    rng = np.random.default_rng(100 + world)
    ctx = [int(c) for c in rng.integers(512, 32769, 64 * world)]
    shards = partition_sequences(ctx, world, "lpt_equal")
    assert sorted(i for s in shards for i in s) == list(range(64 * world))
    assert all(len(s) == 64 for s in shards)
    loads = [sum(ctx[i] for i in s) for s in shards]
    assert max(loads) <= 1.02 * (sum(loads) / world)
