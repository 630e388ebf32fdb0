"""Replica sharding and the cross-rank reduction of timings (gloo, two CPU ranks)."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from white_matter_b200.replicas import aggregate_throughput, shard_batch_heads, shard_range


def test_shard_range_covers_everything_once():
    for total in (1, 7, 16, 64):
        for world in (1, 2, 3, 8):
            pieces = [shard_range(total, r, world) for r in range(world)]
            assert pieces[0][0] == 0 and pieces[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))
            sizes = [e - b for b, e in pieces]
            assert max(sizes) - min(sizes) <= 1


def test_batch_first_then_heads():
    assert shard_batch_heads(16, 16, 3, 8) == (slice(6, 8), slice(0, 16))
    assert shard_batch_heads(2, 16, 3, 4) == (slice(1, 2), slice(8, 16))
    with pytest.raises(ValueError):
        shard_batch_heads(2, 16, 0, 3)


def test_grouped_heads_are_cut_between_kv_heads():
    # 8 query heads over 2 KV heads, 2 rows on 4 ranks: a rank gets one row, one KV head and its 4 query heads
    assert shard_batch_heads(2, 8, 3, 4, kv_heads=2) == (slice(1, 2), slice(4, 8), slice(1, 2))
    assert shard_batch_heads(4, 8, 1, 2, kv_heads=2) == (slice(2, 4), slice(0, 8), slice(0, 2))
    with pytest.raises(ValueError):
        shard_batch_heads(1, 8, 0, 4, kv_heads=2)  # four ranks cannot share two KV heads


def _worker(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # each rank owns its shard of a (batch, heads) problem and reports its own time and work
        rows, heads = shard_batch_heads(6, 4, rank, world)
        units = float((rows.stop - rows.start) * (heads.stop - heads.start))
        ms, total = aggregate_throughput(10.0 + 5.0 * rank, units)
        results[rank] = (ms, total)
    finally:
        dist.destroy_process_group()


def test_aggregate_is_max_time_and_summed_work_over_two_ranks():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, 29611, results), nprocs=world, join=True)
    assert results[0] == results[1] == (15.0, 24.0)


def test_aggregate_without_process_group_is_identity():
    assert aggregate_throughput(3.0, 5.0) == (3.0, 5.0)
