"""CPU, world size 2 over gloo: the sequence-sharding rule and the max-over-ranks timing reduction of the harness."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from anna_b200.sharding import (HeadGather, aggregate_throughput, balance_by_tokens, shard_kv_heads,
                                shard_sequences)


def _free_port() -> int:
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _worker(rank: int, world: int, port: int, total: int):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shard = shard_sequences(total, world, rank)
        owned = torch.zeros(total, dtype=torch.int64)
        owned[shard.start:shard.stop] = 1
        dist.all_reduce(owned)  # every sequence is owned exactly once
        assert owned.tolist() == [1] * total
        # the harness reports max over ranks of the step time and the sum of the units
        elapsed = torch.tensor([0.5 + rank], dtype=torch.float64)
        units = torch.tensor([shard.count], dtype=torch.int64)
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        dist.all_reduce(units)
        assert elapsed.item() == 0.5 + (world - 1) and units.item() == total
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_sequence_shards_cover_every_sequence_once_world2():
    mp.spawn(_worker, args=(2, _free_port(), 513), nprocs=2, join=True)


def test_shard_rule_and_balancing():
    shards = [shard_sequences(512, 8, r) for r in range(8)]
    assert [s.count for s in shards] == [64] * 8 and shards[0].start == 0 and shards[-1].stop == 512
    shards = [shard_sequences(10, 4, r) for r in range(4)]
    assert [(s.start, s.stop) for s in shards] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert shard_sequences(0, 2, 1).count == 0 and shards[1].owns(4) and not shards[1].owns(6)
    with pytest.raises(ValueError):
        shard_sequences(4, 2, 2)
    lengths = [8192, 1024, 4096, 4096, 2048, 6144, 1024, 2048]
    owners = balance_by_tokens(lengths, 2)
    assert sorted(owners[0] + owners[1]) == list(range(8))
    loads = [sum(lengths[i] for i in bucket) for bucket in owners]
    assert max(loads) - min(loads) <= 1024
    assert aggregate_throughput([64, 64], [0.5, 1.0]) == 128.0


def _head_worker(rank: int, world: int, port: int):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        batch, q_heads, kv_heads, dim = 3, 8, 4, 16
        shard = shard_kv_heads(q_heads, kv_heads, world, rank)
        full = torch.arange(batch * q_heads * dim, dtype=torch.float32).view(batch, q_heads, 1, dim)
        kv = torch.arange(batch * kv_heads * 5 * dim, dtype=torch.float32).view(batch, kv_heads, 5, dim)
        assert shard.slice_kv(kv).shape[1] == kv_heads // world and shard.slice_q(full).shape[1] == q_heads // world
        gather = HeadGather()
        for _ in range(2):  # the second call reuses the buffers
            out = gather(shard.slice_q(full))
            assert out.shape == full.shape and torch.equal(out, full)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_kv_head_shards_and_output_gather_world2():
    mp.spawn(_head_worker, args=(2, _free_port()), nprocs=2, join=True)


def test_kv_head_shard_rule():
    shards = [shard_kv_heads(32, 8, 8, r) for r in range(8)]
    assert [(s.kv_start, s.kv_stop, s.q_start, s.q_stop) for s in shards][:2] == [(0, 1, 0, 4), (1, 2, 4, 8)]
    assert shards[-1].q_stop == 32
    with pytest.raises(ValueError):
        shard_kv_heads(32, 8, 3, 0)
    with pytest.raises(ValueError):
        shard_kv_heads(30, 8, 2, 0)
