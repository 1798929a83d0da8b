"""Multi-GPU layout of the decode path: sequences are independent, so they are sharded across ranks.

Every rank owns a disjoint set of sequences together with their pages, block tables and window rings; no
collective touches KV data.  The only cross-rank traffic is bookkeeping (a barrier and a max over step times).
The reference is single-device (there is no torch.distributed use anywhere in it), so this file has no reference
counterpart; it states the partition rule the harness and the tests share.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class SequenceShard:
    rank: int
    world_size: int
    start: int
    stop: int

    @property
    def count(self) -> int:
        return self.stop - self.start

    def owns(self, sequence: int) -> bool:
        return self.start <= sequence < self.stop


def shard_sequences(num_sequences: int, world_size: int, rank: int) -> SequenceShard:
    """Contiguous, balanced partition: the first ``num_sequences % world_size`` ranks get one extra sequence."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if num_sequences < 0:
        raise ValueError("num_sequences must be non-negative")
    base, extra = divmod(num_sequences, world_size)
    start = rank * base + min(rank, extra)
    stop = start + base + (1 if rank < extra else 0)
    return SequenceShard(rank=rank, world_size=world_size, start=start, stop=stop)


def balance_by_tokens(lengths: list[int], world_size: int) -> list[list[int]]:
    """Greedy longest-first assignment of ragged sequences to ranks so that token counts (= KV bytes) even out."""
    order = sorted(range(len(lengths)), key=lambda i: (-lengths[i], i))
    loads = [0] * world_size
    owners: list[list[int]] = [[] for _ in range(world_size)]
    for index in order:
        rank = min(range(world_size), key=lambda r: (loads[r], r))
        owners[rank].append(index)
        loads[rank] += lengths[index]
    for bucket in owners:
        bucket.sort()
    return owners


def aggregate_throughput(units_per_rank: list[int], seconds_per_rank: list[float]) -> float:
    """Whole-job throughput: every rank's units over the slowest rank's time."""
    slowest = max(seconds_per_rank)
    return sum(units_per_rank) / slowest if slowest > 0 else 0.0
