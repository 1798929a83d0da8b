"""Multi-GPU layouts of the decode path.

Default: sequences are independent, so they are sharded across ranks.  Every rank owns a disjoint set of sequences
together with their pages, block tables and window rings; no collective touches KV data.  The only cross-rank traffic
is bookkeeping (a barrier and a max over step times).

Second layout: KV heads are sharded.  Every rank holds all sequences but only its own KV heads (and the query heads of
their groups); block tables are replicated, the pools shrink by the world size, and after the decode one all-gather
of ``[B, Hq / N, D]`` outputs rebuilds ``[B, Hq, D]`` on every rank.

The reference is single-device (there is no torch.distributed use anywhere in it), so this file has no reference
counterpart; it states the partition rules the harness and the tests share.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


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


@dataclass(frozen=True)
class KvHeadShard:
    """KV heads [kv_start, kv_stop) and the query heads [q_start, q_stop) of their groups."""
    rank: int
    world_size: int
    kv_start: int
    kv_stop: int
    q_start: int
    q_stop: int

    def slice_kv(self, states: torch.Tensor) -> torch.Tensor:
        """``[B, Hkv, T, D]`` -> this rank's ``[B, Hkv / N, T, D]`` (a view)."""
        return states[:, self.kv_start:self.kv_stop]

    def slice_q(self, states: torch.Tensor) -> torch.Tensor:
        """``[B, Hq, 1, D]`` -> this rank's ``[B, Hq / N, 1, D]`` (a view)."""
        return states[:, self.q_start:self.q_stop]


def shard_kv_heads(num_q_heads: int, num_kv_heads: int, world_size: int, rank: int) -> KvHeadShard:
    """Equal contiguous blocks of KV heads; the world size has to divide the number of KV heads."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if num_kv_heads <= 0 or num_q_heads % num_kv_heads != 0:
        raise ValueError("query heads must be a positive multiple of kv heads")
    if num_kv_heads % world_size != 0:
        raise ValueError(f"{num_kv_heads} kv heads cannot be split evenly over {world_size} ranks")
    per_rank = num_kv_heads // world_size
    groups = num_q_heads // num_kv_heads
    kv_start = rank * per_rank
    return KvHeadShard(rank=rank, world_size=world_size, kv_start=kv_start, kv_stop=kv_start + per_rank,
                       q_start=kv_start * groups, q_stop=(kv_start + per_rank) * groups)


class HeadGather:
    """All-gather of per-rank decode outputs ``[B, Hq / N, 1, D]`` into ``[B, Hq, 1, D]`` on every rank.

    One collective per call on the process group's backend (NCCL on GPUs: the ranks' blocks land in one staging
    buffer ``[N, B, Hq / N, D]``, which a single strided copy turns into head-major order).  Buffers are kept
    between calls, so a decode loop allocates nothing."""

    def __init__(self, group=None) -> None:
        import torch.distributed as dist

        self._dist = dist
        self.group = group
        self.world_size = dist.get_world_size(group)
        self._staging: torch.Tensor | None = None
        self._full: torch.Tensor | None = None

    def __call__(self, local: torch.Tensor) -> torch.Tensor:
        if local.dim() != 4 or local.shape[2] != 1:
            raise ValueError("HeadGather expects [batch, local_heads, 1, head_dim]")
        batch, heads, _, dim = (int(v) for v in local.shape)
        world = self.world_size
        if world == 1:
            return local
        local = local.contiguous()
        shape = (world, batch, heads, dim)
        if (self._staging is None or tuple(self._staging.shape) != shape or self._staging.dtype != local.dtype
                or self._staging.device != local.device):
            self._staging = torch.empty(shape, dtype=local.dtype, device=local.device)
            self._full = torch.empty((batch, world * heads, 1, dim), dtype=local.dtype, device=local.device)
        self._dist.all_gather_into_tensor(self._staging.view(world * batch, heads, dim),
                                          local.view(batch, heads, dim), group=self.group)
        assert self._full is not None
        self._full.view(batch, world, heads, dim).copy_(self._staging.permute(1, 0, 2, 3))
        return self._full
