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


class PeerHeadGather:
    """KV-head-sharded decode without a collective: every rank's decode kernel stores its output rows straight into
    the ``[B, Hq, 1, D]`` output tensors of all ranks (peer stores over NVLink from the kernel's merge epilogue), then
    one warp per rank publishes an arrival flag to the peers and waits, with a time limit, for theirs.

    The tensors live in memory that all ranks of the group map (``torch.distributed._symmetric_memory``): two output
    tensors, used in turn, so that a rank that is one step ahead writes where no peer still reads, and one array of
    arrival flags.  Use::

        gather = PeerHeadGather(shard, batch=B, q_heads=Hq, head_dim=D, dtype=torch.bfloat16, device=device)
        local_out, peers = gather.begin()                      # this rank's head slice of the step's tensor
        cache.turboquant_single_token_decode_attention(0, q_local, ..., output=local_out, peer_outputs=peers)
        full = gather.finish()                                 # [B, Hq, 1, D], valid on the current stream

    ``check()`` synchronises and raises if a wait ran out.  The reference is single-device: no counterpart."""

    FLAG_BYTES = 256

    def __init__(self, shard: KvHeadShard, *, batch: int, q_heads: int, head_dim: int, dtype: torch.dtype,
                 device: torch.device, group=None, timeout_ms: int = 2000) -> None:
        import os

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib

        if device.type != "cuda":
            raise RuntimeError("PeerHeadGather needs CUDA devices with peer access; use HeadGather on other backends")
        # plain peer loads / stores only: nothing here needs an NVLink multicast binding of the buffer
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self._lib = _lib
        self.shard = shard
        self.group = dist.group.WORLD if group is None else group
        self.world_size = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world_size != shard.world_size or self.rank != shard.rank:
            raise ValueError("the shard does not describe this rank of the group")
        if self.world_size > 8:
            raise ValueError("PeerHeadGather serves the GPUs of one box (at most 8 ranks)")
        self.shape = (batch, q_heads, 1, head_dim)
        self.dtype = dtype
        self.device = device
        self.timeout_ms = int(timeout_ms)
        elems = batch * q_heads * head_dim
        self._out_bytes = (elems * torch.empty((), dtype=dtype).element_size() + 255) // 256 * 256
        self._buffer = symm_mem.empty(self.FLAG_BYTES + 2 * self._out_bytes, dtype=torch.uint8, device=device)
        self._buffer.zero_()
        self._handle = symm_mem.rendezvous(self._buffer, self.group)
        self._bases = [int(p) for p in self._handle.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(self.group)  # every rank's flags are zero before anybody publishes a step
        self._status = torch.zeros(1, dtype=torch.int32, device=device)
        self._step = 0
        self._head_offset = shard.q_start * head_dim * torch.empty((), dtype=dtype).element_size()

    def _tensor(self, parity: int) -> torch.Tensor:
        start = self.FLAG_BYTES + parity * self._out_bytes
        count = self.shape[0] * self.shape[1] * self.shape[3]
        flat = self._buffer[start:start + self._out_bytes].view(self.dtype)[:count]
        return flat.view(self.shape)

    def begin(self) -> tuple[torch.Tensor, tuple[int, ...]]:
        """This rank's ``[B, Hq / N, 1, D]`` slice of the next step's output tensor and the addresses of the same slice
        in the other ranks' tensors."""
        parity = (self._step + 1) & 1
        local = self._tensor(parity)[:, self.shard.q_start:self.shard.q_stop]
        offset = self.FLAG_BYTES + parity * self._out_bytes + self._head_offset
        peers = tuple(base + offset for r, base in enumerate(self._bases) if r != self.rank)
        return local, peers

    def finish(self) -> torch.Tensor:
        """Publishes this rank's arrival for the step begun last and waits (on the device, bounded) for the peers;
        returns the full ``[B, Hq, 1, D]`` tensor of the step."""
        import ctypes

        from .fused_ops import on_device, ptr, stream_ptr

        self._step += 1
        flags = (ctypes.c_void_p * self.world_size)(*self._bases)
        with on_device(self.device):
            self._lib.check(self._lib.lib().anna_peer_signal_wait(
                flags, self.rank, self.world_size, self._step, self.timeout_ms, ptr(self._status),
                stream_ptr(self.device)), "anna_peer_signal_wait")
        return self._tensor(self._step & 1)

    def check(self) -> None:
        status = int(self._status.item())
        if status != 0:
            raise RuntimeError(f"a peer did not arrive within {self.timeout_ms} ms (device status {status})")
