"""TurboQuant KV rows on the GPU: the per-sequence handle and the batched launches behind it.

Mirrors the public surface of ``TurboQuantKVRow`` (``src/anna/model/turboquant.py:480-1443``): ``append``,
``decode_attention``, ``materialize``, ``clone``, ``length`` / ``quantized_length`` / ``residual_length``.  A row here
owns no tensors of its own; it is a handle on a window ring slot and a block table inside the layer's
``TurboQuantLayerPool``, so moving rows between batches (stack / split / compact) never copies KV bytes, and a
whole batch of rows is appended or decoded by one launch.
"""
from __future__ import annotations

import torch

from . import _lib
from .fused_ops import MetadataUploader, dtype_code, on_device, ptr, query_scratch, split_scratch, stream_ptr
from .pools import TurboQuantLayerPool, resolve_value_group_size
from .tq_tables import key_tables

# KV-cache TurboQuant bit-widths allowed by Anna runtimes (turboquant.py:52).
VALID_KV_CACHE_QUANT_BITS: frozenset[int] = frozenset((2, 3, 4))


def turboquant_is_available() -> bool:
    """True when the CUDA library that implements the quantizer can be loaded (turboquant.py:43-48)."""
    try:
        _lib.lib()
    except RuntimeError:
        return False
    return True


def _i32(values, device: torch.device) -> torch.Tensor:
    return torch.tensor(values, dtype=torch.int32, device=device)


def _i64(values, device: torch.device) -> torch.Tensor:
    return torch.tensor(values, dtype=torch.int64, device=device)


def _require_cuda(tensor: torch.Tensor, what: str) -> None:
    if tensor.device.type != "cuda":
        raise RuntimeError(f"{what}: tensors must live on a CUDA device; there is no CPU fallback for this path.")


def launch_tq_append(pool: TurboQuantLayerPool, key_states: torch.Tensor, value_states: torch.Tensor,
                     table_dev: torch.Tensor | None, slots: list[int], past: list[int], *,
                     slots_dev: torch.Tensor | None = None, past_dev: torch.Tensor | None = None,
                     new_lengths_dev: torch.Tensor | None = None) -> None:
    """Append ``[B, Hkv, T, D]`` to B rows of one layer: ring update + quantize-on-overflow + page scatter.

    ``slots_dev`` / ``past_dev`` (optional, int64 ``[B]`` on the device) are copies of ``slots`` / ``past`` that the
    caller already holds there; ``new_lengths_dev`` (optional) receives ``past + T`` from the kernel."""
    _require_cuda(key_states, "TurboQuant append")
    key_states = key_states if key_states.stride(3) == 1 else key_states.contiguous()
    if value_states.stride() != key_states.stride():
        key_states, value_states = key_states.contiguous(), value_states.contiguous()
    device = key_states.device
    batch, kv_heads, tokens, dim = (int(v) for v in key_states.shape)
    tables = key_tables(head_dim=dim, bits=pool.bits, device=device)
    if slots_dev is None or past_dev is None:
        meta = MetadataUploader.for_device(device).upload([past, slots])
        past_dev = meta[0] if past_dev is None else past_dev
        slots_dev = meta[1] if slots_dev is None else slots_dev
    assert pool.window is not None
    table_stride = 0 if table_dev is None else table_dev.stride(0)
    max_blocks = 0 if table_dev is None else int(table_dev.shape[1])
    with on_device(device):
        _lib.check(_lib.lib().anna_tq_append(
            ptr(key_states), ptr(value_states), key_states.stride(0), key_states.stride(1), key_states.stride(2),
            ptr(pool.packed_pages), ptr(table_dev), table_stride, ptr(pool.window), ptr(slots_dev), ptr(past_dev),
            ptr(new_lengths_dev), ptr(tables.signs1), ptr(tables.signs2), ptr(tables.centroids), ptr(tables.boundaries), batch, kv_heads,
            tokens, dim, pool.block_size, pool.residual_len, pool.bits, pool.value_group, pool.capacity(), max_blocks,
            dtype_code(key_states.dtype), ptr(pool.status), stream_ptr(device)), "anna_tq_append")


def launch_tq_decode(pool: TurboQuantLayerPool, query_states: torch.Tensor, table_dev: torch.Tensor | None,
                     slots: list[int], lengths: list[int], scaling: float, gate: torch.Tensor | None, *,
                     slots_dev: torch.Tensor | None = None, lengths_dev: torch.Tensor | None = None) -> torch.Tensor:
    """Decode ``[B, Hq, 1, D]`` queries against B rows of one layer (packed prefix + window ring).

    ``slots_dev`` / ``lengths_dev`` (optional, int64 ``[B]`` on the device) are copies of ``slots`` / ``lengths``
    that the caller already holds there."""
    _require_cuda(query_states, "TurboQuant decode")
    query = query_states if query_states.stride(3) == 1 else query_states.contiguous()
    if gate is not None and gate.stride(3) != 1:
        gate = gate.contiguous()
    device = query.device
    batch, heads, _, dim = (int(v) for v in query.shape)
    if query.dtype != pool.dtype:
        raise RuntimeError(f"query dtype {query.dtype} must match the cache dtype {pool.dtype}")
    tables = key_tables(head_dim=dim, bits=pool.bits, device=device)
    if slots_dev is None or lengths_dev is None:
        meta = MetadataUploader.for_device(device).upload([lengths, slots])
        lengths_dev = meta[0] if lengths_dev is None else lengths_dev
        slots_dev = meta[1] if slots_dev is None else slots_dev
    out = torch.empty((batch, heads, 1, dim), dtype=query.dtype, device=device)
    table_stride = 0 if table_dev is None else table_dev.stride(0)
    max_blocks = 0 if table_dev is None else int(table_dev.shape[1])
    max_len = max_blocks * pool.block_size + pool.residual_len
    stats, values, capacity, counters = split_scratch(device, batch, heads, dim, pool.kv_heads, max_len,
                                                      turboquant=(max_blocks, pool.block_size, pool.residual_len))
    frags = query_scratch(device, batch, heads, pool.kv_heads, dim)
    with on_device(device):
        _lib.check(_lib.lib().anna_tq_paged_decode(
            ptr(query), query.stride(0), query.stride(1), ptr(pool.packed_pages), ptr(table_dev), table_stride,
            ptr(pool.window), ptr(slots_dev), ptr(lengths_dev), ptr(tables.signs1), ptr(tables.signs2),
            ptr(tables.centroids), ptr(gate), 0 if gate is None else gate.stride(0),
            0 if gate is None else gate.stride(1), ptr(out), out.stride(0), out.stride(1), ptr(stats), ptr(values),
            capacity, 0, ptr(counters), ptr(frags), frags.numel(), batch, heads, pool.kv_heads, dim, pool.block_size,
            pool.residual_len, pool.bits,
            pool.value_group, pool.capacity(), max_blocks, float(scaling), dtype_code(query.dtype),
            stream_ptr(device)), "anna_tq_paged_decode")
    return out


def launch_tq_materialize(pool: TurboQuantLayerPool, table_dev: torch.Tensor, quantized_lengths: list[int],
                          key_out: torch.Tensor, value_out: torch.Tensor) -> None:
    """De-quantize the packed prefix of B rows into dense ``[B, Hkv, Lq_max, D]`` tensors (strided views allowed)."""
    _require_cuda(key_out, "TurboQuant materialize")
    device = key_out.device
    if key_out.stride() != value_out.stride() or key_out.stride(3) != 1:
        raise ValueError("materialize outputs must share strides and be contiguous in the last dimension")
    batch, kv_heads, max_lq, dim = (int(v) for v in key_out.shape)
    tables = key_tables(head_dim=dim, bits=pool.bits, device=device)
    lq_dev = _i64(quantized_lengths, device)
    with on_device(device):
        _lib.check(_lib.lib().anna_tq_materialize(
            ptr(pool.packed_pages), ptr(table_dev), table_dev.stride(0), ptr(lq_dev), ptr(tables.signs1),
            ptr(tables.signs2), ptr(tables.centroids), ptr(key_out), ptr(value_out), key_out.stride(0),
            key_out.stride(1), key_out.stride(2), batch, kv_heads, dim, pool.block_size, pool.bits, pool.value_group,
            pool.capacity(), int(table_dev.shape[1]), max_lq, dtype_code(key_out.dtype), stream_ptr(device)),
            "anna_tq_materialize")


class TurboQuantKVRow:
    """One sequence of one TurboQuant layer: newest ``residual_len`` tokens in a ring, older tokens packed in pages."""

    def __init__(self, *, bits: int, residual_len: int, value_group_size: int | None = None) -> None:
        self.bits = int(bits)
        self.residual_len = max(1, int(residual_len))
        self.value_group_size = None if value_group_size is None else max(1, int(value_group_size))
        self.device: torch.device | None = None
        self.dtype: torch.dtype | None = None
        self.head_dim: int | None = None
        self.num_heads: int | None = None
        self.pool: TurboQuantLayerPool | None = None
        self.slot = -1
        self.block_table: list[int] = []
        self._length = 0

    # -- state ----------------------------------------------------------------------------------------------------------

    @property
    def initialized(self) -> bool:
        return self.pool is not None and self.slot >= 0

    @property
    def length(self) -> int:
        return self._length

    @property
    def quantized_length(self) -> int:
        return max(0, self._length - self.residual_len)

    @property
    def residual_length(self) -> int:
        return min(self._length, self.residual_len)

    def _bind(self, pool: TurboQuantLayerPool, *, kv_heads: int, head_dim: int, dtype: torch.dtype,
              device: torch.device) -> None:
        pool.configure(kv_heads=kv_heads, head_dim=head_dim, bits=self.bits, residual_len=self.residual_len,
                       dtype=dtype, device=device, value_group=self.value_group_size)
        self.pool = pool
        self.device, self.dtype = device, dtype
        self.head_dim, self.num_heads = int(head_dim), int(kv_heads)
        self.value_group_size = pool.value_group
        self.slot = pool.allocate_slot()

    def _reserve_blocks(self, new_length: int) -> None:
        """Take pages for every block the quantized prefix will reach once the row holds new_length tokens."""
        assert self.pool is not None
        quantized = max(0, int(new_length) - self.residual_len)
        need = (quantized + self.pool.block_size - 1) // self.pool.block_size
        if need > len(self.block_table):
            self.block_table.extend(self.pool.allocate(need - len(self.block_table)))

    def _table_on_device(self) -> torch.Tensor | None:
        if not self.block_table:
            return None
        assert self.device is not None
        return _i32([self.block_table], self.device)

    # -- reference surface ----------------------------------------------------------------------------------------------

    def append(self, key_states: torch.Tensor, value_states: torch.Tensor) -> None:
        """Append ``[Hkv, T, D]`` keys / values (turboquant.py:1027-1140)."""
        if key_states.ndim != 3 or value_states.ndim != 3:
            raise ValueError("TurboQuantKVRow expects key/value tensors shaped [heads, tokens, dim].")
        if key_states.shape != value_states.shape:
            raise ValueError(
                f"TurboQuantKVRow key/value shape mismatch: {tuple(key_states.shape)} vs {tuple(value_states.shape)}")
        if key_states.shape[1] <= 0:
            return
        if not self.initialized:
            pool = self.pool or TurboQuantLayerPool(block_size=16)
            self._bind(pool, kv_heads=int(key_states.shape[0]), head_dim=int(key_states.shape[-1]),
                       dtype=key_states.dtype, device=key_states.device)
        elif int(key_states.shape[0]) != self.num_heads or int(key_states.shape[-1]) != self.head_dim:
            raise ValueError(
                f"TurboQuantKVRow shape mismatch: expected heads={self.num_heads} head_dim={self.head_dim}, "
                f"got {tuple(key_states.shape)}")
        assert self.pool is not None and self.dtype is not None
        if key_states.dtype != self.dtype:
            key_states, value_states = key_states.to(self.dtype), value_states.to(self.dtype)
        tokens = int(key_states.shape[1])
        self._reserve_blocks(self._length + tokens)
        launch_tq_append(self.pool, key_states.unsqueeze(0), value_states.unsqueeze(0), self._table_on_device(),
                         [self.slot], [self._length])
        self._length += tokens

    def decode_attention(self, query: torch.Tensor, *, scaling: float, num_key_value_groups: int,
                         gate: torch.Tensor | None = None) -> torch.Tensor:
        """``[Hq, 1, D]`` query (+ optional gate) -> ``[Hq, 1, D]`` (turboquant.py:1181-1293)."""
        if not self.initialized:
            raise RuntimeError("TurboQuantKVRow is not initialized.")
        if query.ndim != 3 or query.shape[1] != 1:
            raise ValueError(
                f"TurboQuantKVRow single-token decode expects [query_heads, 1, dim], got {tuple(query.shape)}")
        if int(query.shape[-1]) != self.head_dim:
            raise ValueError(
                f"TurboQuantKVRow decode head_dim mismatch: expected {self.head_dim}, got {int(query.shape[-1])}")
        if int(query.shape[0]) != self.num_heads * num_key_value_groups:
            raise ValueError(f"Expected {self.num_heads * num_key_value_groups} query heads, got {int(query.shape[0])}.")
        if gate is not None and tuple(gate.shape) != tuple(query.shape):
            raise ValueError(f"TurboQuantKVRow decode gate expects [query_heads, 1, head_dim], got {tuple(gate.shape)}")
        if self._length <= 0:
            return query.new_zeros(query.shape)
        assert self.pool is not None
        out = launch_tq_decode(self.pool, query.unsqueeze(0), self._table_on_device(), [self.slot], [self._length],
                               scaling, None if gate is None else gate.unsqueeze(0))
        return out.squeeze(0)

    def materialize(self, *, device: torch.device | None = None, dtype: torch.dtype | None = None):
        """Dense ``[Hkv, L, D]`` keys and values: de-quantized prefix followed by the window (turboquant.py:1142-1179)."""
        if not self.initialized:
            raise RuntimeError("TurboQuantKVRow is not initialized.")
        assert self.pool is not None and self.device is not None and self.dtype is not None
        heads, dim, length, lq = self.num_heads, self.head_dim, self._length, self.quantized_length
        keys = torch.empty((1, heads, length, dim), dtype=self.dtype, device=self.device)
        values = torch.empty_like(keys)
        if lq > 0:
            launch_tq_materialize(self.pool, self._table_on_device(), [lq], keys[:, :, :lq, :], values[:, :, :lq, :])
        if length > lq:
            assert self.pool.window is not None
            ring = torch.arange(lq, length, device=self.device) % self.residual_len
            keys[0, :, lq:, :] = self.pool.window[self.slot, 0].index_select(1, ring)
            values[0, :, lq:, :] = self.pool.window[self.slot, 1].index_select(1, ring)
        keys, values = keys[0], values[0]
        if device is not None or dtype is not None:
            keys = keys.to(device=device or keys.device, dtype=dtype or keys.dtype)
            values = values.to(device=device or values.device, dtype=dtype or values.dtype)
        return keys, values

    def clone(self) -> "TurboQuantKVRow":
        """Deep copy inside the same pool: fresh pages and a fresh ring slot (turboquant.py:1348-1377)."""
        cloned = TurboQuantKVRow(bits=self.bits, residual_len=self.residual_len,
                                 value_group_size=self.value_group_size)
        if not self.initialized:
            return cloned
        assert self.pool is not None and self.device is not None and self.dtype is not None
        cloned._bind(self.pool, kv_heads=self.num_heads, head_dim=self.head_dim, dtype=self.dtype, device=self.device)
        cloned._length = self._length
        if self.block_table:
            cloned.block_table = self.pool.allocate(len(self.block_table))
            src = torch.tensor(self.block_table, dtype=torch.long, device=self.device)
            dst = torch.tensor(cloned.block_table, dtype=torch.long, device=self.device)
            self.pool.packed_pages.index_copy_(0, dst, self.pool.packed_pages.index_select(0, src))
        self.pool.window[cloned.slot].copy_(self.pool.window[self.slot])
        return cloned

    def release(self) -> None:
        """Give the pages and the ring slot back to the pool; the row is empty afterwards."""
        if self.pool is not None and self.slot >= 0:
            self.pool.release_pages(self.block_table)
            self.pool.release_slot(self.slot)
        self.block_table = []
        self.slot = -1
        self._length = 0

    def to(self, *, device: torch.device | None = None, dtype: torch.dtype | None = None) -> "TurboQuantKVRow":
        if device is not None and self.device is not None and torch.device(device) != self.device:
            raise RuntimeError("TurboQuantKVRow cannot change device: its bytes live in the layer's page pool.")
        if dtype is not None and self.dtype is not None and dtype != self.dtype:
            raise RuntimeError("TurboQuantKVRow cannot change dtype: its bytes live in the layer's page pool.")
        return self
