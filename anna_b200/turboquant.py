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
                     new_lengths_dev: torch.Tensor | None = None, shared_blocks: torch.Tensor | None = None) -> None:
    """Append ``[B, Hkv, T, D]`` to B rows of one layer: ring update + quantize-on-overflow + page scatter.

    ``slots_dev`` / ``past_dev`` (optional, int64 ``[B]`` on the device) are copies of ``slots`` / ``past`` that the
    caller already holds there; ``new_lengths_dev`` (optional) receives ``past + T`` from the kernel;
    ``shared_blocks`` (optional, int32 ``[B, words]`` bit mask on the device) marks blocks whose pages already hold
    their tokens' codes (mapped from a sequence with the same prompt prefix)."""
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
            ptr(pool.packed_pages), ptr(table_dev), table_stride, ptr(shared_blocks),
            0 if shared_blocks is None else shared_blocks.stride(0), ptr(pool.window), ptr(slots_dev), ptr(past_dev),
            ptr(new_lengths_dev), ptr(tables.signs1), ptr(tables.signs2), ptr(tables.centroids), ptr(tables.boundaries), batch, kv_heads,
            tokens, dim, pool.block_size, pool.residual_len, pool.bits, pool.value_group, pool.capacity(), max_blocks,
            dtype_code(key_states.dtype), ptr(pool.status), stream_ptr(device)), "anna_tq_append")


def launch_tq_decode(pool: TurboQuantLayerPool, query_states: torch.Tensor, table_dev: torch.Tensor | None,
                     slots: list[int], lengths: list[int], scaling: float, gate: torch.Tensor | None, *,
                     slots_dev: torch.Tensor | None = None, lengths_dev: torch.Tensor | None = None,
                     output: torch.Tensor | None = None, peer_outputs: tuple[int, ...] = ()) -> torch.Tensor:
    """Decode ``[B, Hq, 1, D]`` queries against B rows of one layer (packed prefix + window ring).

    ``slots_dev`` / ``lengths_dev`` (optional, int64 ``[B]`` on the device) are copies of ``slots`` / ``lengths``
    that the caller already holds there.  ``output`` (optional, ``[B, Hq, 1, D]``, last dimension contiguous) receives
    the result instead of a new tensor; ``peer_outputs`` are device addresses, in other GPUs' memory, of tensors with
    the strides of ``output`` that receive the same rows (KV-head-sharded decode, see ``sharding.PeerHeadGather``)."""
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
    if output is None:
        out = torch.empty((batch, heads, 1, dim), dtype=query.dtype, device=device)
    else:
        if tuple(output.shape) != (batch, heads, 1, dim) or output.dtype != query.dtype or output.device != device \
                or output.stride(3) != 1:
            raise ValueError("output must be [batch, heads, 1, head_dim] in the query dtype on the query device with "
                             "a contiguous last dimension")
        out = output
    table_stride = 0 if table_dev is None else table_dev.stride(0)
    max_blocks = 0 if table_dev is None else int(table_dev.shape[1])
    max_len = max_blocks * pool.block_size + pool.residual_len
    stats, values, capacity, counters = split_scratch(device, batch, heads, dim, pool.kv_heads, max_len,
                                                      turboquant=(max_blocks, pool.block_size, pool.residual_len))
    frags = query_scratch(device, batch, heads, pool.kv_heads, dim)
    common = (
        ptr(query), query.stride(0), query.stride(1), ptr(pool.packed_pages), ptr(table_dev), table_stride,
        ptr(pool.window), ptr(slots_dev), ptr(lengths_dev), ptr(tables.signs1), ptr(tables.signs2),
        ptr(tables.centroids), ptr(gate), 0 if gate is None else gate.stride(0),
        0 if gate is None else gate.stride(1), ptr(out), out.stride(0), out.stride(1), ptr(stats), ptr(values),
        capacity, 0, ptr(counters), ptr(frags), frags.numel(), batch, heads, pool.kv_heads, dim, pool.block_size,
        pool.residual_len, pool.bits, pool.value_group, pool.capacity(), max_blocks, float(scaling),
        dtype_code(query.dtype))
    with on_device(device):
        if peer_outputs:
            import ctypes

            peers = (ctypes.c_void_p * len(peer_outputs))(*peer_outputs)
            _lib.check(_lib.lib().anna_tq_paged_decode_peers(*common, peers, len(peer_outputs), stream_ptr(device)),
                       "anna_tq_paged_decode_peers")
        else:
            _lib.check(_lib.lib().anna_tq_paged_decode(*common, stream_ptr(device)), "anna_tq_paged_decode")
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


def launch_tq_gather_dense(pool: TurboQuantLayerPool, table_dev: torch.Tensor | None, slots: list[int], lengths: list[int],
                           max_len: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Dense ``[B, Hkv, max_len, D]`` keys and values of B rows of one layer in one launch: de-quantized prefix, window
    tokens, zero padding; and the rows' lengths as the int64 device tensor the launch read them from."""
    assert pool.window is not None and pool.device is not None and pool.dtype is not None
    device = pool.device
    batch = len(lengths)
    tables = key_tables(head_dim=pool.head_dim, bits=pool.bits, device=device)
    meta = MetadataUploader.for_device(device).upload([lengths, slots])
    keys = torch.empty((batch, pool.kv_heads, max_len, pool.head_dim), dtype=pool.dtype, device=device)
    values = torch.empty_like(keys)
    table_stride = 0 if table_dev is None else table_dev.stride(0)
    max_blocks = 0 if table_dev is None else int(table_dev.shape[1])
    with on_device(device):
        _lib.check(_lib.lib().anna_tq_gather_dense(
            ptr(pool.packed_pages), ptr(table_dev), table_stride, ptr(pool.window), ptr(meta[1]), ptr(meta[0]),
            ptr(tables.signs1), ptr(tables.signs2), ptr(tables.centroids), ptr(keys), ptr(values), keys.stride(0),
            keys.stride(1), keys.stride(2), batch, pool.kv_heads, pool.head_dim, pool.block_size, pool.residual_len,
            pool.bits, pool.value_group, pool.capacity(), max_blocks, int(max_len), dtype_code(pool.dtype),
            stream_ptr(device)), "anna_tq_gather_dense")
    return keys, values, meta[0]


class TurboQuantTensorRow:
    """History of one tensor (the K or the V of one sequence) with MSE-only TurboQuant codes for everything older than
    the newest ``residual_len`` tokens; mirrors ``TurboQuantTensorRow`` of the Gemma4 runtime
    (src/anna/model/turboquant.py:335-477): ``append([heads, tokens, dim])``, ``materialize``, ``clone``, ``to``.

    Codes live in growable device buffers (indices packed to ``bits`` / 4-bit fields, fp32 norms); the quantizer and
    its inverse are CUDA kernels, nothing is computed on the host."""

    def __init__(self, *, bits: int, residual_len: int) -> None:
        self.bits = int(bits)
        self.residual_len = max(1, int(residual_len))
        self.device: torch.device | None = None
        self.dtype: torch.dtype | None = None
        self.head_dim: int | None = None
        self._codes: torch.Tensor | None = None   # uint8 [heads, capacity, row_bytes]
        self._norms: torch.Tensor | None = None   # float32 [heads, capacity]
        self._quantized = 0
        self._residual: torch.Tensor | None = None
        self._length = 0

    @property
    def length(self) -> int:
        return self._length

    @property
    def quantized_length(self) -> int:
        return self._quantized

    @property
    def initialized(self) -> bool:
        return self.device is not None and self.dtype is not None and self.head_dim is not None

    def _ensure_capacity(self, heads: int, tokens: int) -> None:
        assert self.device is not None and self.head_dim is not None
        have = 0 if self._codes is None else int(self._codes.shape[1])
        if tokens <= have:
            return
        capacity = max(tokens, 16, 2 * have)  # growth rule of the reference buffers (turboquant.py:576-581)
        row_bytes = _lib.lib().anna_tq_tensor_row_bytes(self.head_dim, self.bits)
        if row_bytes <= 0:
            raise RuntimeError(f"unsupported TurboQuant tensor geometry: head_dim={self.head_dim}, bits={self.bits}")
        codes = torch.empty((heads, capacity, row_bytes), dtype=torch.uint8, device=self.device)
        norms = torch.empty((heads, capacity), dtype=torch.float32, device=self.device)
        if self._codes is not None and self._quantized > 0:
            codes[:, : self._quantized].copy_(self._codes[:, : self._quantized])
            norms[:, : self._quantized].copy_(self._norms[:, : self._quantized])
        self._codes, self._norms = codes, norms

    def append(self, tensor: torch.Tensor) -> None:
        if tensor.ndim != 3:
            raise ValueError(f"TurboQuantTensorRow expects [heads, tokens, dim], got {tuple(tensor.shape)}")
        if tensor.shape[1] <= 0:
            return
        if not self.initialized:
            _require_cuda(tensor, "TurboQuantTensorRow.append")
            self.device, self.dtype, self.head_dim = tensor.device, tensor.dtype, int(tensor.shape[-1])
            self._residual = tensor.detach().contiguous()
            self._length = int(tensor.shape[1])
        else:
            if tensor.device != self.device:
                tensor = tensor.to(device=self.device)
            if tensor.dtype != self.dtype:
                tensor = tensor.to(dtype=self.dtype)
            if int(tensor.shape[-1]) != self.head_dim:
                raise ValueError(
                    f"TurboQuantTensorRow head_dim mismatch: expected {self.head_dim}, got {int(tensor.shape[-1])}")
            residual = self._residual
            self._residual = (tensor.detach().contiguous() if residual is None
                              else torch.cat((residual, tensor.detach()), dim=1).contiguous())
            self._length += int(tensor.shape[1])
        residual = self._residual
        if residual is None or residual.shape[1] <= self.residual_len:
            return
        overflow = int(residual.shape[1] - self.residual_len)
        heads = int(residual.shape[0])
        self._ensure_capacity(heads, self._quantized + overflow)
        assert self._codes is not None and self._norms is not None and self.device is not None
        tables = key_tables(head_dim=self.head_dim, bits=self.bits, device=self.device, variant="mse")
        with on_device(self.device):
            _lib.check(_lib.lib().anna_tq_tensor_quantize(
                ptr(residual), residual.stride(0), residual.stride(1), ptr(self._codes), ptr(self._norms),
                int(self._codes.shape[1]), self._quantized, heads, overflow, self.head_dim, self.bits,
                ptr(tables.signs1), ptr(tables.boundaries), dtype_code(residual.dtype), stream_ptr(self.device)),
                "anna_tq_tensor_quantize")
        self._quantized += overflow
        self._residual = residual[:, overflow:, :].contiguous()

    def materialize(self, *, device: torch.device | None = None, dtype: torch.dtype | None = None) -> torch.Tensor:
        if not self.initialized:
            raise RuntimeError("TurboQuantTensorRow is not initialized.")
        assert self.device is not None and self.dtype is not None and self.head_dim is not None
        residual = self._residual
        window = 0 if residual is None else int(residual.shape[1])
        if self._quantized == 0 and window == 0:
            out = torch.empty((0, 0, self.head_dim), device=self.device, dtype=self.dtype)
        else:
            heads = int(self._codes.shape[0]) if self._quantized else int(residual.shape[0])
            out = torch.empty((heads, self._quantized + window, self.head_dim), device=self.device, dtype=self.dtype)
            if self._quantized:
                tables = key_tables(head_dim=self.head_dim, bits=self.bits, device=self.device, variant="mse")
                with on_device(self.device):
                    _lib.check(_lib.lib().anna_tq_tensor_dequantize(
                        ptr(self._codes), ptr(self._norms), int(self._codes.shape[1]), 0, ptr(out), out.stride(0),
                        out.stride(1), heads, self._quantized, self.head_dim, self.bits, ptr(tables.signs1),
                        ptr(tables.centroids), dtype_code(out.dtype), stream_ptr(self.device)),
                        "anna_tq_tensor_dequantize")
            if window:
                out[:, self._quantized:].copy_(residual)
        kwargs: dict[str, object] = {}
        if device is not None:
            kwargs["device"] = device
        if dtype is not None:
            kwargs["dtype"] = dtype
        return out.to(**kwargs) if kwargs else out

    def clone(self) -> "TurboQuantTensorRow":
        cloned = TurboQuantTensorRow(bits=self.bits, residual_len=self.residual_len)
        cloned.device, cloned.dtype, cloned.head_dim = self.device, self.dtype, self.head_dim
        cloned._length, cloned._quantized = self._length, self._quantized
        cloned._codes = None if self._codes is None else self._codes.clone()
        cloned._norms = None if self._norms is None else self._norms.clone()
        cloned._residual = None if self._residual is None else self._residual.clone()
        return cloned

    def to(self, *, device: torch.device | None = None, dtype: torch.dtype | None = None) -> "TurboQuantTensorRow":
        if not self.initialized:
            return self
        if device is not None and torch.device(device).type != "cuda":
            raise RuntimeError("TurboQuantTensorRow lives on a CUDA device; there is no CPU implementation.")
        if device is not None:
            if self._codes is not None:
                self._codes = self._codes.to(device=device)
                self._norms = self._norms.to(device=device)
            if self._residual is not None:
                self._residual = self._residual.to(device=device)
            self.device = torch.device(device)
        if dtype is not None:
            if self._residual is not None:
                self._residual = self._residual.to(dtype=dtype)
            self.dtype = dtype
        return self


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
        self._table_np = None   # int32 mirror of block_table (see table_array)
        self._table_np_valid = 0
        self._length = 0
        self._privatized_block: int | None = None  # block whose page id changed by copy on write (see _reserve_blocks)

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

    def _privatize_partial_block(self, new_length: int) -> None:
        """Copy on first write: a clone shares its packed pages with the row it was cloned from.  Full blocks are never
        written again, but the last, partly filled block is: before an append that reaches it, a row that is not the
        only owner of that page copies it, maps the copy and leaves the block index in ``_privatized_block`` so that
        the owner of the device block table uploads the new id."""
        assert self.pool is not None
        pool = self.pool
        quantized_now = self.quantized_length
        if max(0, int(new_length) - self.residual_len) <= quantized_now or quantized_now % pool.block_size == 0:
            return
        blk = quantized_now // pool.block_size
        if blk >= len(self.block_table) or pool.page_owners(self.block_table[blk]) <= 1:
            return
        shared = self.block_table[blk]
        private = pool.allocate(1)[0]
        assert pool.packed_pages is not None
        pool.packed_pages[private].copy_(pool.packed_pages[shared])
        self.block_table[blk] = private
        self._table_np_valid = min(self._table_np_valid, blk)
        pool.release_pages([shared])
        self._privatized_block = blk

    def _reserve_blocks(self, new_length: int) -> None:
        """Take pages for every block the quantized prefix will reach once the row holds new_length tokens."""
        assert self.pool is not None
        self._privatize_partial_block(new_length)
        quantized = max(0, int(new_length) - self.residual_len)
        need = (quantized + self.pool.block_size - 1) // self.pool.block_size
        if need > len(self.block_table):
            self.block_table.extend(self.pool.allocate(need - len(self.block_table)))

    def table_array(self):
        """``block_table`` as an int32 numpy array.  The array is kept between calls and only entries added (or
        replaced by copy on write) since the last call are converted, so rebuilding the device table of a re-stacked
        batch costs a memory copy per row instead of a list conversion."""
        import numpy as np

        n = len(self.block_table)
        arr = self._table_np
        valid = min(self._table_np_valid, n)
        if arr is None or arr.shape[0] < n:
            grown = np.empty(max(n, 16, 0 if arr is None else 2 * arr.shape[0]), dtype=np.int32)
            if valid:
                grown[:valid] = arr[:valid]
            arr = self._table_np = grown
        if valid < n:
            arr[valid:n] = self.block_table[valid:n]
        self._table_np_valid = n
        return arr[:n]

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
        """An independent copy of the row's state (turboquant.py:1348-1377) that copies no packed page: the clone maps
        the same pages (one more owner each) and gets a window ring of its own; whichever of the two rows appends into
        the partly filled last block first copies that one page (``_reserve_blocks``)."""
        cloned = TurboQuantKVRow(bits=self.bits, residual_len=self.residual_len,
                                 value_group_size=self.value_group_size)
        if not self.initialized:
            return cloned
        assert self.pool is not None and self.device is not None and self.dtype is not None
        cloned._bind(self.pool, kv_heads=self.num_heads, head_dim=self.head_dim, dtype=self.dtype, device=self.device)
        cloned._length = self._length
        for page_id in self.block_table:
            self.pool.retain_page(page_id)
        cloned.block_table = list(self.block_table)
        self.pool.window[cloned.slot].copy_(self.pool.window[self.slot])
        return cloned

    def release(self) -> None:
        """Give the pages and the ring slot back to the pool; the row is empty afterwards."""
        if self.pool is not None and self.slot >= 0:
            self.pool.release_pages(self.block_table)
            self.pool.release_slot(self.slot)
        self.block_table = []
        self._table_np_valid = 0
        self.slot = -1
        self._length = 0

    def to(self, *, device: torch.device | None = None, dtype: torch.dtype | None = None) -> "TurboQuantKVRow":
        if device is not None and self.device is not None and torch.device(device) != self.device:
            raise RuntimeError("TurboQuantKVRow cannot change device: its bytes live in the layer's page pool.")
        if dtype is not None and self.dtype is not None and dtype != self.dtype:
            raise RuntimeError("TurboQuantKVRow cannot change dtype: its bytes live in the layer's page pool.")
        return self
