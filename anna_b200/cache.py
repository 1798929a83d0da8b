"""KV-cache manager of the decode path: page allocators, block tables and the batched cache object.

Host-side mirror of ``Qwen3PagedLayerAllocator`` / ``Qwen3PageAllocator`` / ``Qwen3DynamicCache``
(``src/anna/model/ops.py:92-1439``) with the same constructor arguments, lifecycle methods and allocation policy
(LIFO free list, growth by ``max(n, capacity or 16)``, reversed release order, refcounts), so block tables match the
reference's for the same sequence of calls.  What differs is where the bytes live and who moves them:

* un-quantized layers keep ``key_pages`` / ``value_pages`` ``[P, Hkv, S, D]`` on the GPU and one CUDA launch writes
  the new tokens of every row (``anna_paged_kv_write``) instead of per-row slice copies (ops.py:748-777);
* TurboQuant layers keep *packed* pages ``uint8 [P, Hkv, chunk_bytes]`` plus a ring of the newest ``residual_len``
  tokens per sequence; one launch (``anna_tq_append``) does ring update, quantize-on-overflow, bit-packing and page
  scatter for the whole batch, and one launch pair decodes the whole batch (``anna_tq_paged_decode``) instead of
  the per-row Python loops at ops.py:632 and :1057.  The reference never pages quantized rows (ops.py:903-904); the
  rule here is: quantized token ``j`` of a row lives in block ``j // S`` of the row's table, allocated from the
  layer's packed pool when the quantized length first reaches it.

There is no CPU path: tensors must be CUDA tensors and the CUDA library must be built.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

import numpy as np
import torch

from . import _lib
from .fused_ops import MetadataUploader, dtype_code, on_device, ptr, stream_ptr
from .pools import Qwen3PagedLayerAllocator, TurboQuantLayerPool
from .prefix_block_cache import PrefixBlockPool
from .turboquant import (VALID_KV_CACHE_QUANT_BITS, TurboQuantKVRow, launch_tq_append, launch_tq_decode,
                         launch_tq_gather_dense)


@dataclass
class KVCacheConfig:
    """The fields of Qwen3_5TextConfig that the cache reads (qwen3_5_text_config.py:150, ops.py:255-270)."""

    num_hidden_layers: int
    layer_types: tuple[str, ...] | list[str] = field(default_factory=tuple)
    cache_block_size: int = 32

    def __post_init__(self) -> None:
        if not self.layer_types:
            self.layer_types = tuple("full_attention" for _ in range(self.num_hidden_layers))


class Qwen3PageAllocator:
    """One allocator per engine: per-layer page pools + prefix block registry (ops.py:248-339)."""

    def __init__(self, config, *, maintain_full_attention_mirror: bool = False):
        self.config = config
        self.block_size = max(1, int(config.cache_block_size))
        self.prefix_block_pool = PrefixBlockPool()
        self.layers = [
            Qwen3PagedLayerAllocator(
                self.block_size,
                on_page_freed=lambda pid, li=layer_idx: self.prefix_block_pool.discard_page(li, pid),
                on_trim=lambda li=layer_idx: self.prefix_block_pool.clear_layer(li),
                listening=lambda: len(self.prefix_block_pool) > 0,
            )
            for layer_idx in range(config.num_hidden_layers)
        ]
        # packed pages of quantized layers are shared the same way, keyed by the whole prompt prefix up to the block
        self.packed_prefix_block_pool = PrefixBlockPool()
        self.turboquant_layers = [
            TurboQuantLayerPool(
                self.block_size,
                on_page_freed=lambda pid, li=layer_idx: self.packed_prefix_block_pool.discard_page(li, pid),
                listening=lambda: len(self.packed_prefix_block_pool) > 0)
            for layer_idx in range(config.num_hidden_layers)
        ]
        # The reference keeps a contiguous dense mirror of full-attention layers by default; this build gathers the
        # dense view from the pages on demand, so the switch is accepted and ignored.
        self.maintain_full_attention_mirror = False
        self.full_attention_layer_indices = tuple(
            idx for idx, layer_type in enumerate(config.layer_types) if layer_type == "full_attention")
        self.mirrored_full_attention_layer_indices: tuple[int, ...] = ()

    def allocate(self, layer_idx: int, num_pages: int, *, key_template: torch.Tensor,
                 value_template: torch.Tensor) -> list[int]:
        return self.layers[layer_idx].allocate(num_pages, key_template=key_template, value_template=value_template)

    def release_pages(self, layer_idx: int, page_ids: list[int]) -> None:
        if page_ids:
            self.layers[layer_idx].release_pages(page_ids)

    def free(self, layer_idx: int, page_ids: list[int]) -> None:
        self.release_pages(layer_idx, page_ids)

    def retain_shared_page(self, layer_idx: int, page_id: int) -> None:
        self.layers[layer_idx].retain_page(page_id)

    def ensure_capacity(self, layer_idx: int, required_pages: int, *, key_template: torch.Tensor,
                        value_template: torch.Tensor) -> int:
        return self.layers[layer_idx].ensure_capacity(required_pages, key_template=key_template,
                                                      value_template=value_template)

    def trim(self) -> int:
        return sum(layer.trim() for layer in self.layers) + sum(pool.trim() for pool in self.turboquant_layers)

    def clear(self) -> int:
        released = 0
        for layer in self.layers:
            released += layer.capacity()
            layer._book.clear()
            layer.key_pages = None
            layer.value_pages = None
        for pool in self.turboquant_layers:
            released += pool.clear()
        self.prefix_block_pool.clear()
        self.packed_prefix_block_pool.clear()
        return released

    def to(self, *, device: torch.device | None = None, dtype: torch.dtype | None = None) -> "Qwen3PageAllocator":
        for layer in self.layers:
            layer.to(device=device, dtype=dtype)
        return self

    def uses_contiguous_full_attention_mirror(self, layer_idx: int) -> bool:
        return False


# ---------------------------------------------------------------------------------------------------------------
# the batched cache object


def _i32(values, device: torch.device) -> torch.Tensor:
    return torch.tensor(values, dtype=torch.int32, device=device)


class _DeviceLengths:
    """Row lengths (and TurboQuant ring slots) of one layer, kept on the device between steps.

    ``rows`` is a small ring of int64 ``[B]`` tensors; ``rows[pos]`` mirrors the host list ``host``.  An append reads
    ``rows[pos]`` as the lengths before the call and lets the kernel write the lengths after it into the next row of
    the ring, so a steady decode loop uploads no metadata at all.  Tensors handed out from the ring stay valid until
    the ring wraps (``DEPTH - 1`` further appends to the same layer)."""

    DEPTH = 4
    __slots__ = ("rows", "pos", "host", "slots_dev", "slots_host", "device")

    def __init__(self, batch: int, device: torch.device) -> None:
        self.rows = list(torch.zeros((self.DEPTH, batch), dtype=torch.int64, device=device).unbind(0))
        self.pos = 0
        self.host: list[int] | None = None
        self.slots_dev: torch.Tensor | None = None
        self.slots_host: list[int] | None = None
        self.device = device

    def current(self, lengths: list[int]) -> torch.Tensor | None:
        """Device copy of ``lengths`` if the ring holds exactly these values."""
        return self.rows[self.pos] if self.host == lengths else None

    def before_append(self, past: list[int]) -> tuple[torch.Tensor, torch.Tensor]:
        """(lengths before the append on the device, ring row that will receive the lengths after it)."""
        past_dev = self.current(past)
        if past_dev is None:
            past_dev = MetadataUploader.for_device(self.device).upload([past])[0]
        return past_dev, self.rows[(self.pos + 1) % self.DEPTH]

    def after_append(self, lengths: list[int]) -> None:
        self.pos = (self.pos + 1) % self.DEPTH
        self.host = list(lengths)

    def slots(self, slots: list[int]) -> torch.Tensor:
        if self.slots_dev is None or self.slots_host != slots:
            self.slots_dev = MetadataUploader.for_device(self.device).upload([slots])[0]
            self.slots_host = list(slots)
        return self.slots_dev


class Qwen3DynamicCache:
    def __init__(self, config, *, allocator: Qwen3PageAllocator | None = None, batch_size: int = 0,
                 kv_cache_quantization: str = "none", kv_cache_quant_bits: int = 4, kv_cache_residual_len: int = 128):
        self.config = config
        self.allocator = allocator or Qwen3PageAllocator(config)
        self.kv_cache_quantization = kv_cache_quantization.strip().lower()
        if self.kv_cache_quantization not in {"none", "turboquant"}:
            raise ValueError(f"Unsupported Qwen3 KV-cache quantization mode: {kv_cache_quantization}")
        self.kv_cache_quant_bits = int(kv_cache_quant_bits)
        if self.kv_cache_quant_bits not in VALID_KV_CACHE_QUANT_BITS:
            raise ValueError(
                f"Unsupported Qwen3 TurboQuant bit-width: {kv_cache_quant_bits}. "
                f"Expected one of {sorted(VALID_KV_CACHE_QUANT_BITS)}.")
        self.kv_cache_residual_len = max(1, int(kv_cache_residual_len))
        self._turboquant_layer_index_set = {
            idx for idx, layer_type in enumerate(config.layer_types)
            if self.kv_cache_quantization == "turboquant" and layer_type == "full_attention"
        }
        layers = config.num_hidden_layers
        self.conv_states: list[torch.Tensor | None] = [None] * layers
        self.recurrent_states: list[torch.Tensor | None] = [None] * layers
        self.block_size = max(1, int(config.cache_block_size))
        self.layer_lengths: list[list[int]] = [[0] * batch_size for _ in range(layers)]
        self.page_tables: list[list[list[int]]] = [[[] for _ in range(batch_size)] for _ in range(layers)]
        self.turboquant_rows: list[list[TurboQuantKVRow | None]] = [[None] * batch_size for _ in range(layers)]
        self.page_table_caches: list[torch.Tensor | None] = [None] * layers
        self.page_table_capacities: list[int] = [0] * layers
        self._table_host: list[np.ndarray | None] = [None] * layers       # host mirror of page_table_caches
        self._table_rows_synced: list[list[int] | None] = [None] * layers  # blocks already on the device per row
        self._table_blocks_total: list[int] = [-1] * layers                # sum of table lengths at the last sync
        self._dev_lengths: list[_DeviceLengths | None] = [None] * layers  # device mirror of layer_lengths
        # per layer: tokens every row can still take without a new page (None = unknown), and the block-table view
        # returned by the last sync (valid while no table has changed)
        self._page_headroom: list[int | None] = [None] * layers
        self._table_view: list[torch.Tensor | None] = [None] * layers
        self.seen_tokens = 0
        self.rope_deltas: torch.Tensor | None = None
        self.reserved_seq_capacity = 0
        self._released = False
        self._prefill_input_ids: torch.Tensor | None = None
        self._prompt_token_ids: list[int] | None = None
        self._prompt_prefix_keys: list[tuple] | None = None   # per full prompt block: key of the prefix ending there
        self._packed_blocks_registered: list[int] = [0] * layers  # prompt blocks of row 0 already offered for sharing
        self._prefix_kv_share = os.environ.get("ANNA_PREFIX_KV_SHARE", "1") != "0"

    # -- small bookkeeping (ops.py:398-441, :859-889) ----------------------------------------------------------------

    def attach_prefill_input_ids(self, input_ids: torch.Tensor | None) -> None:
        self._prefill_input_ids = input_ids

    def detach_prefill_input_ids(self) -> None:
        self._prefill_input_ids = None

    def set_prompt_token_ids(self, input_ids: torch.Tensor | None) -> None:
        if input_ids is None or not self._prefix_kv_share or self._prompt_token_ids is not None:
            return
        if int(input_ids.shape[0]) != 1 or self.get_seq_length() != 0 or int(input_ids.shape[1]) <= 0:
            return
        self._prompt_token_ids = [int(t) for t in input_ids[0].tolist()]
        self._prompt_prefix_keys = None

    def reserve_sequence_capacity(self, seq_length: int) -> None:
        self.reserved_seq_capacity = max(0, int(seq_length))
        self._page_headroom = [None] * len(self._page_headroom)  # tables may have to grow at the next append

    @property
    def has_previous_state(self) -> bool:
        return any(s is not None for s in self.conv_states) or any(s is not None for s in self.recurrent_states)

    def _ensure_batch_size(self, batch_size: int) -> None:
        if not self.layer_lengths or not self.layer_lengths[0]:
            layers = self.config.num_hidden_layers
            self.layer_lengths = [[0] * batch_size for _ in range(layers)]
            self.page_tables = [[[] for _ in range(batch_size)] for _ in range(layers)]
            self.turboquant_rows = [[None] * batch_size for _ in range(layers)]
            return
        if len(self.layer_lengths[0]) != batch_size:
            raise ValueError(f"Cache batch size mismatch: expected {len(self.layer_lengths[0])}, got {batch_size}")

    def uses_turboquant_for_layer(self, layer_idx: int) -> bool:
        return layer_idx in self._turboquant_layer_index_set

    def get_batch_size(self) -> int:
        if self.layer_lengths and self.layer_lengths[0]:
            return len(self.layer_lengths[0])
        for group in (self.conv_states, self.recurrent_states):
            for state in group:
                if state is not None:
                    return int(state.shape[0])
        if self.rope_deltas is not None:
            return int(self.rope_deltas.shape[0])
        return 0

    def _request_seq_length(self, batch_idx: int) -> int:
        for layer_idx in range(self.config.num_hidden_layers):
            length = self.layer_lengths[layer_idx][batch_idx]
            if length > 0:
                return length
        return 0

    def get_seq_length(self, batch_idx: int | None = None) -> int:
        if batch_idx is not None:
            return self._request_seq_length(batch_idx)
        batch_size = self.get_batch_size()
        if batch_size == 0:
            return 0
        return max(self._request_seq_length(idx) for idx in range(batch_size))

    def get_seq_lengths(self, *, device: torch.device | None = None) -> torch.Tensor:
        lengths = [self._request_seq_length(idx) for idx in range(self.get_batch_size())]
        return torch.tensor(lengths, dtype=torch.long, device=device)

    # -- device-side block tables ----------------------------------------------------------------------------------

    def _tables_of(self, layer_idx: int) -> list[list[int]]:
        if self.uses_turboquant_for_layer(layer_idx):
            return [[] if row is None else row.block_table for row in self.turboquant_rows[layer_idx]]
        return self.page_tables[layer_idx]

    def _sync_page_table_layer_buffer(self, layer_idx: int, *, batch_size: int,
                                      device: torch.device) -> torch.Tensor | None:
        """Device copy of the layer's block tables: int32 [B, capacity], -1 padded (ops.py:532-588).

        Only rows whose table grew since the last call are uploaded."""
        tables = self._tables_of(layer_idx)
        total = 0
        required = 0
        for table in tables:
            n = len(table)
            total += n
            if n > required:
                required = n
        if required <= 0:
            self.page_table_caches[layer_idx] = None
            self.page_table_capacities[layer_idx] = 0
            self._table_rows_synced[layer_idx] = None
            self._table_host[layer_idx] = None
            self._table_blocks_total[layer_idx] = -1
            return None
        buffer = self.page_table_caches[layer_idx]
        synced = self._table_rows_synced[layer_idx]
        if (buffer is not None and synced is not None and buffer.shape[0] == batch_size and buffer.device == device
                and buffer.shape[1] >= required and self._table_blocks_total[layer_idx] == total):
            return buffer[:, :required]  # nothing was appended since the last sync
        if (buffer is None or buffer.shape[0] != batch_size or buffer.device != device
                or buffer.shape[1] < required or synced is None):
            capacity = max(required, max(1, self.page_table_capacities[layer_idx] * 2))
            # host mirror of the device table; a full build goes up through the pinned staging ring in one copy
            host = np.full((batch_size, capacity), -1, dtype=np.int32)
            tq_rows = self.turboquant_rows[layer_idx] if self.uses_turboquant_for_layer(layer_idx) else None
            for row_idx, table in enumerate(tables):
                if table:
                    row = None if tq_rows is None else tq_rows[row_idx]
                    host[row_idx, : len(table)] = table if row is None else row.table_array()
            if device.type == "cuda":
                buffer = MetadataUploader.for_device(device).upload_i32(host.reshape(-1)).view(batch_size, capacity)
            else:  # host-side bookkeeping of a cache that holds no device memory
                buffer = torch.from_numpy(host.copy())
            self.page_table_caches[layer_idx] = buffer
            self.page_table_capacities[layer_idx] = capacity
            self._table_host[layer_idx] = host
            self._table_rows_synced[layer_idx] = [len(t) for t in tables]
            self._table_blocks_total[layer_idx] = total
            return buffer[:, :required]
        # Patch: the new entries go up as (row, column, page id) triples through a pinned staging buffer and a small
        # scatter kernel writes them into the device table, so a step in which a few rows of a ragged batch take a page
        # moves a few dozen bytes and never waits for the GPU.  Entries are write-once while a row lives.
        host = self._table_host[layer_idx]
        tq_rows = self.turboquant_rows[layer_idx] if self.uses_turboquant_for_layer(layer_idx) else None
        pieces: list[np.ndarray] = []
        for row_idx, table in enumerate(tables):
            have = synced[row_idx]
            n = len(table)
            if n > have:
                row = None if tq_rows is None else tq_rows[row_idx]
                new_pages = np.asarray(table[have:], dtype=np.int32) if row is None else row.table_array()[have:n]
                host[row_idx, have:n] = new_pages
                synced[row_idx] = n
                piece = np.empty((n - have, 3), dtype=np.int32)
                piece[:, 0] = row_idx
                piece[:, 1] = np.arange(have, n, dtype=np.int32)
                piece[:, 2] = new_pages
                pieces.append(piece)
        if pieces:
            patch = pieces[0] if len(pieces) == 1 else np.concatenate(pieces)
            if device.type != "cuda":  # host-side bookkeeping of a cache that holds no device memory
                buffer[patch[:, 0].astype(np.int64), patch[:, 1].astype(np.int64)] = torch.from_numpy(
                    np.ascontiguousarray(patch[:, 2]))
            else:
                entries = MetadataUploader.for_device(device).upload_i32(patch.reshape(-1))
                with on_device(device):
                    _lib.check(_lib.lib().anna_block_table_patch(
                        ptr(buffer), buffer.stride(0), int(buffer.shape[0]), int(buffer.shape[1]), ptr(entries),
                        int(patch.shape[0]), stream_ptr(device)), "anna_block_table_patch")
        self._table_blocks_total[layer_idx] = total
        return buffer[:, :required]

    # -- append ------------------------------------------------------------------------------------------------------

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int, *,
               require_dense_cache: bool = True):
        """Append ``[B, Hkv, T, D]`` keys / values; returns ``(K | None, V | None, past_lengths)`` (ops.py:662-746)."""
        if key_states.shape != value_states.shape or key_states.dim() != 4:
            raise ValueError("update expects matching [batch, kv_heads, tokens, head_dim] key and value tensors")
        if self.uses_turboquant_for_layer(layer_idx):
            return self._update_turboquant_layer(key_states, value_states, layer_idx,
                                                 require_dense_cache=require_dense_cache)
        batch_size, kv_heads, append_length, head_dim = (int(v) for v in key_states.shape)
        self._ensure_batch_size(batch_size)
        device = key_states.device
        past = self.layer_lengths[layer_idx]
        use_prefix_share = self._prefix_kv_share and batch_size == 1 and self._prompt_token_ids is not None
        segments = [(0, append_length)]  # token ranges of this append that must be written
        headroom = self._page_headroom[layer_idx]
        table_dev = None
        if headroom is not None and headroom >= append_length and not use_prefix_share:
            # steady decode: every row still has room in its last page, so no table changes
            self._page_headroom[layer_idx] = headroom - append_length
            lengths = [n + append_length for n in past]
            self.layer_lengths[layer_idx] = lengths
            table_dev = self._table_view[layer_idx]
        else:
            reserved_length = max(append_length, self.reserved_seq_capacity)
            hint = (reserved_length + self.block_size - 1) // self.block_size
            if hint > 0:
                self.allocator.ensure_capacity(layer_idx, hint * batch_size, key_template=key_states,
                                               value_template=value_states)
            lengths = list(past)
            headroom = None
            for batch_idx in range(batch_size):
                required = past[batch_idx] + append_length
                table = self.page_tables[layer_idx][batch_idx]
                if append_length > 0:
                    self._privatize_last_block(layer_idx, batch_idx, key_states, value_states)
                if use_prefix_share:
                    segments = self._map_prefix_shared_blocks(key_states, value_states, layer_idx, batch_idx,
                                                              append_length)
                blocks = (max(required, self.reserved_seq_capacity) + self.block_size - 1) // self.block_size
                if len(table) < blocks:
                    table.extend(self.allocator.allocate(layer_idx, blocks - len(table), key_template=key_states,
                                                         value_template=value_states))
                lengths[batch_idx] = required
                room = len(table) * self.block_size - required
                headroom = room if headroom is None or room < headroom else headroom
            self.layer_lengths[layer_idx] = lengths
            self._page_headroom[layer_idx] = headroom
            self._table_view[layer_idx] = None
        newest = max(lengths, default=0)
        if newest > self.seen_tokens:
            self.seen_tokens = newest
        if device.type == "cuda":
            state = self._device_lengths_of(layer_idx, batch_size, device)
            past_lengths, new_lengths = state.before_append(past)
        else:  # bookkeeping only (the launch below refuses CPU tensors)
            state = None
            past_lengths, new_lengths = torch.tensor(past, device=device, dtype=torch.long), None
        if table_dev is None:
            table_dev = self._sync_page_table_layer_buffer(layer_idx, batch_size=batch_size, device=device)
            self._table_view[layer_idx] = table_dev
        layer = self.allocator.layers[layer_idx]
        if table_dev is not None and append_length > 0:
            if segments == [(0, append_length)]:
                self._launch_page_write(layer, key_states, value_states, table_dev, past, past_dev=past_lengths,
                                        new_lengths_dev=new_lengths)
                if state is not None:
                    state.after_append(lengths)
            else:
                for start, end in segments:
                    if end > start:
                        self._launch_page_write(layer, key_states[:, :, start:end, :],
                                                value_states[:, :, start:end, :], table_dev,
                                                [p + start for p in past])
                if state is not None:
                    state.host = None  # the ring does not hold the new lengths
        if not require_dense_cache:
            return None, None, past_lengths
        gathered_key, gathered_value, _ = self._gather_layer_cache(layer_idx)
        return gathered_key, gathered_value, past_lengths

    def _resync_row_from(self, layer_idx: int, batch_idx: int, block: int) -> None:
        """Entries of row `batch_idx` from column `block` on go to the device again at the next table sync."""
        synced = self._table_rows_synced[layer_idx]
        if synced is not None and batch_idx < len(synced) and synced[batch_idx] > block:
            synced[batch_idx] = block
            self._table_blocks_total[layer_idx] = -1
        self._table_view[layer_idx] = None

    def _privatize_last_block(self, layer_idx: int, batch_idx: int, key_states: torch.Tensor,
                              value_states: torch.Tensor) -> None:
        """Copy on first write for un-quantized pages: a cache made by ``clone`` maps the pages of its source.  Full
        blocks are never written again; the partly filled last block is, so the first append of either cache copies
        that one page and maps the copy."""
        length = self.layer_lengths[layer_idx][batch_idx]
        if length % self.block_size == 0:
            return
        table = self.page_tables[layer_idx][batch_idx]
        blk = length // self.block_size
        layer = self.allocator.layers[layer_idx]
        if blk >= len(table) or layer.page_owners(table[blk]) <= 1:
            return
        shared = table[blk]
        private = self.allocator.allocate(layer_idx, 1, key_template=key_states, value_template=value_states)[0]
        layer = self.allocator.layers[layer_idx]
        assert layer.key_pages is not None and layer.value_pages is not None
        layer.key_pages[private].copy_(layer.key_pages[shared])
        layer.value_pages[private].copy_(layer.value_pages[shared])
        table[blk] = private
        self.allocator.release_pages(layer_idx, [shared])
        self._resync_row_from(layer_idx, batch_idx, blk)

    def _device_lengths_of(self, layer_idx: int, batch_size: int, device: torch.device) -> _DeviceLengths:
        state = self._dev_lengths[layer_idx]
        if state is None or state.device != device or int(state.rows[0].shape[0]) != batch_size:
            state = self._dev_lengths[layer_idx] = _DeviceLengths(batch_size, device)
        return state

    def _launch_page_write(self, layer: Qwen3PagedLayerAllocator, key_states, value_states, table_dev, past,
                           past_dev: torch.Tensor | None = None, new_lengths_dev: torch.Tensor | None = None):
        key_states = key_states if key_states.stride(3) == 1 else key_states.contiguous()
        if value_states.stride() != key_states.stride():
            key_states, value_states = key_states.contiguous(), value_states.contiguous()
        device = key_states.device
        if device.type != "cuda":
            raise RuntimeError("anna_b200 caches live on a CUDA device; there is no CPU fallback for update().")
        batch, kv_heads, tokens, dim = (int(v) for v in key_states.shape)
        if past_dev is None:
            past_dev = MetadataUploader.for_device(device).upload([past])[0]
        assert layer.key_pages is not None and layer.value_pages is not None
        with on_device(device):
            _lib.check(_lib.lib().anna_paged_kv_write(
                ptr(key_states), ptr(value_states), key_states.stride(0), key_states.stride(1), key_states.stride(2),
                ptr(layer.key_pages), ptr(layer.value_pages), ptr(table_dev), table_dev.stride(0), ptr(past_dev),
                ptr(new_lengths_dev), batch, kv_heads, tokens, dim, self.block_size, layer.capacity(), int(table_dev.shape[1]),
                dtype_code(key_states.dtype), None, stream_ptr(device)), "anna_paged_kv_write")

    def _map_prefix_shared_blocks(self, key_states, value_states, layer_idx: int, batch_idx: int,
                                  append_length: int) -> list[tuple[int, int]]:
        """Prefix page sharing for a single-row prompt (ops.py:779-857): a full prompt block that another sequence
        already wrote is mapped by reference (retain, no write); every other block gets a page and, if it is a
        full prompt block touched for the first time, is registered for later sequences.  Returns the token ranges
        of this append that still have to be written."""
        prompt = self._prompt_token_ids
        assert prompt is not None
        current = self.layer_lengths[layer_idx][batch_idx]
        required = current + append_length
        table = self.page_tables[layer_idx][batch_idx]
        pool = self.allocator.prefix_block_pool
        bs = self.block_size
        pos = current
        segments: list[tuple[int, int]] = []
        while pos < required:
            blk = pos // bs
            hi = min(required, (blk + 1) * bs)
            full_block = (hi - pos) == bs and pos == blk * bs
            first_touch = len(table) <= blk
            hit = None
            if first_touch and full_block and hi <= len(prompt):
                hit = pool.lookup(layer_idx, tuple(prompt[pos:hi]))
            if first_touch:
                if hit is not None:
                    self.allocator.retain_shared_page(layer_idx, hit)
                    table.append(hit)
                else:
                    table.append(self.allocator.allocate(layer_idx, 1, key_template=key_states,
                                                         value_template=value_states)[0])
            page_id = table[blk]
            if not (full_block and hit is not None and page_id == hit):
                lo_rel, hi_rel = pos - current, hi - current
                if segments and segments[-1][1] == lo_rel:
                    segments[-1] = (segments[-1][0], hi_rel)
                else:
                    segments.append((lo_rel, hi_rel))
                if full_block and first_touch and hit is None and hi <= len(prompt):
                    pool.register(layer_idx, tuple(prompt[pos:hi]), page_id)
            pos = hi
        return segments

    # -- TurboQuant layers ----------------------------------------------------------------------------------------------

    def _tq_pool(self, layer_idx: int) -> TurboQuantLayerPool:
        return self.allocator.turboquant_layers[layer_idx]

    def _prefix_keys(self) -> list[tuple]:
        """One key per full block of the prompt: (block index, chained hash of all tokens up to its end, the block's
        own tokens).  Packed codes depend on the whole prefix (keys and values come out of causal layers), so the
        registry is keyed by the prefix, not by the block's tokens alone."""
        if self._prompt_prefix_keys is None:
            prompt, bs = self._prompt_token_ids or [], self.block_size
            keys, chain = [], 0
            for j in range(len(prompt) // bs):
                block = tuple(prompt[j * bs:(j + 1) * bs])
                chain = hash((chain, block))
                keys.append((j, chain, block))
            self._prompt_prefix_keys = keys
        return self._prompt_prefix_keys

    def _reserve_shared_packed_blocks(self, row: TurboQuantKVRow, pool: TurboQuantLayerPool, layer_idx: int,
                                      new_length: int) -> list[int]:
        """Single-row prompt path: like ``row._reserve_blocks`` but a block whose whole prompt prefix was packed by an
        earlier sequence is mapped by reference.  Returns the indices of the blocks mapped that way in this call."""
        row._privatize_partial_block(new_length)
        quantized = max(0, int(new_length) - row.residual_len)
        need = (quantized + pool.block_size - 1) // pool.block_size
        keys = self._prefix_keys()
        registry = self.allocator.packed_prefix_block_pool
        shared: list[int] = []
        table = row.block_table
        while len(table) < need:
            j = len(table)
            hit = None
            if j < len(keys) and (j + 1) * pool.block_size <= quantized:  # a full prompt block, packed by this call
                hit = registry.lookup(layer_idx, keys[j])
            if hit is not None:
                pool.retain_page(hit)
                table.append(hit)
                shared.append(j)
            else:
                table.extend(pool.allocate(1))
        return shared

    def _register_packed_blocks(self, row: TurboQuantKVRow, pool: TurboQuantLayerPool, layer_idx: int) -> None:
        """Offer every prompt block of the row that is completely packed by now to later sequences."""
        keys = self._prefix_keys()
        registry = self.allocator.packed_prefix_block_pool
        done = min(row.quantized_length // pool.block_size, len(keys), len(row.block_table))
        for j in range(self._packed_blocks_registered[layer_idx], done):
            registry.register(layer_idx, keys[j], row.block_table[j])
        self._packed_blocks_registered[layer_idx] = max(self._packed_blocks_registered[layer_idx], done)

    def _update_turboquant_layer(self, key_states, value_states, layer_idx: int, *, require_dense_cache: bool):
        batch_size, kv_heads, append_length, head_dim = (int(v) for v in key_states.shape)
        self._ensure_batch_size(batch_size)
        device = key_states.device
        pool = self._tq_pool(layer_idx)
        pool.configure(kv_heads=kv_heads, head_dim=head_dim, bits=self.kv_cache_quant_bits,
                       residual_len=self.kv_cache_residual_len, dtype=key_states.dtype, device=device)
        rows = self.turboquant_rows[layer_idx]
        past = list(self.layer_lengths[layer_idx])
        missing = sum(1 for row in rows if row is None)
        if missing:
            pool.ensure_slot_capacity(pool.slot_capacity() - len(pool.free_slots) + missing)
        use_prefix_share = self._prefix_kv_share and batch_size == 1 and self._prompt_token_ids is not None
        shared_blocks: list[int] = []
        for batch_idx in range(batch_size):
            row = rows[batch_idx]
            if row is None:
                row = TurboQuantKVRow(bits=self.kv_cache_quant_bits, residual_len=self.kv_cache_residual_len)
                row._bind(pool, kv_heads=kv_heads, head_dim=head_dim, dtype=key_states.dtype, device=device)
                rows[batch_idx] = row
            if use_prefix_share:
                shared_blocks = self._reserve_shared_packed_blocks(row, pool, layer_idx, row.length + append_length)
            else:
                row._reserve_blocks(row.length + append_length)
            if row._privatized_block is not None:  # copy on write replaced a page id: upload that entry again
                self._resync_row_from(layer_idx, batch_idx, row._privatized_block)
                row._privatized_block = None
        slots = [row.slot for row in rows]
        lengths = self.layer_lengths[layer_idx]
        for batch_idx, row in enumerate(rows):
            row._length += append_length
            lengths[batch_idx] = row._length
        if device.type == "cuda":
            state = self._device_lengths_of(layer_idx, batch_size, device)
            past_lengths, new_lengths = state.before_append(past)
            slots_dev = state.slots(slots)
        else:  # bookkeeping only (the launch below refuses CPU tensors)
            state, slots_dev, new_lengths = None, None, None
            past_lengths = torch.tensor(past, device=device, dtype=torch.long)
        if append_length > 0:
            table_dev = self._sync_page_table_layer_buffer(layer_idx, batch_size=batch_size, device=device)
            mask_dev = None
            if shared_blocks and table_dev is not None:
                words = np.zeros((1, (int(table_dev.shape[1]) + 31) // 32), dtype=np.uint32)
                for j in shared_blocks:
                    words[0, j >> 5] |= np.uint32(1 << (j & 31))
                mask_dev = torch.from_numpy(words.view(np.int32)).to(device)
            launch_tq_append(pool, key_states, value_states, table_dev, slots, past, slots_dev=slots_dev,
                             past_dev=past_lengths if state is not None else None, new_lengths_dev=new_lengths,
                             shared_blocks=mask_dev)
            if state is not None:
                state.after_append(lengths)
            if use_prefix_share:
                self._register_packed_blocks(rows[0], pool, layer_idx)
        self.seen_tokens = max(self.seen_tokens, max(lengths, default=0))
        if not require_dense_cache:
            return None, None, past_lengths
        keys, values, _ = self._gather_layer_cache(layer_idx)
        return keys, values, past_lengths

    def turboquant_single_token_decode_attention(self, layer_idx: int, query_states: torch.Tensor, *, scaling: float,
                                                 num_key_value_groups: int, gate: torch.Tensor | None = None,
                                                 output: torch.Tensor | None = None,
                                                 peer_outputs: tuple[int, ...] = ()):
        """One launch pair for the whole batch (ops.py:1024-1070 loops over rows).  ``output`` / ``peer_outputs``: see
        ``launch_tq_decode`` (not part of the reference's signature; used by the KV-head-sharded layout)."""
        if not self.uses_turboquant_for_layer(layer_idx):
            raise ValueError(f"Layer {layer_idx} does not use TurboQuant-backed KV storage.")
        if query_states.ndim != 4 or query_states.shape[2] != 1:
            raise ValueError("TurboQuant decode attention expects query_states shaped [batch, query_heads, 1, head_dim].")
        if gate is not None and gate.shape != query_states.shape:
            raise ValueError(
                f"TurboQuant decode gate expects query layout {tuple(query_states.shape)}, got {tuple(gate.shape)}.")
        batch = int(query_states.shape[0])
        rows = self.turboquant_rows[layer_idx]
        if batch != len(rows):
            raise ValueError(f"Cache batch size mismatch: expected {len(rows)}, got {batch}")
        pool = self._tq_pool(layer_idx)
        if not pool.configured or all(row is None or row.length <= 0 for row in rows):
            if output is not None or peer_outputs:
                raise RuntimeError("an empty TurboQuant cache cannot decode into caller-provided outputs")
            return query_states.new_zeros(query_states.shape)
        if int(query_states.shape[1]) != pool.kv_heads * num_key_value_groups:
            raise ValueError(
                f"Expected {pool.kv_heads * num_key_value_groups} query heads, got {int(query_states.shape[1])}.")
        device = query_states.device
        table_dev = self._sync_page_table_layer_buffer(layer_idx, batch_size=batch, device=device)
        lengths = [0 if row is None else row.length for row in rows]
        slots = [0 if row is None else row.slot for row in rows]
        state = self._dev_lengths[layer_idx]
        lengths_dev = slots_dev = None
        if state is not None and state.device == device:
            lengths_dev = state.current(lengths)
            slots_dev = state.slots(slots)
        return launch_tq_decode(pool, query_states, table_dev, slots, lengths, scaling, gate, slots_dev=slots_dev,
                                lengths_dev=lengths_dev, output=output, peer_outputs=peer_outputs)

    # -- dense views -------------------------------------------------------------------------------------------------------

    def paged_attention_state(self, layer_idx: int):
        """``(key_pages, value_pages, page_table, visible_lengths)`` for the paged decode op (ops.py:899-929)."""
        if self.uses_turboquant_for_layer(layer_idx):
            return None
        batch_size = self.get_batch_size()
        if batch_size == 0:
            return None
        layer = self.allocator.layers[layer_idx]
        if layer.key_pages is None or layer.value_pages is None:
            return None
        lengths = self.layer_lengths[layer_idx]
        required = max((len(t) for t in self.page_tables[layer_idx]), default=0)
        if required <= 0 or max(lengths, default=0) <= 0:
            return None
        device = layer.key_pages.device
        page_table = self._table_view[layer_idx]
        if page_table is None or page_table.device != device:
            page_table = self._sync_page_table_layer_buffer(layer_idx, batch_size=batch_size, device=device)
            if page_table is None:
                return None
            if self._page_headroom[layer_idx] is not None:  # tables are known not to change before the next append
                self._table_view[layer_idx] = page_table
        state = self._dev_lengths[layer_idx]
        visible_lengths = None if state is None or state.device != device else state.current(lengths)
        if visible_lengths is None:
            visible_lengths = torch.tensor(lengths, dtype=torch.long, device=device)
        return layer.key_pages, layer.value_pages, page_table, visible_lengths

    def _gather_layer_cache(self, layer_idx: int):
        """Dense ``[B, Hkv, Lmax, D]`` keys / values, zero padded, plus visible lengths (ops.py:931-1006)."""
        batch_size = self.get_batch_size()
        if batch_size == 0:
            return None, None, torch.zeros(0, dtype=torch.long)
        lengths = self.layer_lengths[layer_idx]
        max_length = max(lengths, default=0)
        if self.uses_turboquant_for_layer(layer_idx):
            if max_length <= 0:
                return None, None, torch.tensor(lengths, dtype=torch.long)
            rows = self.turboquant_rows[layer_idx]
            if any(row is None for row in rows):
                raise RuntimeError(f"TurboQuant cache row for layer {layer_idx} is missing.")
            pool = self._tq_pool(layer_idx)
            device = pool.device
            assert device is not None
            table_dev = self._sync_page_table_layer_buffer(layer_idx, batch_size=batch_size, device=device)
            # the lengths come back as the device tensor the launch read them from (no second host-to-device copy)
            return launch_tq_gather_dense(pool, table_dev, [row.slot for row in rows], list(lengths), max_length)
        layer = self.allocator.layers[layer_idx]
        if layer.key_pages is None or layer.value_pages is None or max_length <= 0:
            return None, None, torch.tensor(lengths, dtype=torch.long)
        device = layer.key_pages.device
        table = self._sync_page_table_layer_buffer(layer_idx, batch_size=batch_size, device=device)
        visible = torch.tensor(lengths, dtype=torch.long, device=device)
        if table is None:
            return None, None, visible
        keys = torch.empty((batch_size, int(layer.key_pages.shape[1]), max_length, int(layer.key_pages.shape[3])),
                           dtype=layer.key_pages.dtype, device=device)
        values = torch.empty_like(keys)
        with on_device(device):
            _lib.check(_lib.lib().anna_paged_kv_gather(
                ptr(layer.key_pages), ptr(layer.value_pages), ptr(table), table.stride(0), ptr(visible), ptr(keys),
                ptr(values), keys.stride(0), keys.stride(1), keys.stride(2), batch_size, int(keys.shape[1]),
                int(keys.shape[3]), self.block_size, layer.capacity(), int(table.shape[1]), max_length,
                dtype_code(keys.dtype), stream_ptr(device)), "anna_paged_kv_gather")
        return keys, values, visible

    def visible_key_cache(self, layer_idx: int):
        return self._gather_layer_cache(layer_idx)[0]

    def visible_value_cache(self, layer_idx: int):
        return self._gather_layer_cache(layer_idx)[1]

    # -- batch membership (ops.py:1072-1321) -------------------------------------------------------------------------------

    def _new_like(self, batch_size: int) -> "Qwen3DynamicCache":
        return Qwen3DynamicCache(self.config, allocator=self.allocator, batch_size=batch_size,
                                 kv_cache_quantization=self.kv_cache_quantization,
                                 kv_cache_quant_bits=self.kv_cache_quant_bits,
                                 kv_cache_residual_len=self.kv_cache_residual_len)

    @classmethod
    def stack(cls, caches: list["Qwen3DynamicCache"], config, *, clone_turboquant_rows: bool = True):
        if not caches:
            return cls(config)
        if any(cache.allocator is not caches[0].allocator for cache in caches):
            raise ValueError("Cannot stack caches from different allocators.")
        rows: list[Qwen3DynamicCache] = []
        for cache in caches:
            rows.extend([cache] if cache.get_batch_size() <= 1 else cache.split_batch())
        stacked = rows[0]._new_like(len(rows))
        layers = config.num_hidden_layers
        for layer_idx in range(layers):
            stacked.layer_lengths[layer_idx] = [row.layer_lengths[layer_idx][0] for row in rows]
        stacked.seen_tokens = max(stacked.get_seq_lengths().tolist(), default=0)
        stacked.rope_deltas = None if rows[0].rope_deltas is None else torch.cat([r.rope_deltas for r in rows], dim=0)
        stacked.reserved_seq_capacity = max((row.reserved_seq_capacity for row in rows), default=0)
        for layer_idx in range(layers):
            if stacked.uses_turboquant_for_layer(layer_idx):
                for batch_idx, row in enumerate(rows):
                    tq_row = row.turboquant_rows[layer_idx][0]
                    stacked.turboquant_rows[layer_idx][batch_idx] = (
                        None if tq_row is None else (tq_row.clone() if clone_turboquant_rows else tq_row))
                continue
            stacked.page_tables[layer_idx] = [list(row.page_tables[layer_idx][0]) for row in rows]
            for name in ("conv_states", "recurrent_states"):
                states = [getattr(row, name)[layer_idx] for row in rows]
                if all(state is None for state in states):
                    continue
                if any(state is None for state in states):
                    raise ValueError(f"Cannot stack partially initialized {name} at layer {layer_idx}")
                getattr(stacked, name)[layer_idx] = torch.cat(states, dim=0)
        return stacked

    def split_batch(self, *, clone_turboquant_rows: bool = True) -> list["Qwen3DynamicCache"]:
        batch_size = self.get_batch_size()
        if batch_size <= 1:
            return [self]
        outputs = [self._new_like(1) for _ in range(batch_size)]
        layers = self.config.num_hidden_layers
        for batch_idx, cache in enumerate(outputs):
            for layer_idx in range(layers):
                cache.layer_lengths[layer_idx][0] = self.layer_lengths[layer_idx][batch_idx]
            cache.seen_tokens = cache.get_seq_length()
            cache.reserved_seq_capacity = self.reserved_seq_capacity
        if self.rope_deltas is not None:
            for idx, chunk in enumerate(self.rope_deltas.split(1, dim=0)):
                outputs[idx].rope_deltas = chunk
        for layer_idx in range(layers):
            for idx in range(batch_size):
                outputs[idx].page_tables[layer_idx][0] = list(self.page_tables[layer_idx][idx])
                tq_row = self.turboquant_rows[layer_idx][idx]
                if tq_row is not None:
                    outputs[idx].turboquant_rows[layer_idx][0] = tq_row.clone() if clone_turboquant_rows else tq_row
            for name in ("conv_states", "recurrent_states"):
                state = getattr(self, name)[layer_idx]
                if state is not None:
                    for idx, chunk in enumerate(state.split(1, dim=0)):
                        getattr(outputs[idx], name)[layer_idx] = chunk.clone()
        return outputs

    def compact_batch_rows(self, row_indices, *, release_unselected: bool = True) -> "Qwen3DynamicCache":
        """Move the selected rows into a smaller cache; dropped rows give their pages back (ops.py:1220-1321)."""
        batch_size = self.get_batch_size()
        rows = [int(idx) for idx in row_indices]
        if not rows:
            self.release()
            return self._new_like(0)
        if len(set(rows)) != len(rows):
            raise ValueError("compact_batch_rows requires unique row indices.")
        if any(idx < 0 or idx >= batch_size for idx in rows):
            raise IndexError(f"compact_batch_rows row indices out of range for batch size {batch_size}: {rows}")
        if rows == list(range(batch_size)):
            return self
        selected = set(rows)
        compacted = self._new_like(len(rows))
        compacted.reserved_seq_capacity = self.reserved_seq_capacity
        if self.rope_deltas is not None:
            index = torch.tensor(rows, device=self.rope_deltas.device, dtype=torch.long)
            compacted.rope_deltas = self.rope_deltas.index_select(0, index)
        for layer_idx in range(self.config.num_hidden_layers):
            compacted.layer_lengths[layer_idx] = [self.layer_lengths[layer_idx][idx] for idx in rows]
            if self.uses_turboquant_for_layer(layer_idx):
                for new_idx, old_idx in enumerate(rows):
                    compacted.turboquant_rows[layer_idx][new_idx] = self.turboquant_rows[layer_idx][old_idx]
                if release_unselected:
                    for old_idx in range(batch_size):
                        row = self.turboquant_rows[layer_idx][old_idx]
                        if old_idx not in selected and row is not None:
                            row.release()
            else:
                for new_idx, old_idx in enumerate(rows):
                    compacted.page_tables[layer_idx][new_idx] = list(self.page_tables[layer_idx][old_idx])
                if release_unselected:
                    for old_idx, page_ids in enumerate(self.page_tables[layer_idx]):
                        if old_idx not in selected:
                            self.allocator.release_pages(layer_idx, page_ids)
            for name in ("conv_states", "recurrent_states"):
                state = getattr(self, name)[layer_idx]
                if state is not None:
                    index = torch.tensor(rows, device=state.device, dtype=torch.long)
                    getattr(compacted, name)[layer_idx] = state.index_select(0, index)
        compacted.seen_tokens = max(compacted.get_seq_lengths().tolist(), default=0)
        self._forget_rows()
        return compacted

    def _forget_rows(self) -> None:
        batch_size = self.get_batch_size()
        self._prefill_input_ids = None
        self._prompt_token_ids = None
        self._prompt_prefix_keys = None
        self._packed_blocks_registered = [0] * self.config.num_hidden_layers
        for layer_idx in range(self.config.num_hidden_layers):
            self.layer_lengths[layer_idx] = [0] * batch_size
            self.page_tables[layer_idx] = [[] for _ in range(batch_size)]
            self.turboquant_rows[layer_idx] = [None] * batch_size
            self.conv_states[layer_idx] = None
            self.recurrent_states[layer_idx] = None
            self.page_table_caches[layer_idx] = None
            self.page_table_capacities[layer_idx] = 0
            self._table_rows_synced[layer_idx] = None
            self._table_host[layer_idx] = None
            self._table_blocks_total[layer_idx] = -1
            self._dev_lengths[layer_idx] = None
            self._page_headroom[layer_idx] = None
            self._table_view[layer_idx] = None
        self.seen_tokens = 0
        self.rope_deltas = None
        self.reserved_seq_capacity = 0
        self._released = True

    def clone(self) -> "Qwen3DynamicCache":
        """An independent copy of the cache state (ops.py:1323-1381) that copies no page: un-quantized and packed pages
        get one more owner each and are mapped by both caches; only window rings are duplicated.  The first append of
        either cache into a partly filled last block copies that one page (copy on first write)."""
        batch_size = self.get_batch_size()
        cloned = self._new_like(batch_size)
        for layer_idx in range(self.config.num_hidden_layers):
            cloned.layer_lengths[layer_idx] = list(self.layer_lengths[layer_idx])
        cloned.seen_tokens = self.seen_tokens
        cloned.reserved_seq_capacity = self.reserved_seq_capacity
        if self.rope_deltas is not None:
            cloned.rope_deltas = self.rope_deltas.clone()
        for layer_idx in range(self.config.num_hidden_layers):
            for name in ("conv_states", "recurrent_states"):
                state = getattr(self, name)[layer_idx]
                if state is not None:
                    getattr(cloned, name)[layer_idx] = state.clone()
            for batch_idx, row in enumerate(self.turboquant_rows[layer_idx]):
                if row is not None:
                    cloned.turboquant_rows[layer_idx][batch_idx] = row.clone()
            if self.uses_turboquant_for_layer(layer_idx):
                continue
            for batch_idx, page_ids in enumerate(self.page_tables[layer_idx]):
                for page_id in page_ids:
                    self.allocator.retain_shared_page(layer_idx, page_id)
                cloned.page_tables[layer_idx][batch_idx] = list(page_ids)
            # both caches now have to look at their last blocks before the next append
            self._page_headroom[layer_idx] = None
        if self._prompt_token_ids is not None:
            cloned._prompt_token_ids = list(self._prompt_token_ids)
        return cloned

    def release(self) -> None:
        """Give every page and window ring of this cache back to the allocator (ops.py:1383-1410)."""
        if self._released:
            return
        for layer_idx in range(self.config.num_hidden_layers):
            if self.uses_turboquant_for_layer(layer_idx):
                for row in self.turboquant_rows[layer_idx]:
                    if row is not None:
                        row.release()
            else:
                for page_ids in self.page_tables[layer_idx]:
                    self.allocator.release_pages(layer_idx, page_ids)
        self._forget_rows()

    def to(self, *, device: torch.device | None = None, dtype: torch.dtype | None = None) -> "Qwen3DynamicCache":
        def move(tensor):
            if tensor is None:
                return None
            kwargs = {}
            if device is not None:
                kwargs["device"] = device
            if dtype is not None and tensor.is_floating_point():
                kwargs["dtype"] = dtype
            return tensor.to(**kwargs) if kwargs else tensor

        self.conv_states = [move(t) for t in self.conv_states]
        self.recurrent_states = [move(t) for t in self.recurrent_states]
        self.rope_deltas = move(self.rope_deltas)
        if device is not None and torch.device(device).type != "cuda":
            raise RuntimeError("anna_b200 caches cannot leave the GPU: there is no CPU implementation of this path.")
        return self
