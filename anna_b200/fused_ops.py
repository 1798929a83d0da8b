"""Operator boundary of the decode path: the ``run_*`` wrappers and ``torch.ops.anna.*`` schemas of Anna.

Mirrors the decode part of ``src/anna/model/fused_ops.py`` (:306-323 availability probes, :414-448 library loading,
:451-609 wrappers) and the schemas the reference registers in
``src/anna/model/custom_ops/gated_delta_fused_op.sycl:7621-7679``; here they are registered for the CUDA dispatch
key and forward to the C ABI of ``libanna_b200_kv.so`` with raw pointers on the current CUDA stream.  As in the
reference there is no CPU fallback: a missing library or op raises ``RuntimeError``.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

from . import _lib

_LOAD_LOCK = threading.Lock()
_REGISTERED = False
_LIBRARY: torch.library.Library | None = None
_LOADED_LIBRARIES: set[str] = set()

_DTYPE_CODES = {torch.float32: _lib.DTYPE_F32, torch.float16: _lib.DTYPE_F16, torch.bfloat16: _lib.DTYPE_BF16}

SCHEMAS = {
    "gqa_decode_fused":
        "(Tensor query, Tensor key, Tensor value, Tensor visible_lengths, float scaling, Tensor? gate=None) -> Tensor",
    "gqa_decode_splitkv_fused":
        "(Tensor query, Tensor key, Tensor value, float scaling, int block_size, Tensor? gate=None) -> Tensor",
    "gqa_decode_splitkv_fused_out":
        "(Tensor query, Tensor key, Tensor value, Tensor(a!) output, Tensor(b!) partial_stats, "
        "Tensor(c!) partial_values, float scaling, int block_size, Tensor? gate=None) -> Tensor(a!)",
    "gqa_decode_splitkv_turboquant_fused_out":
        "(Tensor query, Tensor quantized_key, Tensor value_data, Tensor value_scales, Tensor value_zeros, "
        "Tensor residual_key, Tensor residual_value, Tensor(a!) output, Tensor(b!) partial_stats, "
        "Tensor(c!) partial_values, float scaling, int value_bits, int value_group_size, int block_size, "
        "Tensor? gate=None) -> Tensor(a!)",
    "paged_gqa_decode_fused":
        "(Tensor query, Tensor key_pages, Tensor value_pages, Tensor page_table, Tensor visible_lengths, "
        "float scaling, Tensor? gate=None) -> Tensor",
}

# Ops for the steps that are Python loops in the reference and kernels here: the page write of un-quantized layers
# (Qwen3DynamicCache._write_pages, src/anna/model/ops.py:748-777), the fused TurboQuant append (TurboQuantKVRow.append,
# src/anna/model/turboquant.py:1027-1140) and the decode over packed pages (turboquant.py:1181-1293).  They sit in the
# same namespace as the five schemas above, which stay what the reference registers (gated_delta_fused_op.sycl:7621-7679).
NEW_SCHEMAS = {
    "paged_kv_write":
        "(Tensor key_states, Tensor value_states, Tensor(a!) key_pages, Tensor(b!) value_pages, Tensor page_table, "
        "Tensor past_lengths) -> ()",
    "tq_append":
        "(Tensor key_states, Tensor value_states, Tensor(a!) packed_pages, Tensor page_table, Tensor(b!) window, "
        "Tensor window_slots, Tensor past_lengths, int bits, int residual_len, int block_size, int value_group_size) "
        "-> ()",
    "tq_paged_decode":
        "(Tensor query, Tensor packed_pages, Tensor page_table, Tensor window, Tensor window_slots, Tensor lengths, "
        "float scaling, int bits, int residual_len, int block_size, int value_group_size, Tensor? gate=None) -> Tensor",
}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODES[dtype]
    except KeyError:
        raise RuntimeError(f"anna_b200 kernels support float16, bfloat16 and float32 inputs, got {dtype}") from None


def ptr(tensor: torch.Tensor | None) -> int | None:
    """Device address for a ``void*`` argument (ctypes turns an int into the pointer, None into NULL)."""
    return None if tensor is None else tensor.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device: torch.device) -> int | None:
    """Handle of the current CUDA stream of ``device`` (None = the legacy default stream)."""
    index = device.index
    if index is None:
        index = torch.cuda.current_device()
    handle = _raw_stream(index) if _raw_stream is not None else torch.cuda.current_stream(device).cuda_stream
    return handle or None


class on_device:
    """``with on_device(dev):`` makes ``dev`` the current CUDA device, skipping the switch when it already is."""

    __slots__ = ("index", "previous")

    def __init__(self, device: torch.device) -> None:
        self.index = device.index if device.index is not None else torch.cuda.current_device()
        self.previous = -1

    def __enter__(self) -> None:
        current = torch.cuda.current_device()
        if current != self.index:
            self.previous = current
            torch.cuda.set_device(self.index)

    def __exit__(self, *exc) -> None:
        if self.previous >= 0:
            torch.cuda.set_device(self.previous)


class MetadataUploader:
    """Small per-step integer metadata (lengths, ring slots) goes to the GPU through a ring of pinned host buffers
    with one asynchronous copy per call, instead of a synchronous ``torch.tensor(list, device=...)`` per array."""

    _instances: dict[int, "MetadataUploader"] = {}

    def __init__(self, device: torch.device, slots: int = 16) -> None:
        self.device = device
        self.slots = slots
        self.capacity = 0
        self.buffers: list[torch.Tensor] = []
        self.views: list = []
        self.events: list[torch.cuda.Event | None] = []
        self.next = 0

    @classmethod
    def for_device(cls, device: torch.device) -> "MetadataUploader":
        index = device.index if device.index is not None else torch.cuda.current_device()
        inst = cls._instances.get(index)
        if inst is None:
            inst = cls._instances[index] = cls(torch.device("cuda", index))
        return inst

    def _ensure(self, count: int) -> None:
        if count <= self.capacity:
            return
        self.capacity = max(1024, 2 * count)
        self.buffers = [torch.empty(self.capacity, dtype=torch.int64).pin_memory() for _ in range(self.slots)]
        self.views = [buf.numpy() for buf in self.buffers]
        self.events = [None] * self.slots

    def upload(self, rows: list[list[int]]) -> torch.Tensor:
        """int64 [len(rows), len(rows[0])] on the device; the copy is ordered on the current stream."""
        width = len(rows[0])
        count = len(rows) * width
        self._ensure(count)
        slot = self.next
        self.next = (slot + 1) % self.slots
        event = self.events[slot]
        if event is not None:
            event.synchronize()  # the previous copy out of this buffer has finished (normally long ago)
        view = self.views[slot]
        for idx, row in enumerate(rows):
            view[idx * width:(idx + 1) * width] = row
        out = torch.empty((len(rows), width), dtype=torch.int64, device=self.device)
        out.view(-1).copy_(self.buffers[slot][:count], non_blocking=True)
        if event is None:
            event = self.events[slot] = torch.cuda.Event()
        event.record()
        return out

    def upload_i32(self, values) -> torch.Tensor:
        """int32 copy of a flat numpy int32 array on the device, through the same pinned ring."""
        count = int(values.size)
        self._ensure((count + 1) // 2)
        slot = self.next
        self.next = (slot + 1) % self.slots
        event = self.events[slot]
        if event is not None:
            event.synchronize()
        staging = self.buffers[slot].view(torch.int32)
        staging.numpy()[:count] = values
        out = torch.empty(count, dtype=torch.int32, device=self.device)
        out.copy_(staging[:count], non_blocking=True)
        if event is None:
            event = self.events[slot] = torch.cuda.Event()
        event.record()
        return out


def _require_cuda(name: str, **tensors: torch.Tensor | None) -> torch.device:
    device = None
    for label, tensor in tensors.items():
        if tensor is None:
            continue
        if not tensor.is_cuda:
            raise RuntimeError(f"{name}: {label} must be a CUDA tensor (there is no CPU implementation of this op)")
        if device is None:
            device = tensor.device
        elif tensor.device != device:
            raise RuntimeError(f"{name}: {label} must be on the same device as query")
    assert device is not None
    return device


def _last_dim_contiguous(tensor: torch.Tensor) -> torch.Tensor:
    return tensor if tensor.stride(-1) == 1 else tensor.contiguous()


def _check_gate(name: str, query: torch.Tensor, gate: torch.Tensor | None):
    """Validates like validate_gqa_decode_optional_gate (.sycl:1605-1626); returns (tensor, stride_b, stride_h)."""
    if gate is None:
        return None, 0, 0
    heads, dim = int(query.shape[1]), int(query.shape[3])
    if gate.dtype != query.dtype:
        raise RuntimeError("gate must match query dtype")
    if gate.shape[0] != query.shape[0]:
        raise RuntimeError("gate batch size mismatch")
    if gate.dim() == 3:
        if gate.shape[1] != 1 or gate.shape[2] != heads * dim:
            raise RuntimeError("3D gqa_decode gate must be [batch, 1, num_heads * head_dim]")
        gate = _last_dim_contiguous(gate)
        return gate, gate.stride(0), dim
    if gate.dim() == 4:
        if gate.shape[1] != heads or gate.shape[2] != 1 or gate.shape[3] != dim:
            raise RuntimeError("4D gqa_decode gate must match query layout [batch, heads, 1, head_dim]")
        gate = _last_dim_contiguous(gate)
        return gate, gate.stride(0), gate.stride(1)
    raise RuntimeError(
        "gqa_decode gate must be 3D [batch, 1, num_heads * head_dim] or 4D [batch, heads, 1, head_dim] (query layout)")


def _check_query(name: str, query: torch.Tensor) -> torch.Tensor:
    if query.dim() != 4 or query.shape[2] != 1:
        raise RuntimeError(f"{name}: query must be [batch, heads, 1, head_dim] (single-token query)")
    return _last_dim_contiguous(query)


class _Scratch:
    """Per-(device, stream) split-K scratch, grown on demand and reused across calls.

    Holds the float partial buffers and the int32 arrival counters of the fused merge.  The counters are zeroed when
    they are allocated and are left at zero by every launch, so they are never cleared again."""

    def __init__(self) -> None:
        self._buffers: dict[tuple[int, int], torch.Tensor] = {}
        self._counters: dict[tuple[int, int], torch.Tensor] = {}
        self._byte_buffers: dict[tuple[int, int], torch.Tensor] = {}

    @staticmethod
    def _key(device: torch.device) -> tuple[int, int]:
        return (device.index if device.index is not None else torch.cuda.current_device(),
                stream_ptr(device) or 0)

    def get(self, device: torch.device, floats: int) -> torch.Tensor:
        key = self._key(device)
        buf = self._buffers.get(key)
        if buf is None or buf.numel() < floats:
            buf = torch.empty(max(floats, 1 << 16), dtype=torch.float32, device=device)
            self._buffers[key] = buf
            _SPLIT_CACHE.clear()  # cached views point into the old buffer
        return buf

    def bytes(self, device: torch.device, count: int) -> torch.Tensor:
        key = self._key(device)
        buf = self._byte_buffers.get(key)
        if buf is None or buf.numel() < count:
            buf = torch.empty(max(count, 1 << 20), dtype=torch.uint8, device=device)
            self._byte_buffers[key] = buf
        return buf

    def counters(self, device: torch.device, count: int) -> torch.Tensor:
        key = self._key(device)
        buf = self._counters.get(key)
        if buf is None or buf.numel() < count:
            buf = torch.zeros(max(count, 4096), dtype=torch.int32, device=device)
            self._counters[key] = buf
            _SPLIT_CACHE.clear()
        return buf


_SPLIT_CACHE: dict[tuple, tuple] = {}  # split_scratch results by problem shape, device and stream
_SCRATCH = _Scratch()


def query_scratch(device: torch.device, batch: int, heads: int, kv_heads: int, head_dim: int) -> torch.Tensor:
    """Scratch for the rotated query fragments of the packed tensor-core decode."""
    need = int(_lib.lib().anna_tq_query_scratch_bytes(batch, heads, kv_heads, head_dim))
    return _SCRATCH.bytes(device, need)


_PLAN_CACHE: dict[tuple, int] = {}


def split_scratch(device: torch.device, batch: int, heads: int, head_dim: int, kv_heads: int, max_len: int,
                  *, turboquant: tuple[int, int, int] | None = None):
    """(partial_stats, partial_values, chunk_capacity, counters) sized by the library's own plan for this problem.

    ``turboquant=(max_blocks, block_size, residual_len)`` selects the plan of the packed decode (window chunks +
    packed chunks) instead of the plan for ``max_len`` tokens."""
    cache_key = (device.index, stream_ptr(device), batch, heads, head_dim, kv_heads, max_len, turboquant)
    hit = _SPLIT_CACHE.get(cache_key)
    if hit is not None:
        return hit
    key = (batch, kv_heads, int(max_len), turboquant)
    chunks = _PLAN_CACHE.get(key)
    if chunks is None:
        if turboquant is None:
            _, chunks = _lib.decode_plan(batch, kv_heads, max(int(max_len), 1))
        else:
            _, chunks = _lib.tq_decode_plan(batch, kv_heads, *turboquant)
        if len(_PLAN_CACHE) > 4096:
            _PLAN_CACHE.clear()
        _PLAN_CACHE[key] = chunks
    stats_floats = (batch * heads * chunks * 2 + 3) // 4 * 4  # keeps the value partials 16-byte aligned
    value_floats = batch * heads * chunks * head_dim
    buf = _SCRATCH.get(device, stats_floats + value_floats)
    group_tiles = (heads // kv_heads + 7) // 8
    counters = _SCRATCH.counters(device, 2 * batch * kv_heads * group_tiles)  # arrival counters + tile cursors
    if len(_SPLIT_CACHE) > 256:
        _SPLIT_CACHE.clear()
    result = (buf[:batch * heads * chunks * 2], buf[stats_floats:stats_floats + value_floats], chunks, counters)
    _SPLIT_CACHE[cache_key] = result
    return result


# ---------------------------------------------------------------------------------------------------------------
# op implementations (CUDA dispatch key)


def _gqa_decode_dense(name, query, key, value, visible_lengths, scaling, gate, *, output=None, partial_stats=None,
                      partial_values=None, block_size=0):
    query = _check_query(name, query)
    if key.dim() != 4 or value.dim() != 4:
        raise RuntimeError(f"{name}: key and value must be [batch, kv_heads, key_len, head_dim]")
    if key.shape != value.shape:
        raise RuntimeError("key and value must share the same shape")
    if query.shape[0] != key.shape[0]:
        raise RuntimeError("query/key batch size mismatch")
    if query.shape[3] != key.shape[3]:
        raise RuntimeError("query/key head_dim mismatch")
    if key.shape[1] < 1 or query.shape[1] % key.shape[1] != 0:
        raise RuntimeError("query heads must be divisible by kv_heads")
    if key.shape[2] < 1:
        raise RuntimeError("key_len must be positive")
    if not (query.dtype == key.dtype == value.dtype):
        raise RuntimeError("query, key, and value must share the same dtype")
    device = _require_cuda(name, query=query, key=key, value=value, visible_lengths=visible_lengths, gate=gate)
    if visible_lengths is not None:
        if visible_lengths.dim() != 1 or visible_lengths.shape[0] != query.shape[0]:
            raise RuntimeError("visible_lengths must be [batch]")
        if visible_lengths.dtype != torch.long:
            raise RuntimeError("visible_lengths must be int64")
        visible_lengths = visible_lengths.contiguous()
    key = _last_dim_contiguous(key)
    value = _last_dim_contiguous(value)
    if value.stride() != key.stride():
        value = value.contiguous()
        key = key.contiguous()
    gate, gate_sb, gate_sh = _check_gate(name, query, gate)
    batch, heads, _, dim = (int(v) for v in query.shape)
    kv_heads, key_len = int(key.shape[1]), int(key.shape[2])
    result = output if output is not None else torch.empty((batch, heads, 1, dim), dtype=query.dtype, device=device)
    target = result if result.stride(3) == 1 else torch.empty((batch, heads, 1, dim), dtype=query.dtype, device=device)
    if partial_stats is None:
        partial_stats, partial_values, capacity, counters = split_scratch(device, batch, heads, dim, kv_heads, key_len)
        chunk_tokens = 0
    else:
        capacity = int(partial_stats.shape[2])
        chunk_tokens = min(max(int(block_size), 16), key_len)
        counters = None
    with on_device(device):
        _lib.check(_lib.lib().anna_gqa_decode(
            ptr(query), query.stride(0), query.stride(1), ptr(key), ptr(value), key.stride(0), key.stride(1),
            key.stride(2), ptr(visible_lengths), ptr(gate), gate_sb, gate_sh, ptr(target), target.stride(0),
            target.stride(1), ptr(partial_stats), ptr(partial_values), capacity, chunk_tokens, ptr(counters), batch,
            heads, kv_heads, key_len, dim, float(scaling), dtype_code(query.dtype), stream_ptr(device)), name)
    if target is not result:
        result.copy_(target)
    return result


def _op_gqa_decode_fused(query, key, value, visible_lengths, scaling, gate=None):
    if visible_lengths is None:
        raise RuntimeError("visible_lengths must be [batch]")
    return _gqa_decode_dense("gqa_decode_fused", query, key, value, visible_lengths, scaling, gate)


def _op_gqa_decode_splitkv_fused(query, key, value, scaling, block_size, gate=None):
    if block_size < 16:
        raise RuntimeError("gqa_decode_splitkv_fused block_size must be at least 16")
    return _gqa_decode_dense("gqa_decode_splitkv_fused", query, key, value, None, scaling, gate)


def _check_split_workspace(name, query, key_len, block_size, output, partial_stats, partial_values):
    """validate_gqa_decode_splitkv_workspace_for_length (.sycl:1521-1556)."""
    batch, heads, _, dim = (int(v) for v in query.shape)
    effective = min(max(int(block_size), 16), int(key_len))
    blocks = (int(key_len) + effective - 1) // effective
    if tuple(output.shape) != tuple(query.shape) or output.dtype != query.dtype or output.device != query.device:
        raise RuntimeError(f"{name} output must match query shape, dtype and device")
    for label, tensor, last in (("partial_stats", partial_stats, 2), ("partial_values", partial_values, dim)):
        if tensor.dim() != 4 or tensor.dtype != torch.float32 or tensor.device != query.device:
            raise RuntimeError(f"{name} {label} must be a float32 [batch, heads, blocks, {last}] tensor on the query device")
        if tensor.shape[0] != batch or tensor.shape[1] != heads or tensor.shape[2] < blocks or tensor.shape[3] != last:
            raise RuntimeError(f"{name} {label} shape/capacity mismatch")
        if not tensor.is_contiguous():
            raise RuntimeError(f"{name} {label} must be contiguous")
    if partial_stats.shape[2] != partial_values.shape[2]:
        raise RuntimeError(f"{name} partial_stats and partial_values must hold the same number of blocks")


def _op_gqa_decode_splitkv_fused_out(query, key, value, output, partial_stats, partial_values, scaling, block_size,
                                     gate=None):
    name = "gqa_decode_splitkv_fused_out"
    if block_size < 16:
        raise RuntimeError(f"{name} block_size must be at least 16")
    if query.dim() != 4 or key.dim() != 4:
        raise RuntimeError(f"{name}: query and key must be 4-D")
    _check_split_workspace(name, query, key.shape[2], block_size, output, partial_stats, partial_values)
    return _gqa_decode_dense(name, query, key, value, None, scaling, gate, output=output, partial_stats=partial_stats,
                             partial_values=partial_values, block_size=block_size)


def _op_gqa_decode_splitkv_turboquant_fused_out(query, quantized_key, value_data, value_scales, value_zeros,
                                                residual_key, residual_value, output, partial_stats, partial_values,
                                                scaling, value_bits, value_group_size, block_size, gate=None):
    """validate_gqa_decode_splitkv_turboquant_inputs (.sycl:1447-1501) + launch."""
    name = "gqa_decode_splitkv_turboquant_fused_out"
    query = _check_query(name, query)
    for label, tensor in (("quantized_key", quantized_key), ("value_data", value_data), ("value_scales", value_scales),
                          ("value_zeros", value_zeros), ("residual_key", residual_key),
                          ("residual_value", residual_value)):
        if tensor.dim() != 4:
            raise RuntimeError(f"{label} must be a 4-D tensor [batch, kv_heads, tokens, ...]")
    if query.shape[0] != quantized_key.shape[0] or query.shape[0] != residual_key.shape[0]:
        raise RuntimeError("query/quantized_key/residual_key batch size mismatch")
    if residual_key.shape != residual_value.shape:
        raise RuntimeError("residual_key and residual_value must share the same shape")
    if quantized_key.shape[1] != residual_key.shape[1]:
        raise RuntimeError("quantized and residual KV head count mismatch")
    if query.shape[1] % quantized_key.shape[1] != 0:
        raise RuntimeError("query heads must be divisible by kv_heads")
    if query.shape[3] != quantized_key.shape[3] or query.shape[3] != residual_key.shape[3]:
        raise RuntimeError("query/key head_dim mismatch")
    if quantized_key.shape[2] < 1:
        raise RuntimeError("gqa_decode_splitkv_turboquant_fused requires a non-empty quantized prefix")
    if value_data.shape[:3] != quantized_key.shape[:3] or value_scales.shape[:3] != quantized_key.shape[:3]:
        raise RuntimeError("value_data / value_scales must match quantized_key in batch, heads and quantized_len")
    if value_zeros.shape != value_scales.shape:
        raise RuntimeError("value_zeros shape must match value_scales")
    if value_bits not in (2, 3, 4):
        raise RuntimeError("TurboQuant value_bits must be 2, 3, or 4")
    dim = int(query.shape[3])
    if value_group_size <= 0 or dim % value_group_size != 0 or value_scales.shape[3] * value_group_size != dim:
        raise RuntimeError("TurboQuant value_group_size must evenly divide head_dim and match value_scales")
    per_byte = 4 if value_bits == 2 else 2
    if value_data.shape[3] * per_byte < dim:
        raise RuntimeError("TurboQuant packed value width is smaller than head_dim")
    if block_size < 16:
        raise RuntimeError("gqa_decode_splitkv_turboquant_fused block_size must be at least 16")
    if value_data.dtype != torch.uint8:
        raise RuntimeError("TurboQuant value_data must be uint8")
    if not (query.dtype == quantized_key.dtype == residual_key.dtype == residual_value.dtype == value_scales.dtype
            == value_zeros.dtype):
        raise RuntimeError("query, keys, residual values, value_scales, and value_zeros must share the same dtype")
    device = _require_cuda(name, query=query, quantized_key=quantized_key, value_data=value_data,
                           value_scales=value_scales, value_zeros=value_zeros, residual_key=residual_key,
                           residual_value=residual_value, gate=gate)
    quantized_len, residual_len = int(quantized_key.shape[2]), int(residual_key.shape[2])
    _check_split_workspace(name, query, quantized_len + residual_len, block_size, output, partial_stats, partial_values)
    quantized_key = _last_dim_contiguous(quantized_key)
    value_data = _last_dim_contiguous(value_data)
    value_scales = _last_dim_contiguous(value_scales)
    value_zeros = _last_dim_contiguous(value_zeros)
    if value_zeros.stride() != value_scales.stride():
        value_scales, value_zeros = value_scales.contiguous(), value_zeros.contiguous()
    residual_key = _last_dim_contiguous(residual_key)
    residual_value = _last_dim_contiguous(residual_value)
    if residual_value.stride() != residual_key.stride():
        residual_key, residual_value = residual_key.contiguous(), residual_value.contiguous()
    gate, gate_sb, gate_sh = _check_gate(name, query, gate)
    batch, heads = int(query.shape[0]), int(query.shape[1])
    kv_heads = int(quantized_key.shape[1])
    target = output if output.stride(3) == 1 else torch.empty((batch, heads, 1, dim), dtype=query.dtype, device=device)
    chunk_tokens = min(max(int(block_size), 16), quantized_len + residual_len)
    with on_device(device):
        _lib.check(_lib.lib().anna_gqa_decode_turboquant_values(
            ptr(query), query.stride(0), query.stride(1), ptr(quantized_key), quantized_key.stride(0),
            quantized_key.stride(1), quantized_key.stride(2), ptr(value_data), value_data.stride(0),
            value_data.stride(1), value_data.stride(2), ptr(value_scales), ptr(value_zeros), value_scales.stride(0),
            value_scales.stride(1), value_scales.stride(2), ptr(residual_key) if residual_len else None,
            ptr(residual_value) if residual_len else None, residual_key.stride(0), residual_key.stride(1),
            residual_key.stride(2), ptr(gate), gate_sb, gate_sh, ptr(target), target.stride(0), target.stride(1),
            ptr(partial_stats), ptr(partial_values), int(partial_stats.shape[2]), chunk_tokens, batch, heads, kv_heads,
            quantized_len, residual_len, dim, int(value_bits), int(value_group_size), float(scaling),
            dtype_code(query.dtype), stream_ptr(device)), name)
    if target is not output:
        output.copy_(target)
    return output


def _op_paged_gqa_decode_fused(query, key_pages, value_pages, page_table, visible_lengths, scaling, gate=None):
    name = "paged_gqa_decode_fused"
    query = _check_query(name, query)
    if key_pages.dim() != 4 or value_pages.dim() != 4:
        raise RuntimeError("key_pages and value_pages must be [pages, kv_heads, block_size, head_dim]")
    if key_pages.shape != value_pages.shape:
        raise RuntimeError("key_pages and value_pages must share the same shape")
    if page_table.dim() != 2 or page_table.shape[0] != query.shape[0]:
        raise RuntimeError("page_table must be [batch, max_blocks]")
    if visible_lengths.dim() != 1 or visible_lengths.shape[0] != query.shape[0]:
        raise RuntimeError("visible_lengths must be [batch]")
    if key_pages.shape[0] < 1 or key_pages.shape[1] < 1 or key_pages.shape[2] < 1:
        raise RuntimeError("pages, kv_heads and block_size must be positive")
    if query.shape[1] % key_pages.shape[1] != 0:
        raise RuntimeError("query heads must be divisible by kv_heads")
    if query.shape[3] != key_pages.shape[3]:
        raise RuntimeError("query/key_pages head_dim mismatch")
    if not (query.dtype == key_pages.dtype == value_pages.dtype):
        raise RuntimeError("query, key_pages, and value_pages must share the same dtype")
    if page_table.dtype != torch.int32:
        raise RuntimeError("page_table must be int32")
    if visible_lengths.dtype != torch.long:
        raise RuntimeError("visible_lengths must be int64")
    device = _require_cuda(name, query=query, key_pages=key_pages, value_pages=value_pages, page_table=page_table,
                           visible_lengths=visible_lengths, gate=gate)
    if not key_pages.is_contiguous():
        key_pages = key_pages.contiguous()
    if not value_pages.is_contiguous():
        value_pages = value_pages.contiguous()
    if page_table.stride(1) != 1:
        page_table = page_table.contiguous()
    if visible_lengths.stride(0) != 1:
        visible_lengths = visible_lengths.contiguous()
    gate, gate_sb, gate_sh = _check_gate(name, query, gate)
    batch, heads, _, dim = (int(v) for v in query.shape)
    pages, kv_heads, block = int(key_pages.shape[0]), int(key_pages.shape[1]), int(key_pages.shape[2])
    max_blocks = int(page_table.shape[1])
    out = torch.empty((batch, heads, 1, dim), dtype=query.dtype, device=device)
    if max_blocks == 0:
        return out.zero_()
    stats, values, capacity, counters = split_scratch(device, batch, heads, dim, kv_heads, max_blocks * block)
    with on_device(device):
        _lib.check(_lib.lib().anna_paged_gqa_decode(
            ptr(query), query.stride(0), query.stride(1), ptr(key_pages), ptr(value_pages), ptr(page_table),
            page_table.stride(0), ptr(visible_lengths), ptr(gate), gate_sb, gate_sh, ptr(out), out.stride(0),
            out.stride(1), ptr(stats), ptr(values), capacity, 0, ptr(counters), batch, heads, kv_heads, dim, block,
            pages, max_blocks, float(scaling), dtype_code(query.dtype), stream_ptr(device)), name)
    return out


def _op_paged_kv_write(key_states, value_states, key_pages, value_pages, page_table, past_lengths):
    """key_states / value_states [B, Hkv, T, D] -> pages [P, Hkv, S, D] at positions past_lengths[b] .. + T."""
    name = "paged_kv_write"
    if key_states.dim() != 4 or key_states.shape != value_states.shape:
        raise RuntimeError(f"{name}: key_states and value_states must be matching [batch, kv_heads, tokens, head_dim]")
    if key_pages.dim() != 4 or key_pages.shape != value_pages.shape:
        raise RuntimeError(f"{name}: key_pages and value_pages must be matching [pages, kv_heads, block_size, head_dim]")
    if key_pages.shape[1] != key_states.shape[1] or key_pages.shape[3] != key_states.shape[3]:
        raise RuntimeError(f"{name}: pages and states disagree on kv_heads / head_dim")
    if page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.shape[0] != key_states.shape[0]:
        raise RuntimeError(f"{name}: page_table must be int32 [batch, max_blocks]")
    if past_lengths.dtype != torch.long or past_lengths.shape != (key_states.shape[0],):
        raise RuntimeError(f"{name}: past_lengths must be int64 [batch]")
    if not (key_states.dtype == value_states.dtype == key_pages.dtype == value_pages.dtype):
        raise RuntimeError(f"{name}: states and pages must share the same dtype")
    device = _require_cuda(name, key_states=key_states, value_states=value_states, key_pages=key_pages,
                           value_pages=value_pages, page_table=page_table, past_lengths=past_lengths)
    if not key_pages.is_contiguous() or not value_pages.is_contiguous():
        raise RuntimeError(f"{name}: page pools must be contiguous")
    key_states = key_states if key_states.stride(3) == 1 else key_states.contiguous()
    if value_states.stride() != key_states.stride():
        key_states, value_states = key_states.contiguous(), value_states.contiguous()
    if page_table.stride(1) != 1:
        page_table = page_table.contiguous()
    batch, kv_heads, tokens, dim = (int(v) for v in key_states.shape)
    if tokens == 0 or batch == 0:
        return
    with on_device(device):
        _lib.check(_lib.lib().anna_paged_kv_write(
            ptr(key_states), ptr(value_states), key_states.stride(0), key_states.stride(1), key_states.stride(2),
            ptr(key_pages), ptr(value_pages), ptr(page_table), page_table.stride(0), ptr(past_lengths.contiguous()),
            None, batch, kv_heads, tokens, dim, int(key_pages.shape[2]), int(key_pages.shape[0]),
            int(page_table.shape[1]), dtype_code(key_states.dtype), None, stream_ptr(device)), name)


def _check_tq_geometry(name, packed_pages, page_table, window, window_slots, lengths, batch, head_dim, bits,
                       residual_len, block_size, value_group_size, dtype):
    if bits not in (2, 3, 4):
        raise RuntimeError(f"{name}: bits must be 2, 3 or 4")
    if packed_pages.dtype != torch.uint8 or packed_pages.dim() != 3 or not packed_pages.is_contiguous():
        raise RuntimeError(f"{name}: packed_pages must be contiguous uint8 [pages, kv_heads, chunk_bytes]")
    layout = _lib.tq_page_layout(head_dim, bits, block_size, dtype_code(dtype), value_group_size)
    if int(packed_pages.shape[2]) != layout["chunk_bytes"]:
        raise RuntimeError(f"{name}: packed page chunks are {int(packed_pages.shape[2])} bytes, the layout for "
                           f"head_dim={head_dim} bits={bits} block_size={block_size} needs {layout['chunk_bytes']}")
    if window.dim() != 5 or window.shape[1] != 2 or window.shape[3] != residual_len or window.shape[4] != head_dim:
        raise RuntimeError(f"{name}: window must be [slots, 2, kv_heads, residual_len, head_dim]")
    if window.dtype != dtype or not window.is_contiguous():
        raise RuntimeError(f"{name}: window must be contiguous and share the dtype of the states")
    if page_table.dtype != torch.int32 or page_table.dim() != 2 or page_table.shape[0] != batch:
        raise RuntimeError(f"{name}: page_table must be int32 [batch, max_blocks]")
    for label, tensor in (("window_slots", window_slots), ("lengths", lengths)):
        if tensor.dtype != torch.long or tensor.shape != (batch,):
            raise RuntimeError(f"{name}: {label} must be int64 [batch]")


def _op_tq_append(key_states, value_states, packed_pages, page_table, window, window_slots, past_lengths, bits,
                  residual_len, block_size, value_group_size):
    """Ring update + quantize-on-overflow + bit packing + page scatter for B rows in one launch."""
    from .tq_tables import key_tables

    name = "tq_append"
    if key_states.dim() != 4 or key_states.shape != value_states.shape or key_states.dtype != value_states.dtype:
        raise RuntimeError(f"{name}: key_states and value_states must be matching [batch, kv_heads, tokens, head_dim]")
    batch, kv_heads, tokens, dim = (int(v) for v in key_states.shape)
    _check_tq_geometry(name, packed_pages, page_table, window, window_slots, past_lengths, batch, dim, bits,
                       residual_len, block_size, value_group_size, key_states.dtype)
    device = _require_cuda(name, key_states=key_states, value_states=value_states, packed_pages=packed_pages,
                           page_table=page_table, window=window, window_slots=window_slots, past_lengths=past_lengths)
    if tokens == 0 or batch == 0:
        return
    key_states = key_states if key_states.stride(3) == 1 else key_states.contiguous()
    if value_states.stride() != key_states.stride():
        key_states, value_states = key_states.contiguous(), value_states.contiguous()
    if page_table.stride(1) != 1:
        page_table = page_table.contiguous()
    tables = key_tables(head_dim=dim, bits=bits, device=device)
    status = torch.zeros(1, dtype=torch.int32, device=device)
    with on_device(device):
        _lib.check(_lib.lib().anna_tq_append(
            ptr(key_states), ptr(value_states), key_states.stride(0), key_states.stride(1), key_states.stride(2),
            ptr(packed_pages), ptr(page_table), page_table.stride(0), None, 0, ptr(window),
            ptr(window_slots.contiguous()), ptr(past_lengths.contiguous()), None, ptr(tables.signs1),
            ptr(tables.signs2), ptr(tables.centroids), ptr(tables.boundaries), batch, kv_heads, tokens, dim,
            block_size, residual_len, bits, value_group_size, int(packed_pages.shape[0]), int(page_table.shape[1]),
            dtype_code(key_states.dtype), ptr(status), stream_ptr(device)), name)


def _op_tq_paged_decode(query, packed_pages, page_table, window, window_slots, lengths, scaling, bits, residual_len,
                        block_size, value_group_size, gate=None):
    """Single-token GQA decode over [packed prefix | window ring] of B rows."""
    from .tq_tables import key_tables

    name = "tq_paged_decode"
    query = _check_query(name, query)
    batch, heads, _, dim = (int(v) for v in query.shape)
    _check_tq_geometry(name, packed_pages, page_table, window, window_slots, lengths, batch, dim, bits, residual_len,
                       block_size, value_group_size, query.dtype)
    kv_heads = int(packed_pages.shape[1])
    if heads % kv_heads != 0 or int(window.shape[2]) != kv_heads:
        raise RuntimeError(f"{name}: query heads must be a multiple of the kv heads of the pages and the window")
    device = _require_cuda(name, query=query, packed_pages=packed_pages, page_table=page_table, window=window,
                           window_slots=window_slots, lengths=lengths, gate=gate)
    gate, gate_sb, gate_sh = _check_gate(name, query, gate)
    if page_table.stride(1) != 1:
        page_table = page_table.contiguous()
    out = torch.empty((batch, heads, 1, dim), dtype=query.dtype, device=device)
    max_blocks = int(page_table.shape[1])
    tables = key_tables(head_dim=dim, bits=bits, device=device)
    stats, values, capacity, counters = split_scratch(device, batch, heads, dim, kv_heads,
                                                      max_blocks * block_size + residual_len,
                                                      turboquant=(max_blocks, block_size, residual_len))
    frags = query_scratch(device, batch, heads, kv_heads, dim)
    with on_device(device):
        _lib.check(_lib.lib().anna_tq_paged_decode(
            ptr(query), query.stride(0), query.stride(1), ptr(packed_pages), ptr(page_table), page_table.stride(0),
            ptr(window), ptr(window_slots.contiguous()), ptr(lengths.contiguous()), ptr(tables.signs1),
            ptr(tables.signs2), ptr(tables.centroids), ptr(gate), gate_sb, gate_sh, ptr(out), out.stride(0),
            out.stride(1), ptr(stats), ptr(values), capacity, 0, ptr(counters), ptr(frags), frags.numel(), batch, heads,
            kv_heads, dim, block_size, residual_len, bits, value_group_size, int(packed_pages.shape[0]), max_blocks,
            float(scaling), dtype_code(query.dtype), stream_ptr(device)), name)
    return out


_IMPLS = {
    "paged_kv_write": _op_paged_kv_write,
    "tq_append": _op_tq_append,
    "tq_paged_decode": _op_tq_paged_decode,
    "gqa_decode_fused": _op_gqa_decode_fused,
    "gqa_decode_splitkv_fused": _op_gqa_decode_splitkv_fused,
    "gqa_decode_splitkv_fused_out": _op_gqa_decode_splitkv_fused_out,
    "gqa_decode_splitkv_turboquant_fused_out": _op_gqa_decode_splitkv_turboquant_fused_out,
    "paged_gqa_decode_fused": _op_paged_gqa_decode_fused,
}


def _meta_like_query(query, *args, **kwargs):
    return torch.empty_like(query)


def _meta_splitkv_out(query, key, value, output, *args, **kwargs):
    return output  # the op returns its `output` argument (Tensor(a!))


def _meta_turboquant_out(query, quantized_key, value_data, value_scales, value_zeros, residual_key, residual_value,
                         output, *args, **kwargs):
    return output


def _meta_none(*args, **kwargs):
    return None


_META = {
    "gqa_decode_fused": _meta_like_query,
    "gqa_decode_splitkv_fused": _meta_like_query,
    "gqa_decode_splitkv_fused_out": _meta_splitkv_out,
    "gqa_decode_splitkv_turboquant_fused_out": _meta_turboquant_out,
    "paged_gqa_decode_fused": _meta_like_query,
    "paged_kv_write": _meta_none,
    "tq_append": _meta_none,
    "tq_paged_decode": _meta_like_query,
}


def _register_ops() -> None:
    """CUDA kernels, Meta (shape-only) kernels and an autograd fall-through for every op, like the reference's
    registration (gated_delta_fused_op.sycl:7916-7983)."""
    global _REGISTERED, _LIBRARY
    if _REGISTERED:
        return
    library = torch.library.Library("anna", "FRAGMENT")
    for name, schema in {**SCHEMAS, **NEW_SCHEMAS}.items():
        library.define(name + schema)
        library.impl(name, _IMPLS[name], "CUDA")
        library.impl(name, _META[name], "Meta")
        library.impl(name, torch.library.fallthrough_kernel, "Autograd")
    _LIBRARY = library
    _REGISTERED = True


# ---------------------------------------------------------------------------------------------------------------
# public surface (names follow src/anna/model/fused_ops.py)


def maybe_load_gated_delta_library(path: str | os.PathLike[str] | None = None) -> bool:
    """Load libanna_b200_kv.so and register the ``anna::`` decode ops; True when they are available.

    ``path`` and ``ANNA_GATED_DELTA_OP_LIB`` are accepted for call-site compatibility with the reference
    (fused_ops.py:414-448); the library that is loaded is always the one built next to this package.
    """
    with _LOAD_LOCK:
        if _REGISTERED:
            return True
        try:
            _lib.lib()
        except RuntimeError:
            return False
        _register_ops()
        _LOADED_LIBRARIES.add(str(_lib.library_path()))
    return True


def loaded_fused_library_paths() -> tuple[str, ...]:
    return tuple(sorted(_LOADED_LIBRARIES))


def _op(name: str):
    namespace = getattr(torch.ops, "anna", None)
    if namespace is None or not _REGISTERED:
        return None
    return getattr(namespace, name, None)


def gqa_decode_fused_is_available() -> bool:
    return _op("gqa_decode_fused") is not None


def gqa_decode_splitkv_fused_is_available() -> bool:
    return _op("gqa_decode_splitkv_fused") is not None


def gqa_decode_splitkv_fused_out_is_available() -> bool:
    return _op("gqa_decode_splitkv_fused_out") is not None


def gqa_decode_splitkv_turboquant_fused_out_is_available() -> bool:
    return _op("gqa_decode_splitkv_turboquant_fused_out") is not None


def paged_gqa_decode_fused_is_available() -> bool:
    return _op("paged_gqa_decode_fused") is not None


def _resolve(name: str):
    op = _op(name)
    if op is None:
        maybe_load_gated_delta_library()
        op = _op(name)
    if op is None:
        raise RuntimeError(
            f"Anna {name} op is not registered. Build the CUDA library first (python -m anna_b200.build); "
            "there is no CPU fallback for this op.")
    return op


def run_gqa_decode_fused(*, query, key, value, visible_lengths, scaling, gate=None):
    _resolve("gqa_decode_fused")
    op = _op_gqa_decode_fused  # same function the dispatcher would reach for CUDA tensors
    if gate is None:
        return op(query, key, value, visible_lengths, float(scaling))
    return op(query, key, value, visible_lengths, float(scaling), gate)


def run_gqa_decode_splitkv_fused(*, query, key, value, scaling, block_size, gate=None):
    _resolve("gqa_decode_splitkv_fused")
    op = _op_gqa_decode_splitkv_fused  # same function the dispatcher would reach for CUDA tensors
    if gate is None:
        return op(query, key, value, float(scaling), int(block_size))
    return op(query, key, value, float(scaling), int(block_size), gate)


def run_gqa_decode_splitkv_fused_out(*, query, key, value, output, partial_stats, partial_values, scaling, block_size,
                                     gate=None):
    _resolve("gqa_decode_splitkv_fused_out")
    op = _op_gqa_decode_splitkv_fused_out  # same function the dispatcher would reach for CUDA tensors
    if gate is None:
        return op(query, key, value, output, partial_stats, partial_values, float(scaling), int(block_size))
    return op(query, key, value, output, partial_stats, partial_values, float(scaling), int(block_size), gate)


def run_gqa_decode_splitkv_turboquant_fused_out(*, query, quantized_key, value_data, value_scales, value_zeros,
                                                residual_key, residual_value, output, partial_stats, partial_values,
                                                scaling, value_bits, value_group_size, block_size, gate=None):
    _resolve("gqa_decode_splitkv_turboquant_fused_out")
    return _op_gqa_decode_splitkv_turboquant_fused_out(
        query, quantized_key, value_data, value_scales, value_zeros, residual_key, residual_value, output,
        partial_stats, partial_values, float(scaling), int(value_bits), int(value_group_size), int(block_size), gate)


def run_paged_gqa_decode_fused(*, query, key_pages, value_pages, page_table, visible_lengths, scaling, gate=None):
    _resolve("paged_gqa_decode_fused")
    op = _op_paged_gqa_decode_fused  # same function the dispatcher would reach for CUDA tensors
    if gate is None:
        return op(query, key_pages, value_pages, page_table, visible_lengths, float(scaling))
    return op(query, key_pages, value_pages, page_table, visible_lengths, float(scaling), gate)
