"""Oracle restatement of the cache-side state machines (numpy, host only).  Test infrastructure.

* ``OracleLayerAllocator``   follows Qwen3PagedLayerAllocator (src/anna/model/ops.py:92-245): LIFO free list,
  growth by ``max(n, old_capacity or 16)``, reversed release order, refcounts.  Only the bookkeeping is
  restated; page bytes are not held here.
* ``OracleTurboQuantRow``    follows TurboQuantKVRow.append / materialize / decode_attention
  (src/anna/model/turboquant.py:1027-1140, :1142-1179, :1275-1293): newest ``residual_len`` tokens stay in the
  cache dtype, every older token is quantized exactly once, in arrival order.
* ``PackedPageLayout`` / ``pack_key_codes`` state the byte layout of a packed page.  The reference never pages
  quantized layers (ops.py:903-904), so the rule is this build's: quantized token ``j`` of a row lives in block
  ``j // S`` of that row's table at slot ``j % S``; a block is taken from the allocator when the quantized
  length first reaches it.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


def paged_blocks_needed(length: int, block_size: int) -> int:
    return (max(0, int(length)) + block_size - 1) // block_size


# --------------------------------------------------------------------------------------------------
# packed byte formats


def pack_key_codes(idx: np.ndarray, sign: np.ndarray, bits: int) -> np.ndarray:
    """[..., D] index + sign planes -> [..., D*bits/8] bytes.

    bits == 4 : one nibble per coordinate, ``idx | sign << 3``; coordinate 2j in the low nibble of byte j.
    bits == 2 : one 2-bit field per coordinate, ``idx | sign << 1``; coordinate 4j+k at bits 2k of byte j.
    bits == 3 : D/4 bytes of 2-bit indices (coordinate 4j+k at bits 2k) followed by D/8 bytes of sign bits
                (coordinate 8j+k at bit k).
    """
    idx = np.asarray(idx, dtype=np.uint8)
    sign = np.asarray(sign, dtype=np.uint8)
    dim = idx.shape[-1]
    lead = idx.shape[:-1]
    if bits == 4:
        code = (idx | (sign << 3)).reshape(*lead, dim // 2, 2)
        return (code[..., 0] | (code[..., 1] << 4)).astype(np.uint8)
    if bits == 2:
        code = (idx | (sign << 1)).reshape(*lead, dim // 4, 4)
        return (code[..., 0] | (code[..., 1] << 2) | (code[..., 2] << 4) | (code[..., 3] << 6)).astype(np.uint8)
    if bits == 3:
        i4 = idx.reshape(*lead, dim // 4, 4)
        plane = (i4[..., 0] | (i4[..., 1] << 2) | (i4[..., 2] << 4) | (i4[..., 3] << 6)).astype(np.uint8)
        s8 = sign.reshape(*lead, dim // 8, 8).astype(np.uint16)
        sbits = np.zeros(s8.shape[:-1], dtype=np.uint16)
        for k in range(8):
            sbits |= s8[..., k] << k
        return np.concatenate([plane, sbits.astype(np.uint8)], axis=-1)
    raise ValueError(f"unsupported key bit-width {bits}")


def unpack_key_codes(packed: np.ndarray, bits: int, dim: int) -> tuple[np.ndarray, np.ndarray]:
    packed = np.asarray(packed, dtype=np.uint8)
    lead = packed.shape[:-1]
    if bits == 4:
        code = np.stack([packed & 0x0F, packed >> 4], axis=-1).reshape(*lead, dim)
        return code & 0x7, code >> 3
    if bits == 2:
        code = np.stack([(packed >> s) & 0x3 for s in (0, 2, 4, 6)], axis=-1).reshape(*lead, dim)
        return code & 0x1, code >> 1
    if bits == 3:
        plane, sbytes = packed[..., : dim // 4], packed[..., dim // 4:]
        idx = np.stack([(plane >> s) & 0x3 for s in (0, 2, 4, 6)], axis=-1).reshape(*lead, dim)
        sign = np.stack([(sbytes >> k) & 0x1 for k in range(8)], axis=-1).reshape(*lead, dim)
        return idx, sign
    raise ValueError(f"unsupported key bit-width {bits}")


def _align(value: int, to: int) -> int:
    return (value + to - 1) // to * to


@dataclass(frozen=True)
class PackedPageLayout:
    """Byte offsets inside one (page, kv-head) chunk of a packed page pool ``uint8 [P, Hkv, chunk_bytes]``."""

    head_dim: int
    bits: int
    block_size: int
    dtype_bytes: int
    group: int

    @property
    def key_bytes(self) -> int:
        return self.head_dim * self.bits // 8

    @property
    def value_bytes(self) -> int:
        return self.head_dim // (4 if self.bits == 2 else 2)

    @property
    def groups(self) -> int:
        return self.head_dim // self.group

    @property
    def off_kcodes(self) -> int:
        return 0

    @property
    def off_knorm(self) -> int:
        return _align(self.block_size * self.key_bytes, 16)

    @property
    def off_krnorm(self) -> int:
        return _align(self.off_knorm + 4 * self.block_size, 16)

    @property
    def off_vdata(self) -> int:
        return _align(self.off_krnorm + 4 * self.block_size, 16)

    @property
    def off_vscale(self) -> int:
        return _align(self.off_vdata + self.block_size * self.value_bytes, 16)

    @property
    def off_vzero(self) -> int:
        return _align(self.off_vscale + self.block_size * self.groups * self.dtype_bytes, 16)

    @property
    def chunk_bytes(self) -> int:
        return _align(self.off_vzero + self.block_size * self.groups * self.dtype_bytes, 128)

    def bytes_per_token(self) -> int:
        """Algorithmic bytes stored per token per kv head (codes + metadata)."""
        return self.key_bytes + 8 + self.value_bytes + 2 * self.groups * self.dtype_bytes


# --------------------------------------------------------------------------------------------------
# page allocator bookkeeping (ops.py:92-245)


class OracleLayerAllocator:
    def __init__(self) -> None:
        self.capacity = 0
        self.free_pages: list[int] = []
        self.refcount: dict[int, int] = {}

    def _grow(self, num_pages: int) -> list[int]:
        old = self.capacity
        grow_by = max(num_pages, old or 16)
        self.capacity = old + grow_by
        new_ids = list(range(old, self.capacity))
        for page_id in reversed(new_ids[num_pages:]):
            self.free_pages.append(page_id)
        return new_ids[:num_pages]

    def allocate(self, num_pages: int) -> list[int]:
        out: list[int] = []
        while self.free_pages and len(out) < num_pages:
            page_id = self.free_pages.pop()
            self.refcount[page_id] = 1
            out.append(page_id)
        missing = num_pages - len(out)
        if missing > 0:
            fresh = self._grow(missing)
            for page_id in fresh:
                self.refcount[page_id] = 1
            out.extend(fresh)
        return out

    def retain_page(self, page_id: int) -> None:
        self.refcount[page_id] = self.refcount.get(page_id, 0) + 1

    def release_page(self, page_id: int) -> None:
        rc = self.refcount.get(page_id, 0)
        if rc <= 0:
            return
        if rc == 1:
            del self.refcount[page_id]
            self.free_pages.append(page_id)
        else:
            self.refcount[page_id] = rc - 1

    def release_pages(self, page_ids: list[int]) -> None:
        for page_id in reversed(page_ids):
            self.release_page(page_id)

    def ensure_capacity(self, required_pages: int) -> int:
        required = max(0, int(required_pages))
        if required <= self.capacity:
            return self.capacity
        for page_id in reversed(self._grow(required - self.capacity)):
            self.free_pages.append(page_id)
        return self.capacity

    def used_pages(self) -> int:
        return max(0, min(self.capacity, self.capacity - len(self.free_pages)))

    def trim(self) -> int:
        if self.capacity <= 0 or self.used_pages() > 0:
            return 0
        released = self.capacity
        self.capacity = 0
        self.free_pages.clear()
        self.refcount.clear()
        return released


# --------------------------------------------------------------------------------------------------
# one sequence of one layer (turboquant.py:480-1346)


class OracleTurboQuantRow:
    def __init__(self, *, bits: int, residual_len: int, dtype: int, block_size: int = 16,
                 allocator: OracleLayerAllocator | None = None, keep_decode_cache: bool = False) -> None:
        # keep_decode_cache: hold the dense [Hkv, L, D] keys / values that decode_attention multiplies with and extend
        # them in place at every append, as the reference does with _KEEP_DECODE_CACHE (turboquant.py:15, :742-782,
        # :889-923, :1089-1140).  Off: every decode_attention call de-quantizes the whole prefix again.
        self.keep_decode_cache = bool(keep_decode_cache)
        self._full_keys: np.ndarray | None = None
        self._full_values: np.ndarray | None = None
        self.bits = int(bits)
        self.residual_len = max(1, int(residual_len))
        self.dtype = int(dtype)
        self.block_size = int(block_size)
        self.allocator = allocator
        self.block_table: list[int] = []
        self.length = 0
        self.num_heads: int | None = None
        self.head_dim: int | None = None
        self.group: int | None = None
        # quantized state: buffers that double when they run full (turboquant.py:576-581, :583-689), of which the first
        # `quantized_length` tokens are in use; idx / sign / norms / rnorms / vdata / vscales / vzeros are views of them
        self._state: dict[str, np.ndarray] = {}
        self._quantized = 0
        self.residual_keys: np.ndarray | None = None
        self.residual_values: np.ndarray | None = None

    @property
    def quantized_length(self) -> int:
        return self._quantized

    def _view(self, name: str) -> np.ndarray | None:
        return None if self._quantized == 0 else self._state[name][:, :self._quantized]

    idx = property(lambda self: self._view("idx"))
    sign = property(lambda self: self._view("sign"))
    norms = property(lambda self: self._view("norms"))
    rnorms = property(lambda self: self._view("rnorms"))
    vdata = property(lambda self: self._view("vdata"))
    vscales = property(lambda self: self._view("vscales"))
    vzeros = property(lambda self: self._view("vzeros"))

    def _append_quantized_state(self, parts: dict[str, np.ndarray]) -> None:
        count = next(iter(parts.values())).shape[1]
        need = self._quantized + count
        for name, part in parts.items():
            current = self._state.get(name)
            capacity = 0 if current is None else current.shape[1]
            if need > capacity:
                grown = np.empty((part.shape[0], max(need, 16, 2 * capacity)) + part.shape[2:], dtype=part.dtype)
                if current is not None and self._quantized > 0:
                    grown[:, :self._quantized] = current[:, :self._quantized]
                self._state[name] = current = grown
            current[:, self._quantized:need] = part
        self._quantized = need

    @property
    def residual_length(self) -> int:
        return 0 if self.residual_keys is None else int(self.residual_keys.shape[1])

    def append(self, keys, values) -> None:
        """keys/values [Hkv, T, D] float32 arrays holding dtype-exact numbers (turboquant.py:1027-1140)."""
        from . import quantize_keys, quantize_values, resolve_value_group_size

        keys = np.asarray(keys, dtype=np.float32)
        values = np.asarray(values, dtype=np.float32)
        if keys.shape != values.shape or keys.ndim != 3:
            raise ValueError("expected matching [heads, tokens, dim] keys and values")
        if keys.shape[1] == 0:
            return
        if self.num_heads is None:
            self.num_heads, _, self.head_dim = keys.shape
            self.group = resolve_value_group_size(self.head_dim)
            self.residual_keys, self.residual_values = keys.copy(), values.copy()
        else:
            self.residual_keys = np.concatenate([self.residual_keys, keys], axis=1)
            self.residual_values = np.concatenate([self.residual_values, values], axis=1)
        self.length += keys.shape[1]
        if self.keep_decode_cache:
            self._extend_full_cache(keys, values)
        overflow = self.residual_keys.shape[1] - self.residual_len
        if overflow <= 0:
            return
        old_k, old_v = self.residual_keys[:, :overflow], self.residual_values[:, :overflow]
        idx, sign, norms, rnorms = quantize_keys(old_k, self.bits, "ip")
        vdata, vscales, vzeros = quantize_values(old_v, self.bits, self.group, self.dtype)
        self._append_quantized_state({"idx": idx, "sign": sign, "norms": norms, "rnorms": rnorms, "vdata": vdata,
                                      "vscales": vscales, "vzeros": vzeros})
        self.residual_keys = np.ascontiguousarray(self.residual_keys[:, overflow:])
        self.residual_values = np.ascontiguousarray(self.residual_values[:, overflow:])
        if self.keep_decode_cache:
            # the tokens that just left the window are now seen through their codes (turboquant.py:1104-1111, :1134-1140)
            from . import dequantize_keys, dequantize_values, round_dtype

            first = self.quantized_length - overflow
            self._full_keys[:, first:first + overflow] = round_dtype(
                dequantize_keys(idx, sign, norms, rnorms, self.bits), self.dtype)
            self._full_values[:, first:first + overflow] = round_dtype(
                dequantize_values(vdata, vscales, vzeros, self.bits, self.group), self.dtype)
        if self.allocator is not None:
            need = paged_blocks_needed(self.quantized_length, self.block_size)
            if need > len(self.block_table):
                self.block_table.extend(self.allocator.allocate(need - len(self.block_table)))

    def _extend_full_cache(self, keys: np.ndarray, values: np.ndarray) -> None:
        """Write the new tokens behind the cached ones; capacity doubles (min 16) like turboquant.py:576-581."""
        have = self.length - keys.shape[1]
        capacity = 0 if self._full_keys is None else self._full_keys.shape[1]
        if self.length > capacity:
            capacity = max(self.length, 16, 2 * capacity)
            grown_k = np.empty((keys.shape[0], capacity, keys.shape[2]), dtype=np.float32)
            grown_v = np.empty_like(grown_k)
            if have > 0:
                grown_k[:, :have] = self._full_keys[:, :have]
                grown_v[:, :have] = self._full_values[:, :have]
            self._full_keys, self._full_values = grown_k, grown_v
        self._full_keys[:, have:self.length] = keys
        self._full_values[:, have:self.length] = values

    def materialize(self) -> tuple[np.ndarray, np.ndarray]:
        """Dense [Hkv, L, D] keys / values in the cache dtype (turboquant.py:1142-1179)."""
        if self.keep_decode_cache and self._full_keys is not None:
            return self._full_keys[:, :self.length], self._full_values[:, :self.length]
        from . import dequantize_keys, dequantize_values, round_dtype

        if self.num_heads is None:
            raise RuntimeError("row is not initialised")
        k_parts, v_parts = [], []
        if self.quantized_length > 0:
            k_parts.append(round_dtype(dequantize_keys(self.idx, self.sign, self.norms, self.rnorms, self.bits),
                                       self.dtype))
            v_parts.append(round_dtype(dequantize_values(self.vdata, self.vscales, self.vzeros, self.bits,
                                                         self.group), self.dtype))
        if self.residual_length > 0:
            k_parts.append(self.residual_keys)
            v_parts.append(self.residual_values)
        return np.concatenate(k_parts, axis=1), np.concatenate(v_parts, axis=1)

    def decode_attention(self, query, *, scaling: float, gate=None, blas: bool = False) -> np.ndarray:
        """query [Hq, D] -> [Hq, D] float32 (turboquant.py:1275-1293 with fp32 compute)."""
        from . import gqa_decode, gqa_decode_blas

        query = np.asarray(query, dtype=np.float32)
        if self.length <= 0:
            return np.zeros_like(query)
        keys, values = self.materialize()
        fn = gqa_decode_blas if blas else gqa_decode
        return fn(query, keys, values, scaling, gate)

    def packed_chunks(self, layout: PackedPageLayout) -> np.ndarray:
        """Expected bytes of this row's pages: uint8 [blocks, Hkv, chunk_bytes], unused bytes zero."""
        from . import DTYPE_BF16, DTYPE_F16

        blocks = paged_blocks_needed(self.quantized_length, layout.block_size)
        out = np.zeros((blocks, self.num_heads, layout.chunk_bytes), dtype=np.uint8)
        if blocks == 0:
            return out
        kcodes = pack_key_codes(self.idx, self.sign, self.bits)
        for j in range(self.quantized_length):
            blk, slot = divmod(j, layout.block_size)
            for h in range(self.num_heads):
                chunk = out[blk, h]
                o = layout.off_kcodes + slot * layout.key_bytes
                chunk[o:o + layout.key_bytes] = kcodes[h, j]
                chunk[layout.off_knorm + 4 * slot: layout.off_knorm + 4 * slot + 4] = \
                    np.frombuffer(np.float32(self.norms[h, j]).tobytes(), dtype=np.uint8)
                chunk[layout.off_krnorm + 4 * slot: layout.off_krnorm + 4 * slot + 4] = \
                    np.frombuffer(np.float32(self.rnorms[h, j]).tobytes(), dtype=np.uint8)
                o = layout.off_vdata + slot * layout.value_bytes
                chunk[o:o + layout.value_bytes] = self.vdata[h, j]
                for name, base in (("vscales", layout.off_vscale), ("vzeros", layout.off_vzero)):
                    meta = getattr(self, name)[h, j].astype(np.float32)
                    if self.dtype == DTYPE_BF16:
                        raw = (meta.view(np.uint32) >> 16).astype(np.uint16).view(np.uint8)
                    elif self.dtype == DTYPE_F16:
                        raw = meta.astype(np.float16).view(np.uint8)
                    else:
                        raw = meta.view(np.uint8)
                    o = base + slot * layout.groups * layout.dtype_bytes
                    chunk[o:o + raw.size] = raw
        return out
