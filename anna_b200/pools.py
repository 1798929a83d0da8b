"""Device page pools of the KV cache: un-quantized K/V pages, packed TurboQuant pages and window rings.

The bookkeeping (LIFO free list, growth by ``max(n, capacity or 16)``, reversed release order, refcounts) follows
``Qwen3PagedLayerAllocator`` (``src/anna/model/ops.py:92-245``) so page ids come out in the reference's order.
"""
from __future__ import annotations

from collections.abc import Callable

import torch

from . import _lib
from .fused_ops import dtype_code


def resolve_value_group_size(head_dim: int) -> int:
    """Largest of 32, 16, 8, 4, 2, 1 dividing head_dim (src/anna/model/turboquant.py:157-161)."""
    for candidate in (32, 16, 8, 4, 2, 1):
        if candidate <= head_dim and head_dim % candidate == 0:
            return candidate
    return 1


class _PageBook:
    def __init__(self, on_page_freed: Callable[[int], None] | None = None,
                 listening: Callable[[], bool] | None = None) -> None:
        self.free_pages: list[int] = []
        self.refcount: dict[int, int] = {}
        self._on_page_freed = on_page_freed
        self._listening = listening  # optional: False while the callback has nothing to do (an empty registry)
        self._shared = 0  # pages with more than one owner

    def take(self, num_pages: int, capacity: int) -> tuple[list[int], int, list[int]]:
        """Pop up to num_pages from the free list; returns (page ids, new capacity, ids created by growth)."""
        count = min(max(int(num_pages), 0), len(self.free_pages))
        out: list[int] = []
        if count > 0:
            # the last `count` entries of the free list, most recently freed first (the same order as repeated pop())
            out = self.free_pages[-count:]
            out.reverse()
            del self.free_pages[-count:]
            stale = self.refcount.keys() & out
            if stale:
                raise RuntimeError(f"Invariant violated: free list page {min(stale)} has non-zero refcount.")
            self.refcount.update(dict.fromkeys(out, 1))
        missing = num_pages - len(out)
        new_capacity = capacity
        fresh: list[int] = []
        if missing > 0:
            grow_by = max(missing, capacity or 16)
            new_capacity = capacity + grow_by
            new_ids = list(range(capacity, new_capacity))
            fresh = new_ids[:missing]
            self.free_pages.extend(reversed(new_ids[missing:]))
            self.refcount.update(dict.fromkeys(fresh, 1))
            out.extend(fresh)
        return out, new_capacity, fresh

    def grow_free(self, required: int, capacity: int) -> int:
        """ensure_capacity: grow so that capacity >= required, new pages go to the free list."""
        if required <= capacity:
            return capacity
        missing = required - capacity
        grow_by = max(missing, capacity or 16)
        new_capacity = capacity + grow_by
        self.free_pages.extend(reversed(range(capacity, new_capacity)))
        return new_capacity

    def retain(self, page_id: int) -> None:
        rc = self.refcount.get(page_id, 0)
        self.refcount[page_id] = rc + 1
        if rc == 1:
            self._shared += 1

    def release(self, page_id: int) -> None:
        rc = self.refcount.get(page_id, 0)
        if rc <= 0:
            return
        if rc == 1:
            self.refcount.pop(page_id, None)
            self.free_pages.append(page_id)
            if self._on_page_freed is not None:
                self._on_page_freed(page_id)
        else:
            self.refcount[page_id] = rc - 1
            if rc == 2:
                self._shared -= 1

    def release_many(self, page_ids, *, notify: bool = True) -> None:
        """release() for every id of `page_ids`, in the given order, in one pass.  `notify=False` skips the per-page
        callback (for callers that know nobody listens, e.g. an empty prefix registry)."""
        refcount = self.refcount
        ids = page_ids if isinstance(page_ids, list) else list(page_ids)
        if self._shared == 0 and refcount.keys() >= set(ids) and len(set(ids)) == len(ids):
            # nothing is shared and every id is held exactly once: all of them become free, at C speed
            for _ in map(refcount.__delitem__, ids):
                pass
            freed = ids
        else:
            freed = []
            for page_id in ids:
                rc = refcount.get(page_id, 0)
                if rc == 1:
                    del refcount[page_id]
                    freed.append(page_id)
                elif rc > 1:
                    refcount[page_id] = rc - 1
                    if rc == 2:
                        self._shared -= 1
        if freed:
            self.free_pages.extend(freed)
            if notify and self._on_page_freed is not None and (self._listening is None or self._listening()):
                for page_id in freed:
                    self._on_page_freed(page_id)

    def clear(self) -> None:
        self.free_pages.clear()
        self.refcount.clear()
        self._shared = 0


def _grown(old: torch.Tensor | None, shape: tuple[int, ...], like: torch.Tensor, dtype: torch.dtype | None = None):
    new = torch.empty(shape, dtype=dtype or like.dtype, device=like.device)
    if old is not None and old.shape[0] > 0:
        new[: old.shape[0]].copy_(old)
    return new


class Qwen3PagedLayerAllocator:
    """Un-quantized page pool of one layer: ``key_pages`` / ``value_pages`` ``[P, Hkv, S, D]`` (ops.py:92-245)."""

    def __init__(self, block_size: int, *, on_page_freed: Callable[[int], None] | None = None,
                 on_trim: Callable[[], None] | None = None, listening: Callable[[], bool] | None = None) -> None:
        self.block_size = block_size
        self._on_trim = on_trim
        self._book = _PageBook(on_page_freed, listening)
        self.key_pages: torch.Tensor | None = None
        self.value_pages: torch.Tensor | None = None

    @property
    def free_pages(self) -> list[int]:
        return self._book.free_pages

    @property
    def _refcount(self) -> dict[int, int]:
        return self._book.refcount

    def capacity(self) -> int:
        return 0 if self.key_pages is None else int(self.key_pages.shape[0])

    def used_pages(self) -> int:
        capacity = self.capacity()
        return max(0, min(capacity, capacity - len(self.free_pages)))

    def _resize(self, new_capacity: int, key_template: torch.Tensor, value_template: torch.Tensor) -> None:
        if new_capacity == self.capacity():
            return
        key_shape = (new_capacity, key_template.shape[1], self.block_size, key_template.shape[3])
        value_shape = (new_capacity, value_template.shape[1], self.block_size, value_template.shape[3])
        self.key_pages = _grown(self.key_pages, key_shape, key_template)
        self.value_pages = _grown(self.value_pages, value_shape, value_template)

    def allocate(self, num_pages: int, *, key_template: torch.Tensor, value_template: torch.Tensor) -> list[int]:
        page_ids, new_capacity, _ = self._book.take(num_pages, self.capacity())
        self._resize(new_capacity, key_template, value_template)
        return page_ids

    def retain_page(self, page_id: int) -> None:
        cap = self.capacity()
        if page_id < 0 or (cap > 0 and page_id >= cap):
            raise ValueError(f"retain_page: invalid page_id={page_id} capacity={cap}.")
        self._book.retain(page_id)

    def page_owners(self, page_id: int) -> int:
        """How many block tables map this page (0 for a free page)."""
        return self._book.refcount.get(page_id, 0)

    def release_page(self, page_id: int) -> None:
        self._book.release(page_id)

    def release_pages(self, page_ids: list[int]) -> None:
        self._book.release_many(reversed(page_ids))

    def free(self, page_ids: list[int]) -> None:
        self.release_pages(page_ids)

    def ensure_capacity(self, required_pages: int, *, key_template: torch.Tensor, value_template: torch.Tensor) -> int:
        new_capacity = self._book.grow_free(max(0, int(required_pages)), self.capacity())
        self._resize(new_capacity, key_template, value_template)
        return self.capacity()

    def trim(self) -> int:
        capacity = self.capacity()
        if capacity <= 0 or self.used_pages() > 0:
            return 0
        if self._on_trim is not None:
            self._on_trim()
        self._book.clear()
        self.key_pages = None
        self.value_pages = None
        return capacity

    def to(self, *, device: torch.device | None = None, dtype: torch.dtype | None = None) -> None:
        for name in ("key_pages", "value_pages"):
            pages = getattr(self, name)
            if pages is not None:
                setattr(self, name, pages.to(device=device or pages.device, dtype=dtype or pages.dtype))


class TurboQuantLayerPool:
    """Packed page pool + window rings of one TurboQuant layer (geometry fixed by the first append)."""

    def __init__(self, block_size: int, *, on_page_freed: Callable[[int], None] | None = None,
                 listening: Callable[[], bool] | None = None) -> None:
        self.block_size = int(block_size)
        self._book = _PageBook(on_page_freed, listening)
        self.packed_pages: torch.Tensor | None = None  # uint8 [P, Hkv, chunk_bytes]
        self.window: torch.Tensor | None = None        # dtype [slots, 2, Hkv, R, D]
        self.free_slots: list[int] = []
        self.layout: dict[str, int] | None = None
        self.kv_heads = self.head_dim = self.bits = self.residual_len = self.value_group = 0
        self.dtype: torch.dtype | None = None
        self.device: torch.device | None = None
        self.status: torch.Tensor | None = None        # int32 [1] device status word

    @property
    def free_pages(self) -> list[int]:
        return self._book.free_pages

    @property
    def configured(self) -> bool:
        return self.layout is not None

    def configure(self, *, kv_heads: int, head_dim: int, bits: int, residual_len: int, dtype: torch.dtype,
                  device: torch.device, value_group: int | None = None) -> None:
        value_group = value_group or resolve_value_group_size(head_dim)
        if self.configured:
            same = (self.kv_heads, self.head_dim, self.bits, self.residual_len, self.dtype, self.value_group) == (
                kv_heads, head_dim, bits, residual_len, dtype, value_group)
            if not same or self.device != device:
                raise ValueError("TurboQuant layer pool geometry mismatch (heads, head_dim, bits, window, dtype, device)")
            return
        self.layout = _lib.tq_page_layout(head_dim, bits, self.block_size, dtype_code(dtype), value_group)
        self.kv_heads, self.head_dim, self.bits = int(kv_heads), int(head_dim), int(bits)
        self.residual_len, self.value_group = int(residual_len), int(value_group)
        self.dtype, self.device = dtype, device
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def capacity(self) -> int:
        return 0 if self.packed_pages is None else int(self.packed_pages.shape[0])

    def used_pages(self) -> int:
        capacity = self.capacity()
        return max(0, min(capacity, capacity - len(self.free_pages)))

    def _resize(self, new_capacity: int) -> None:
        if new_capacity == self.capacity():
            return
        assert self.layout is not None and self.device is not None
        shape = (new_capacity, self.kv_heads, self.layout["chunk_bytes"])
        new = torch.empty(shape, dtype=torch.uint8, device=self.device)
        if self.packed_pages is not None:
            new[: self.packed_pages.shape[0]].copy_(self.packed_pages)
        self.packed_pages = new

    def allocate(self, num_pages: int) -> list[int]:
        page_ids, new_capacity, _ = self._book.take(num_pages, self.capacity())
        self._resize(new_capacity)
        return page_ids

    def ensure_capacity(self, required_pages: int) -> int:
        self._resize(self._book.grow_free(max(0, int(required_pages)), self.capacity()))
        return self.capacity()

    def release_pages(self, page_ids: list[int]) -> None:
        self._book.release_many(reversed(page_ids))

    def page_owners(self, page_id: int) -> int:
        """How many rows map this packed page (0 for a free page)."""
        return self._book.refcount.get(page_id, 0)

    def retain_page(self, page_id: int) -> None:
        """One more owner of a packed page (a sequence that maps it for a shared prompt prefix, or a clone)."""
        if page_id < 0 or page_id >= self.capacity() or self._book.refcount.get(page_id, 0) <= 0:
            raise ValueError(f"retain_page: page {page_id} is not a live packed page (capacity {self.capacity()}).")
        self._book.retain(page_id)

    def slot_capacity(self) -> int:
        return 0 if self.window is None else int(self.window.shape[0])

    def allocate_slot(self) -> int:
        if not self.free_slots:
            old = self.slot_capacity()
            new_capacity = old + max(1, old or 16)
            assert self.dtype is not None and self.device is not None
            shape = (new_capacity, 2, self.kv_heads, self.residual_len, self.head_dim)
            new = torch.empty(shape, dtype=self.dtype, device=self.device)
            if self.window is not None:
                new[:old].copy_(self.window)
            self.window = new
            self.free_slots.extend(reversed(range(old, new_capacity)))
        return self.free_slots.pop()

    def ensure_slot_capacity(self, required_slots: int) -> None:
        while self.slot_capacity() - 0 < required_slots:
            old = self.slot_capacity()
            new_capacity = max(required_slots, old + max(1, old or 16))
            assert self.dtype is not None and self.device is not None
            shape = (new_capacity, 2, self.kv_heads, self.residual_len, self.head_dim)
            new = torch.empty(shape, dtype=self.dtype, device=self.device)
            if self.window is not None:
                new[:old].copy_(self.window)
            self.window = new
            self.free_slots.extend(reversed(range(old, new_capacity)))

    def release_slot(self, slot: int) -> None:
        self.free_slots.append(int(slot))

    def trim(self) -> int:
        capacity = self.capacity()
        if self.used_pages() > 0 or len(self.free_slots) != self.slot_capacity():
            return 0
        self._book.clear()
        self.packed_pages = None
        self.window = None
        self.free_slots.clear()
        return capacity

    def clear(self) -> int:
        capacity = self.capacity()
        self._book.clear()
        self.packed_pages = None
        self.window = None
        self.free_slots.clear()
        return capacity
