"""Registry of prompt-prefix blocks that already have a physical page (un-quantized paged layers only).

Same surface as ``PrefixBlockPool`` in ``src/anna/model/prefix_block_cache.py:20-62``: ``(layer, token block) ->
page id`` with reverse links so that a recycled page drops every key that pointed at it.
"""
from __future__ import annotations

from collections.abc import Sequence

BlockKey = tuple[int, tuple[int, ...]]


def prompt_token_blocks(tokens: Sequence[int], *, block_size: int) -> list[tuple[int, ...]]:
    if block_size <= 0:
        raise ValueError("block_size must be positive.")
    return [tuple(int(t) for t in tokens[i:i + block_size]) for i in range(0, len(tokens), block_size)]


class PrefixBlockPool:
    def __init__(self) -> None:
        self._page_of: dict[BlockKey, int] = {}
        self._keys_of: dict[tuple[int, int], set[BlockKey]] = {}

    def __len__(self) -> int:
        return len(self._page_of)

    def lookup(self, layer_idx: int, token_block: tuple[int, ...]) -> int | None:
        return self._page_of.get((layer_idx, token_block))

    def register(self, layer_idx: int, token_block: tuple[int, ...], page_id: int) -> None:
        key = (layer_idx, token_block)
        if key not in self._page_of:
            self._page_of[key] = page_id
            self._keys_of.setdefault((layer_idx, page_id), set()).add(key)

    def discard_page(self, layer_idx: int, page_id: int) -> None:
        if not self._keys_of:  # nothing registered: the common case when no prompt prefix is shared
            return
        for key in self._keys_of.pop((layer_idx, page_id), ()):
            self._page_of.pop(key, None)

    def clear_layer(self, layer_idx: int) -> None:
        for key in [k for k in self._page_of if k[0] == layer_idx]:
            page_id = self._page_of.pop(key)
            self._keys_of.pop((layer_idx, page_id), None)

    def clear(self) -> None:
        self._page_of.clear()
        self._keys_of.clear()
