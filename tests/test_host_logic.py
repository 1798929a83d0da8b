"""CPU: host-side logic of the cache manager (allocator policy, block tables, lifecycle, tables, validation).

Kernel launches are replaced by recorders, so these tests check what would be sent to the GPU, not what it computes.
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from anna_b200 import (KVCacheConfig, PrefixBlockPool, Qwen3DynamicCache, Qwen3PageAllocator,
                       Qwen3PagedLayerAllocator, TurboQuantKVRow, cache as cache_module, tq_tables)

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture()
def launches(monkeypatch):
    """Replace the CUDA launches by recorders."""
    calls = {"page_write": [], "tq_append": [], "tq_decode": []}

    def fake_page_write(self, layer, key_states, value_states, table_dev, past, **device_copies):
        calls["page_write"].append({"tokens": int(key_states.shape[2]), "past": list(past),
                                    "table": table_dev.clone()})

    def fake_tq_append(pool, key_states, value_states, table_dev, slots, past, **device_copies):
        calls["tq_append"].append({"tokens": int(key_states.shape[2]), "slots": list(slots), "past": list(past),
                                   "table": None if table_dev is None else table_dev.clone()})

    def fake_tq_decode(pool, query, table_dev, slots, lengths, scaling, gate, **device_copies):
        calls["tq_decode"].append({"slots": list(slots), "lengths": list(lengths)})
        return torch.zeros_like(query)

    monkeypatch.setattr(Qwen3DynamicCache, "_launch_page_write", fake_page_write)
    monkeypatch.setattr(cache_module, "launch_tq_append", fake_tq_append)
    monkeypatch.setattr(cache_module, "launch_tq_decode", fake_tq_decode)
    return calls


def _config(block=16, layers=1):
    return KVCacheConfig(num_hidden_layers=layers, cache_block_size=block)


def test_layer_allocator_follows_reference_trace():
    trace = json.loads((GOLDEN / "allocator_trace.json").read_text())
    alloc = Qwen3PagedLayerAllocator(16)
    template = torch.zeros(1, 2, 1, 8)
    kw = {"key_template": template, "value_template": template}
    for entry in trace:
        op, arg = entry["op"], entry["arg"]
        if op == "allocate":
            assert alloc.allocate(arg, **kw) == entry["result"]
        elif op == "release":
            alloc.release_pages(arg)
        elif op == "ensure_capacity":
            assert alloc.ensure_capacity(arg, **kw) == entry["result"]
        elif op == "retain":
            alloc.retain_page(arg)
        elif op == "release_all":
            for ids in (trace[1]["result"], trace[3]["result"], trace[9]["result"]):
                alloc.release_pages(ids)
        elif op == "trim":
            assert alloc.trim() == entry["result"]
        assert alloc.capacity() == entry["capacity"], entry
        assert alloc.free_pages == entry["free"], entry
        assert alloc.used_pages() == entry["used"], entry
    assert alloc.key_pages is None


def test_allocator_growth_keeps_page_contents():
    alloc = Qwen3PagedLayerAllocator(4)
    template = torch.zeros(1, 2, 1, 8)
    first = alloc.allocate(2, key_template=template, value_template=template)
    alloc.key_pages[first[0]].fill_(3.0)
    alloc.allocate(40, key_template=template, value_template=template)
    assert alloc.capacity() == 16 + 26 and alloc.key_pages.shape == (42, 2, 4, 8)
    assert torch.all(alloc.key_pages[first[0]] == 3.0)
    with pytest.raises(ValueError):
        alloc.retain_page(1000)


def test_paged_block_tables_match_reference(launches):
    """B=2, 40 tokens, S=16, nine decode steps, compaction, re-admission: page ids as the reference assigns them."""
    want = json.loads((GOLDEN / "paged_block_tables.json").read_text())
    allocator = Qwen3PageAllocator(_config())
    cache = Qwen3DynamicCache(_config(), allocator=allocator, batch_size=2)
    kv = torch.zeros(2, 2, 40, 8)
    _, _, past = cache.update(kv, kv, 0, require_dense_cache=False)
    assert past.tolist() == [0, 0]
    assert cache.page_tables[0] == want["after_prefill"]
    assert allocator.layers[0].free_pages == want["free_after_prefill"]
    for _ in range(9):
        cache.update(kv[:, :, :1], kv[:, :, :1], 0, require_dense_cache=False)
    assert cache.page_tables[0] == want["after_9_steps"]
    assert cache.get_seq_lengths().tolist() == [49, 49]
    # device copy: int32 [B, blocks], -1 padded, only appended entries are patched in
    last = launches["page_write"][-1]
    assert last["table"].dtype == torch.int32 and last["table"].tolist() == want["after_9_steps"]
    assert last["past"] == [48, 48] and last["tokens"] == 1
    compacted = cache.compact_batch_rows([1])
    assert allocator.layers[0].free_pages == want["free_after_compact"]
    assert compacted.page_tables[0] == want["survivor"] and compacted.get_seq_lengths().tolist() == [49]
    assert cache.get_seq_lengths().tolist() == [0, 0]
    fresh = Qwen3DynamicCache(_config(), allocator=allocator, batch_size=1)
    fresh.update(kv[:1, :, :33], kv[:1, :, :33], 0, require_dense_cache=False)
    assert fresh.page_tables[0] == want["readmitted"]
    state = compacted.paged_attention_state(0)
    assert state is not None and state[2].tolist() == want["survivor"] and state[3].tolist() == [49]
    assert state[2].dtype == torch.int32 and state[3].dtype == torch.long
    compacted.release()
    fresh.release()
    assert allocator.layers[0].used_pages() == 0
    assert allocator.trim() == 16


def test_reserved_capacity_preallocates_blocks(launches):
    cache = Qwen3DynamicCache(_config(block=4), batch_size=1)
    cache.reserve_sequence_capacity(10)
    kv = torch.zeros(1, 1, 3, 8)
    cache.update(kv, kv, 0, require_dense_cache=False)
    assert len(cache.page_tables[0][0]) == 3  # ceil(10 / 4), ops.py:709-710


def test_turboquant_block_tables_follow_quantized_length(launches):
    """Quantized token j lives in block j // S; a block is taken when the quantized length first reaches it, in row
    order, with the reference allocator policy."""
    cache = Qwen3DynamicCache(_config(block=4), batch_size=2, kv_cache_quantization="turboquant",
                              kv_cache_quant_bits=4, kv_cache_residual_len=6)
    orc_alloc = oracle.OracleLayerAllocator()
    tables = [[], []]
    lengths = [0, 0]
    kv = torch.zeros(2, 2, 1, 64)

    def expect(tokens):
        for b in range(2):
            lengths[b] += tokens
            need = oracle.paged_blocks_needed(max(0, lengths[b] - 6), 4)
            if need > len(tables[b]):
                tables[b].extend(orc_alloc.allocate(need - len(tables[b])))

    for tokens in (5, 1, 1, 1, 9, 1, 1, 1, 1):
        cache.update(kv.expand(2, 2, tokens, 64), kv.expand(2, 2, tokens, 64), 0, require_dense_cache=False)
        expect(tokens)
        rows = cache.turboquant_rows[0]
        assert [row.block_table for row in rows] == tables
        assert [row.length for row in rows] == lengths
        assert [row.quantized_length for row in rows] == [max(0, n - 6) for n in lengths]
        assert [row.residual_length for row in rows] == [min(6, n) for n in lengths]
    assert cache.paged_attention_state(0) is None  # quantized layers are never exposed as dense pages
    last = launches["tq_append"][-1]
    assert last["past"] == [lengths[0] - 1] * 2 and last["slots"] == [row.slot for row in cache.turboquant_rows[0]]
    assert last["table"].tolist() == tables
    pool = cache.allocator.turboquant_layers[0]
    assert pool.used_pages() == sum(len(t) for t in tables)
    out = cache.turboquant_single_token_decode_attention(0, torch.zeros(2, 8, 1, 64), scaling=1.0,
                                                         num_key_value_groups=4)
    assert out.shape == (2, 8, 1, 64) and launches["tq_decode"][-1]["lengths"] == lengths
    cache.release()
    assert pool.used_pages() == 0 and len(pool.free_slots) == pool.slot_capacity()


def test_turboquant_stack_split_compact_move_rows_without_copies(launches):
    config = _config(block=4)
    allocator = Qwen3PageAllocator(config)
    make = lambda: Qwen3DynamicCache(config, allocator=allocator, kv_cache_quantization="turboquant",
                                     kv_cache_quant_bits=2, kv_cache_residual_len=2)
    singles = [make() for _ in range(3)]
    for idx, cache in enumerate(singles):
        kv = torch.zeros(1, 2, 5 + idx, 64)
        cache.update(kv, kv, 0, require_dense_cache=False)
    rows = [cache.turboquant_rows[0][0] for cache in singles]
    stacked = Qwen3DynamicCache.stack(singles, config, clone_turboquant_rows=False)
    assert stacked.get_seq_lengths().tolist() == [5, 6, 7]
    assert all(a is b for a, b in zip(stacked.turboquant_rows[0], rows))
    kv = torch.zeros(3, 2, 1, 64)
    stacked.update(kv, kv, 0, require_dense_cache=False)
    assert launches["tq_append"][-1]["past"] == [5, 6, 7]
    assert launches["tq_append"][-1]["table"].tolist() == [rows[0].block_table + [-1], rows[1].block_table,
                                                            rows[2].block_table]
    pool = allocator.turboquant_layers[0]
    used = pool.used_pages()
    compacted = stacked.compact_batch_rows([2, 0])
    assert compacted.get_seq_lengths().tolist() == [8, 6]
    assert compacted.turboquant_rows[0][0] is rows[2] and compacted.turboquant_rows[0][1] is rows[0]
    assert rows[1].length == 0 and pool.used_pages() == used - 2  # row 1 held two pages; both went back to the pool
    parts = compacted.split_batch(clone_turboquant_rows=False)
    assert [p.get_seq_length() for p in parts] == [8, 6] and parts[0].turboquant_rows[0][0] is rows[2]
    with pytest.raises(ValueError):
        compacted.compact_batch_rows([0, 0])
    with pytest.raises(IndexError):
        compacted.compact_batch_rows([5])
    with pytest.raises(ValueError, match="different allocators"):
        Qwen3DynamicCache.stack([make(), Qwen3DynamicCache(config)], config)


def test_prefix_sharing_maps_full_prompt_blocks_by_reference(launches):
    """ops.py:779-857: the second sequence with the same prompt reuses the full blocks of the first."""
    config = _config(block=4)
    allocator = Qwen3PageAllocator(config)
    prompt = torch.arange(10).reshape(1, 10)
    first = Qwen3DynamicCache(config, allocator=allocator, batch_size=1)
    first.set_prompt_token_ids(prompt)
    kv = torch.zeros(1, 1, 10, 8)
    first.update(kv, kv, 0, require_dense_cache=False)
    assert first.page_tables[0][0] == [0, 1, 2] and launches["page_write"][-1]["tokens"] == 10
    second = Qwen3DynamicCache(config, allocator=allocator, batch_size=1)
    second.set_prompt_token_ids(prompt)
    second.update(kv, kv, 0, require_dense_cache=False)
    assert second.page_tables[0][0] == [0, 1, 3]
    assert launches["page_write"][-1]["tokens"] == 2 and launches["page_write"][-1]["past"] == [8]
    assert allocator.layers[0]._refcount[0] == 2
    first.release()
    assert allocator.layers[0]._refcount[0] == 1 and allocator.prefix_block_pool.lookup(0, (0, 1, 2, 3)) == 0
    second.release()
    assert allocator.prefix_block_pool.lookup(0, (0, 1, 2, 3)) is None


def test_prefix_block_pool_semantics():
    pool = PrefixBlockPool()
    pool.register(0, (1, 2), 7)
    pool.register(0, (1, 2), 9)  # first registration wins
    pool.register(1, (1, 2), 7)
    assert pool.lookup(0, (1, 2)) == 7 and pool.lookup(1, (1, 2)) == 7 and pool.lookup(0, (3,)) is None
    pool.discard_page(0, 7)
    assert pool.lookup(0, (1, 2)) is None and pool.lookup(1, (1, 2)) == 7
    pool.clear_layer(1)
    assert pool.lookup(1, (1, 2)) is None


def test_constructor_validation_and_flag_semantics():
    config = _config()
    with pytest.raises(ValueError, match="quantization mode"):
        Qwen3DynamicCache(config, kv_cache_quantization="int8")
    with pytest.raises(ValueError, match="bit-width"):
        Qwen3DynamicCache(config, kv_cache_quantization="turboquant", kv_cache_quant_bits=5)
    cache = Qwen3DynamicCache(config, kv_cache_quantization=" TurboQuant ", kv_cache_residual_len=0)
    assert cache.kv_cache_residual_len == 1 and cache.uses_turboquant_for_layer(0)
    mixed = KVCacheConfig(num_hidden_layers=2, layer_types=("linear_attention", "full_attention"))
    cache = Qwen3DynamicCache(mixed, kv_cache_quantization="turboquant")
    assert not cache.uses_turboquant_for_layer(0) and cache.uses_turboquant_for_layer(1)
    with pytest.raises(ValueError, match="batch size mismatch"):
        sized = Qwen3DynamicCache(config, batch_size=2)
        sized._ensure_batch_size(3)


def test_cpu_tensors_are_rejected_without_a_fallback():
    cache = Qwen3DynamicCache(_config(), batch_size=1)
    kv = torch.zeros(1, 2, 3, 64)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        cache.update(kv, kv, 0, require_dense_cache=False)
    row = TurboQuantKVRow(bits=4, residual_len=2)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        row.append(torch.zeros(2, 3, 64), torch.zeros(2, 3, 64))


def test_quantizer_tables_agree_with_oracle():
    for dim in (64, 128, 256):
        for stream in (0, 1):
            np.testing.assert_array_equal(np.array(tq_tables.sign_vector(dim, stream), dtype=np.float32),
                                          oracle.signs(dim, stream))
        for bits in (2, 3, 4):
            cent, bnd = tq_tables.codebook(dim, bits - 1)
            want_cent, want_bnd = oracle.codebook(dim, bits - 1)
            np.testing.assert_array_equal(np.array(cent, dtype=np.float32), want_cent)
            np.testing.assert_array_equal(np.array(bnd, dtype=np.float32), want_bnd)
            tables = tq_tables.key_tables(head_dim=dim, bits=bits, device="cpu")
            assert tables.centroids.shape == (1 << (bits - 1),) and tables.boundaries.shape == ((1 << (bits - 1)) - 1,)
    root = Path(__file__).resolve().parent.parent
    assert (root / "oracle" / "tq_codebooks.json").read_text() == \
        (root / "anna_b200" / "data" / "tq_codebooks.json").read_text()


def test_packed_prefix_blocks_are_shared_between_sequences(launches):
    """Two single-row TurboQuant caches with the same prompt on one allocator: the second maps the packed pages of the
    shared prefix by reference (and tells the append launch to leave them alone); pages live until their last owner
    lets go and the registry forgets a page the moment it is freed."""
    recorded = []
    original = cache_module.launch_tq_append

    def recording_append(pool, key_states, value_states, table_dev, slots, past, **device_copies):
        recorded.append(device_copies.get("shared_blocks"))
        return original(pool, key_states, value_states, table_dev, slots, past, **device_copies)

    cache_module.launch_tq_append = recording_append
    try:
        config = _config(block=4)
        allocator = Qwen3PageAllocator(config)
        prompt = torch.arange(100, 130).view(1, -1)  # 30 tokens

        def prefill(tokens):
            cache = Qwen3DynamicCache(config, allocator=allocator, kv_cache_quantization="turboquant",
                                      kv_cache_quant_bits=4, kv_cache_residual_len=6)
            cache.set_prompt_token_ids(tokens)
            states = torch.zeros(1, 2, int(tokens.shape[1]), 32, dtype=torch.bfloat16)
            cache.update(states, states, 0, require_dense_cache=False)
            return cache

        first = prefill(prompt)
        table_a = list(first.turboquant_rows[0][0].block_table)
        assert len(table_a) == 6 and recorded[-1] is None             # 24 packed tokens = 6 blocks, nothing shared
        second = prefill(prompt)
        table_b = second.turboquant_rows[0][0].block_table
        assert table_b == table_a                                      # all six full blocks mapped by reference
        mask = recorded[-1]
        assert mask is not None and int(mask.view(-1)[0]) == 0b111111
        other = prefill(torch.cat((prompt[:, :9], prompt[:, 9:] + 1000), dim=1))
        table_c = other.turboquant_rows[0][0].block_table
        assert table_c[:2] == table_a[:2] and not set(table_c[2:]) & set(table_a)   # prefix of 8 tokens = 2 blocks
        pool = allocator.turboquant_layers[0]
        assert pool.used_pages() == 6 + 4
        # growth of one sequence past the prompt never touches the shared pages
        step = torch.zeros(1, 2, 1, 32, dtype=torch.bfloat16)
        for _ in range(5):
            second.update(step, step, 0, require_dense_cache=False)
        assert second.turboquant_rows[0][0].block_table[:6] == table_a
        first.release()
        assert pool.used_pages() == 6 + 4 + 2          # second still owns the six, plus its two new blocks
        third = prefill(prompt)
        assert third.turboquant_rows[0][0].block_table == table_a
        for cache in (second, third, other):
            cache.release()
        assert pool.used_pages() == 0
        assert not allocator.packed_prefix_block_pool._page_of
    finally:
        cache_module.launch_tq_append = original


def test_clone_maps_pages_by_reference_and_copies_the_last_block_on_first_write(launches):
    """clone() (ops.py:1323-1381) takes no page: both caches map the same pages with two owners each.  The first
    append into the partly filled last block copies that one page; full blocks stay shared until release."""
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=4)
    source = Qwen3DynamicCache(config, batch_size=1)
    k = torch.arange(1 * 2 * 10 * 8, dtype=torch.float32).reshape(1, 2, 10, 8)
    source.update(k, k + 0.5, 0, require_dense_cache=False)
    layer = source.allocator.layers[0]
    pages_before = list(source.page_tables[0][0])
    assert len(pages_before) == 3 and layer.used_pages() == 3
    # the launches are recorders here, so put recognisable bytes into the last page by hand
    layer.key_pages[pages_before[2]].fill_(7.0)
    clone = source.clone()
    assert clone.page_tables[0][0] == pages_before and layer.used_pages() == 3
    assert [layer.page_owners(pid) for pid in pages_before] == [2, 2, 2]
    one = torch.zeros(1, 2, 1, 8)
    clone.update(one, one, 0, require_dense_cache=False)            # token 10 lands in the partly filled block 2
    assert clone.page_tables[0][0][:2] == pages_before[:2] and clone.page_tables[0][0][2] != pages_before[2]
    assert source.page_tables[0][0] == pages_before
    assert [layer.page_owners(pid) for pid in pages_before] == [2, 2, 1] and layer.used_pages() == 4
    assert torch.equal(layer.key_pages[clone.page_tables[0][0][2]], layer.key_pages[pages_before[2]])
    # the device table of the clone carries the new page id
    assert launches["page_write"][-1]["table"][0].tolist()[:3] == clone.page_tables[0][0]
    source.update(one, one, 0, require_dense_cache=False)           # the source is the only owner of its last page now
    assert source.page_tables[0][0] == pages_before and layer.used_pages() == 4
    clone.release()
    assert [layer.page_owners(pid) for pid in pages_before] == [1, 1, 1] and layer.used_pages() == 3
    source.release()
    assert layer.used_pages() == 0


def test_turboquant_clone_shares_packed_pages_until_the_partial_block_is_written(launches):
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=4)
    source = Qwen3DynamicCache(config, batch_size=2, kv_cache_quantization="turboquant", kv_cache_quant_bits=4,
                               kv_cache_residual_len=3)
    k = torch.zeros(2, 2, 9, 64, dtype=torch.bfloat16)
    source.update(k, k, 0, require_dense_cache=False)               # 6 quantized tokens: blocks 0 (full) and 1 (half)
    pool = source.allocator.turboquant_layers[0]
    tables = [list(row.block_table) for row in source.turboquant_rows[0]]
    assert all(len(t) == 2 for t in tables) and pool.used_pages() == 4
    clone = source.clone()
    assert [list(row.block_table) for row in clone.turboquant_rows[0]] == tables and pool.used_pages() == 4
    assert {row.slot for row in clone.turboquant_rows[0]}.isdisjoint({row.slot for row in source.turboquant_rows[0]})
    one = torch.zeros(2, 2, 1, 64, dtype=torch.bfloat16)
    clone.update(one, one, 0, require_dense_cache=False)            # quantizes token 6 into the shared half block
    for row, before in zip(clone.turboquant_rows[0], tables):
        assert row.block_table[0] == before[0] and row.block_table[1] != before[1]
    assert pool.used_pages() == 6
    sent = launches["tq_append"][-1]["table"]
    assert [sent[i].tolist()[:2] for i in range(2)] == [row.block_table for row in clone.turboquant_rows[0]]
    assert [list(row.block_table) for row in source.turboquant_rows[0]] == tables
    clone.release()
    assert pool.used_pages() == 4 and all(pool.page_owners(pid) == 1 for t in tables for pid in t)


def test_one_pass_release_equals_page_by_page_release():
    """release_many (both its all-private fast path and its general path) leaves the free list, the owner counts and
    the callbacks exactly as releasing the pages one by one does (ops.py:214-233 semantics: unknown ids are ignored,
    a shared page only loses an owner)."""
    import random

    from anna_b200.pools import _PageBook

    rng = random.Random(3)
    for case in range(40):
        freed_a: list[int] = []
        freed_b: list[int] = []
        a, b = _PageBook(freed_a.append), _PageBook(freed_b.append)
        for book in (a, b):
            book.take(64, 0)
        shared = rng.sample(range(64), rng.choice([0, 0, 3, 10]))
        for page in shared:
            a.retain(page)
            b.retain(page)
        for _ in range(4):
            ids = rng.sample(range(80), rng.randint(1, 40))  # ids above 63 were never handed out
            if rng.random() < 0.3:
                ids = ids + ids[:2]                           # a page named twice in one call
            a.release_many(list(ids))
            for page in ids:
                b.release(page)
            assert a.free_pages == b.free_pages and a.refcount == b.refcount and freed_a == freed_b, case
            assert a._shared == sum(1 for rc in a.refcount.values() if rc > 1)


def test_block_table_array_follows_the_list():
    """TurboQuantKVRow.table_array(): an int32 mirror that converts only what changed since the last call."""
    from anna_b200.turboquant import TurboQuantKVRow

    row = TurboQuantKVRow(bits=4, residual_len=8)
    assert row.table_array().tolist() == []
    row.block_table.extend([5, 9, 2])
    assert row.table_array().tolist() == [5, 9, 2] and row.table_array().dtype == np.int32
    row.block_table.extend(range(100, 140))                      # grows past the first allocation
    assert row.table_array().tolist() == row.block_table
    row.block_table[1] = 77                                      # what copy on write does ...
    row._table_np_valid = min(row._table_np_valid, 1)            # ... together with this
    assert row.table_array().tolist() == row.block_table
    row.block_table = []                                         # release()
    row._table_np_valid = 0
    row.block_table.extend([4, 4, 4])
    assert row.table_array().tolist() == [4, 4, 4]
