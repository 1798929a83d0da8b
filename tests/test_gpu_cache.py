"""GPU: the cache object end to end on the un-quantized paged path and the TurboQuant dense views."""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from anna_b200 import KVCacheConfig, Qwen3DynamicCache, Qwen3PageAllocator, fused_ops
from tests.helpers import TqPair, outlier_kv, reference_decode, to_np

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def test_paged_update_then_decode_matches_oracle(cuda_device):
    """Config-2-like: ragged rows, pages handed out by the allocator, decode through paged_attention_state."""
    torch.manual_seed(0)
    config = KVCacheConfig(num_hidden_layers=2, cache_block_size=16)
    allocator = Qwen3PageAllocator(config)
    lengths = [37, 16, 90]
    heads, kv_heads, dim = 16, 4, 128
    caches, dense = [], []
    for n in lengths:  # prefill one row at a time, as the scheduler does, then stack
        cache = Qwen3DynamicCache(config, allocator=allocator)
        k = torch.randn(1, kv_heads, n, dim, device=cuda_device, dtype=torch.bfloat16)
        v = torch.randn_like(k)
        gathered_k, gathered_v, past = cache.update(k, v, 1)
        assert past.tolist() == [0] and torch.equal(gathered_k, k) and torch.equal(gathered_v, v)
        caches.append(cache)
        dense.append((k, v))
    stacked = Qwen3DynamicCache.stack(caches, config)
    for step in range(3):
        k1 = torch.randn(3, kv_heads, 1, dim, device=cuda_device, dtype=torch.bfloat16)
        v1 = torch.randn_like(k1)
        none_k, none_v, past = stacked.update(k1, v1, 1, require_dense_cache=False)
        assert none_k is None and none_v is None and past.tolist() == [n + step for n in lengths]
        dense = [(torch.cat((k, k1[i:i + 1]), dim=2), torch.cat((v, v1[i:i + 1]), dim=2))
                 for i, (k, v) in enumerate(dense)]
        key_pages, value_pages, table, visible = stacked.paged_attention_state(1)
        assert table.dtype == torch.int32 and visible.tolist() == [n + step + 1 for n in lengths]
        query = torch.randn(3, heads, 1, dim, device=cuda_device, dtype=torch.bfloat16)
        out = fused_ops.run_paged_gqa_decode_fused(query=query, key_pages=key_pages, value_pages=value_pages,
                                                   page_table=table, visible_lengths=visible, scaling=dim ** -0.5)
        for i, (k, v) in enumerate(dense):
            want = reference_decode(query[i:i + 1], k, v, [k.shape[2]], dim ** -0.5)
            np.testing.assert_allclose(to_np(out[i:i + 1]), want, atol=2e-2, rtol=2e-2)
    gathered_k, gathered_v, visible = stacked._gather_layer_cache(1)
    for i, (k, v) in enumerate(dense):
        assert torch.equal(gathered_k[i, :, :k.shape[2]], k[0]) and torch.equal(gathered_v[i, :, :v.shape[2]], v[0])
        assert torch.count_nonzero(gathered_k[i, :, k.shape[2]:]) == 0
    used = allocator.layers[1].used_pages()
    clone = stacked.clone()  # copy on write: the clone maps the same pages, nothing is taken
    assert clone.page_tables[1] == stacked.page_tables[1] and allocator.layers[1].used_pages() == used
    ck, cv, _ = clone._gather_layer_cache(1)
    assert torch.equal(ck, gathered_k) and torch.equal(cv, gathered_v)
    clone.release()
    assert allocator.layers[1].used_pages() == used
    stacked.release()
    assert allocator.layers[1].used_pages() == 0 and allocator.layers[0].capacity() == 0


def test_paged_block_tables_on_device_match_reference(cuda_device):
    want = json.loads((GOLDEN / "paged_block_tables.json").read_text())
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=16)
    cache = Qwen3DynamicCache(config, batch_size=2)
    kv = torch.zeros(2, 2, 40, 64, device=cuda_device, dtype=torch.bfloat16)
    cache.update(kv, kv, 0, require_dense_cache=False)
    for _ in range(9):
        cache.update(kv[:, :, :1], kv[:, :, :1], 0, require_dense_cache=False)
    state = cache.paged_attention_state(0)
    assert state[2].cpu().tolist() == want["after_9_steps"]


def test_prefix_shared_pages_are_not_rewritten(cuda_device):
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=4)
    allocator = Qwen3PageAllocator(config)
    prompt = torch.arange(10).reshape(1, 10)
    first = Qwen3DynamicCache(config, allocator=allocator)
    first.set_prompt_token_ids(prompt)
    k = torch.randn(1, 2, 10, 64, device=cuda_device, dtype=torch.bfloat16)
    first.update(k, k, 0, require_dense_cache=False)
    second = Qwen3DynamicCache(config, allocator=allocator)
    second.set_prompt_token_ids(prompt)
    other = torch.randn_like(k)
    got_k, _, _ = second.update(other, other, 0)
    assert second.page_tables[0][0][:2] == first.page_tables[0][0][:2]
    assert torch.equal(got_k[:, :, :8], k[:, :, :8])      # shared blocks keep the first sequence's bytes
    assert torch.equal(got_k[:, :, 8:], other[:, :, 8:])  # the private tail is this sequence's


def test_turboquant_dense_view_and_lifecycle(cuda_device):
    """update(require_dense_cache=True) returns [de-quantized prefix | exact window] (ops.py:642-660)."""
    pair = TqPair(device=cuda_device, batch=2, kv_heads=2, head_dim=128, bits=4, residual_len=4, block_size=16,
                  dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(3)
    k = outlier_kv(gen, (2, 2, 21, 128), torch.bfloat16)
    v = outlier_kv(gen, (2, 2, 21, 128), torch.bfloat16)
    dense_k, dense_v, past = pair.cache.update(k.to(cuda_device), v.to(cuda_device), 0)
    for b, row in enumerate(pair.rows):
        row.append(to_np(k[b]), to_np(v[b]))
        want_k, want_v = row.materialize()
        np.testing.assert_array_equal(to_np(dense_v[b]), want_v)
        np.testing.assert_array_equal(to_np(dense_k[b, :, 17:]), want_k[:, 17:])
        np.testing.assert_allclose(to_np(dense_k[b]), want_k, atol=6e-2, rtol=2e-2)
    assert float(((dense_k.float().cpu() - k.float()) ** 2).mean()) < 1.0  # tests/test_model_shapes.py:374
    assert past.tolist() == [0, 0] and dense_k.shape == (2, 2, 21, 128)
    pair.assert_bit_exact()
    pool = pair.pool
    clone = pair.cache.clone()
    # the clone maps the same packed pages (copy on write): no page is taken until one of the two appends
    assert pool.used_pages() == 4 and clone.turboquant_rows[0][0].block_table == pair.cache.turboquant_rows[0][0].block_table
    ck, cv, _ = clone._gather_layer_cache(0)
    assert torch.equal(ck, dense_k) and torch.equal(cv, dense_v)
    clone.release()
    pair.cache.release()
    assert pool.used_pages() == 0
    assert pair.cache.allocator.trim() > 0 and pool.packed_pages is None


def test_packed_prefix_sharing_gives_identical_decode(cuda_device):
    """A sequence that maps the packed pages of a shared prompt prefix decodes bit-identically to one that packed
    everything itself, also after the sequence that first wrote those pages is gone."""
    torch.manual_seed(8)
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=16)
    heads, kv_heads, dim, residual = 8, 2, 128, 8
    prompt = torch.arange(1000, 1100).view(1, -1)                     # 100 tokens: 92 packed = 5 full blocks + 12
    k = torch.randn(1, kv_heads, 100, dim, device=cuda_device, dtype=torch.bfloat16)
    v = torch.randn_like(k)
    k_tail = torch.randn(1, kv_heads, 40, dim, device=cuda_device, dtype=torch.bfloat16)  # a different continuation
    v_tail = torch.randn_like(k_tail)

    def run(allocator, tokens, keys, values):
        cache = Qwen3DynamicCache(config, allocator=allocator, kv_cache_quantization="turboquant",
                                  kv_cache_quant_bits=4, kv_cache_residual_len=residual)
        cache.set_prompt_token_ids(tokens)
        cache.update(keys, values, 0, require_dense_cache=False)
        return cache

    shared_alloc = Qwen3PageAllocator(config)
    writer = run(shared_alloc, prompt, k, v)
    longer_prompt = torch.cat((prompt, torch.arange(5000, 5040).view(1, -1)), dim=1)
    k_long, v_long = torch.cat((k, k_tail), dim=2), torch.cat((v, v_tail), dim=2)
    reader = run(shared_alloc, longer_prompt, k_long, v_long)
    table_w = writer.turboquant_rows[0][0].block_table
    table_r = reader.turboquant_rows[0][0].block_table
    assert table_r[:5] == table_w[:5] and not set(table_r[5:]) & set(table_w)
    alone = run(Qwen3PageAllocator(config), longer_prompt, k_long, v_long)   # nothing to share with
    query = torch.randn(1, heads, 1, dim, device=cuda_device, dtype=torch.bfloat16)

    def decode(cache):
        return cache.turboquant_single_token_decode_attention(0, query, scaling=dim ** -0.5,
                                                              num_key_value_groups=heads // kv_heads)

    want = decode(alone)
    assert torch.equal(decode(reader), want)
    dense_alone = alone._gather_layer_cache(0)
    dense_reader = reader._gather_layer_cache(0)
    assert torch.equal(dense_reader[0], dense_alone[0]) and torch.equal(dense_reader[1], dense_alone[1])
    writer.release()
    assert torch.equal(decode(reader), want)
    step_k = torch.randn(1, kv_heads, 1, dim, device=cuda_device, dtype=torch.bfloat16)
    for cache in (reader, alone):
        cache.update(step_k, step_k, 0, require_dense_cache=False)
    assert torch.equal(decode(reader), decode(alone))
    reader.release()
    assert shared_alloc.turboquant_layers[0].used_pages() == 0
    assert not shared_alloc.packed_prefix_block_pool._page_of


def test_turboquant_batched_dense_view_matches_row_materialize(cuda_device):
    """The one-launch dense view of a ragged batch (shorter than the window, exactly the window, many pages) equals each
    row's own materialize() and is zero past the row's length, whatever the pages held before."""
    torch.manual_seed(4)
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=16)
    allocator = Qwen3PageAllocator(config)
    lengths = [3, 8, 9, 70, 200]
    kv_heads, dim, residual = 2, 128, 8
    caches, inputs = [], []
    for n in lengths:
        cache = Qwen3DynamicCache(config, allocator=allocator, kv_cache_quantization="turboquant",
                                  kv_cache_quant_bits=3, kv_cache_residual_len=residual)
        k = torch.randn(1, kv_heads, n, dim, device=cuda_device, dtype=torch.bfloat16)
        v = torch.randn_like(k)
        cache.update(k, v, 0, require_dense_cache=False)
        caches.append(cache)
        inputs.append((k, v))
    stacked = Qwen3DynamicCache.stack(caches, config)
    keys, values, visible = stacked._gather_layer_cache(0)
    assert keys.shape == (len(lengths), kv_heads, max(lengths), dim) and visible.tolist() == lengths
    for b, n in enumerate(lengths):
        row_k, row_v = stacked.turboquant_rows[0][b].materialize()
        assert torch.equal(keys[b, :, :n], row_k) and torch.equal(values[b, :, :n], row_v)
        assert torch.count_nonzero(keys[b, :, n:]) == 0 and torch.count_nonzero(values[b, :, n:]) == 0
        tail = min(n, residual)
        assert torch.equal(keys[b, :, n - tail:n], inputs[b][0][0, :, n - tail:]) and torch.isfinite(keys[b]).all()


def test_turboquant_churn_matches_oracle(cuda_device):
    """Configuration-4-like churn at small scale: every step some sequences finish (pages and ring slots go back to the
    pool) and new ones are admitted with a chunked prefill, the rest decode one token.  Block tables must follow the
    oracle allocator exactly through the churn and every decode must match the oracle rows."""
    import random

    import oracle
    from tests.helpers import DTYPE_CODE, TQ_ATOL

    rng = random.Random(9)
    gen = torch.Generator().manual_seed(9)
    heads, kv_heads, dim, bits, residual, block = 8, 2, 128, 3, 8, 16
    dtype = torch.bfloat16
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=block)
    allocator = Qwen3PageAllocator(config)
    oracle_allocator = oracle.OracleLayerAllocator()

    def admit(tokens: int):
        cache = Qwen3DynamicCache(config, allocator=allocator, kv_cache_quantization="turboquant",
                                  kv_cache_quant_bits=bits, kv_cache_residual_len=residual)
        row = oracle.OracleTurboQuantRow(bits=bits, residual_len=residual, dtype=DTYPE_CODE[dtype], block_size=block,
                                         allocator=oracle_allocator)
        done = 0
        while done < tokens:  # chunked prefill
            step = min(40, tokens - done)
            k = torch.randn(1, kv_heads, step, dim, generator=gen).to(dtype)
            v = torch.randn(1, kv_heads, step, dim, generator=gen).to(dtype)
            cache.update(k.to(cuda_device), v.to(cuda_device), 0, require_dense_cache=False)
            row.append(to_np(k[0]), to_np(v[0]))
            done += step
        return cache, row

    live = [admit(rng.randint(5, 150)) for _ in range(6)]
    for step in range(8):
        # one or two sequences finish; their pages return in the reference's order, then new ones come in
        for _ in range(rng.randint(1, 2)):
            cache, row = live.pop(rng.randrange(len(live)))
            cache.release()
            oracle_allocator.release_pages(row.block_table)
        while len(live) < 6:
            live.append(admit(rng.randint(5, 150)))
        # rows move into the batch and back out as handles (no page is copied or allocated)
        batch = Qwen3DynamicCache.stack([cache for cache, _ in live], config, clone_turboquant_rows=False)
        k1 = torch.randn(len(live), kv_heads, 1, dim, generator=gen).to(dtype)
        v1 = torch.randn(len(live), kv_heads, 1, dim, generator=gen).to(dtype)
        batch.update(k1.to(cuda_device), v1.to(cuda_device), 0, require_dense_cache=False)
        query = torch.randn(len(live), heads, 1, dim, generator=gen).to(dtype)
        out = batch.turboquant_single_token_decode_attention(0, query.to(cuda_device), scaling=dim ** -0.5,
                                                             num_key_value_groups=heads // kv_heads)
        for b, (_, row) in enumerate(live):
            row.append(to_np(k1[b]), to_np(v1[b]))
            assert batch.turboquant_rows[0][b].block_table == row.block_table, (step, b)
            want = row.decode_attention(to_np(query[b, :, 0]), scaling=dim ** -0.5)
            np.testing.assert_allclose(to_np(out[b, :, 0]), want, atol=TQ_ATOL[dtype], rtol=TQ_ATOL[dtype])
        live = [(cache, row) for cache, (_, row) in zip(batch.split_batch(clone_turboquant_rows=False), live)]
    pool = allocator.turboquant_layers[0]
    assert pool.used_pages() == sum(len(row.block_table) for _, row in live)
    for cache, _ in live:
        cache.release()
    assert pool.used_pages() == 0


def test_clone_is_copy_on_write_for_packed_and_unquantized_pages(cuda_device):
    """clone() maps pages by reference; after the clone and its source append different tokens, each decodes like an
    oracle row that saw its own history, and the pages they still share were not disturbed (ops.py:1323-1381 copies
    every page instead)."""
    import copy

    gen = torch.Generator().manual_seed(12)
    # -- TurboQuant rows: 70 tokens, window 6 -> 64 quantized = 4 full blocks; +5 tokens -> a partly filled block ------
    pair = TqPair(device=cuda_device, batch=2, kv_heads=2, head_dim=128, bits=4, residual_len=6, block_size=16,
                  dtype=torch.bfloat16)
    for tokens in (70, 5):
        pair.append(outlier_kv(gen, (2, 2, tokens, 128), torch.bfloat16),
                    outlier_kv(gen, (2, 2, tokens, 128), torch.bfloat16))
    pool = pair.pool
    used = pool.used_pages()
    clone = pair.cache.clone()
    clone_rows = [copy.deepcopy(row) for row in pair.rows]
    assert pool.used_pages() == used
    k_a, v_a = outlier_kv(gen, (2, 2, 3, 128), torch.bfloat16), outlier_kv(gen, (2, 2, 3, 128), torch.bfloat16)
    k_b, v_b = outlier_kv(gen, (2, 2, 20, 128), torch.bfloat16), outlier_kv(gen, (2, 2, 20, 128), torch.bfloat16)
    clone.update(k_b.to(cuda_device), v_b.to(cuda_device), 0, require_dense_cache=False)
    for b, row in enumerate(clone_rows):
        row.append(to_np(k_b[b]), to_np(v_b[b]))
    pair.append(k_a, v_a)               # the source goes on with other tokens
    pair.assert_bit_exact()             # ... and its codes are still exactly its own
    query = torch.randn(2, 8, 1, 128, generator=gen).to(torch.bfloat16)
    for cache, rows in ((pair.cache, pair.rows), (clone, clone_rows)):
        out = cache.turboquant_single_token_decode_attention(0, query.to(cuda_device), scaling=128 ** -0.5,
                                                             num_key_value_groups=4)
        want = np.stack([row.decode_attention(to_np(query[b, :, 0]), scaling=128 ** -0.5)
                         for b, row in enumerate(rows)])[:, :, None, :]
        np.testing.assert_allclose(to_np(out), want, atol=4e-2, rtol=4e-2)
    shared = set(pair.cache.turboquant_rows[0][0].block_table) & set(clone.turboquant_rows[0][0].block_table)
    assert len(shared) == 4             # the four full blocks are still one copy
    clone.release()
    pair.cache.release()
    assert pool.used_pages() == 0

    # -- un-quantized pages ---------------------------------------------------------------------------------------------
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=16)
    source = Qwen3DynamicCache(config, batch_size=2)
    k0 = torch.randn(2, 2, 37, 128, generator=gen).to(torch.bfloat16)
    v0 = torch.randn(2, 2, 37, 128, generator=gen).to(torch.bfloat16)
    source.update(k0.to(cuda_device), v0.to(cuda_device), 0, require_dense_cache=False)
    layer = source.allocator.layers[0]
    used = layer.used_pages()
    other = source.clone()
    assert layer.used_pages() == used
    k1 = torch.randn(2, 2, 4, 128, generator=gen).to(torch.bfloat16)
    v1 = torch.randn(2, 2, 4, 128, generator=gen).to(torch.bfloat16)
    k2 = torch.randn(2, 2, 30, 128, generator=gen).to(torch.bfloat16)
    v2 = torch.randn(2, 2, 30, 128, generator=gen).to(torch.bfloat16)
    source.update(k1.to(cuda_device), v1.to(cuda_device), 0, require_dense_cache=False)
    other.update(k2.to(cuda_device), v2.to(cuda_device), 0, require_dense_cache=False)
    histories = {id(source): (torch.cat([k0, k1], 2), torch.cat([v0, v1], 2)),
                 id(other): (torch.cat([k0, k2], 2), torch.cat([v0, v2], 2))}
    for cache in (source, other):
        keys, values = histories[id(cache)]
        key_pages, value_pages, table, visible = cache.paged_attention_state(0)
        out = fused_ops.run_paged_gqa_decode_fused(query=query.to(cuda_device), key_pages=key_pages,
                                                   value_pages=value_pages, page_table=table, visible_lengths=visible,
                                                   scaling=128 ** -0.5)
        for b in range(2):
            want = oracle.gqa_decode(to_np(query[b, :, 0]), to_np(keys[b]), to_np(values[b]), 128 ** -0.5)
            np.testing.assert_allclose(to_np(out[b, :, 0]), want, atol=2e-2, rtol=2e-2)
        dense_k, dense_v, _ = cache._gather_layer_cache(0)     # the gather kernel sees the same history
        assert torch.equal(dense_k.cpu(), keys) and torch.equal(dense_v.cpu(), values)
    other.release()
    source.release()
    assert layer.used_pages() == 0
