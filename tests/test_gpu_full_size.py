"""GPU: the benchmark configurations at full size, checked through properties that need no CPU oracle.

The oracle finishes small cases in seconds but not 64 sequences of 32768 tokens, so at full size two independent kernel
paths are played against each other: the paged / packed decode on one side, the dense decode over the gathered (or
de-quantized) cache on the other.  They share no tile, schedule or merge code, so agreement within the tolerance of the
small-size oracle tests carries those results to the full shapes.  A second property: sequences are independent, so a
row decoded alone must give the output it gives inside the batch (up to rounding: the split points of the schedule
depend on the batch)."""
from __future__ import annotations

import pytest
import torch

from anna_b200 import KVCacheConfig, Qwen3DynamicCache, Qwen3PageAllocator, fused_ops

pytestmark = pytest.mark.gpu


def test_config2_full_size_paged_decode_agrees_with_dense_decode(cuda_device):
    """32 sequences, 32 q / 8 kv heads, D=128, page 16, contexts uniform in [1024, 8192], permuted block tables."""
    torch.manual_seed(21)
    batch, heads, kv_heads, dim, page = 32, 32, 8, 128, 16
    lengths = torch.randint(1024, 8193, (batch,), generator=torch.Generator().manual_seed(5)).tolist()
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=page)
    allocator = Qwen3PageAllocator(config)
    template = torch.empty(1, kv_heads, 1, dim, device=cuda_device, dtype=torch.bfloat16)
    layer = allocator.layers[0]
    layer.ensure_capacity(sum((n + page - 1) // page for n in lengths) + 8, key_template=template,
                          value_template=template)
    layer.free_pages[:] = torch.randperm(layer.capacity(), generator=torch.Generator().manual_seed(6)).tolist()
    rows = []
    for n in lengths:
        row = Qwen3DynamicCache(config, allocator=allocator)
        k = torch.randn(1, kv_heads, n, dim, device=cuda_device, dtype=torch.bfloat16)
        row.update(k, torch.randn_like(k), 0, require_dense_cache=False)
        rows.append(row)
    cache = Qwen3DynamicCache.stack(rows, config)
    query = torch.randn(batch, heads, 1, dim, device=cuda_device, dtype=torch.bfloat16)
    key_pages, value_pages, table, visible = cache.paged_attention_state(0)
    paged = fused_ops.run_paged_gqa_decode_fused(query=query, key_pages=key_pages, value_pages=value_pages,
                                                 page_table=table, visible_lengths=visible, scaling=dim ** -0.5)
    keys, values, dense_visible = cache._gather_layer_cache(0)
    assert dense_visible.tolist() == lengths
    dense = fused_ops.run_gqa_decode_fused(query=query, key=keys, value=values, visible_lengths=dense_visible,
                                           scaling=dim ** -0.5)
    assert torch.isfinite(paged).all()
    torch.testing.assert_close(paged.float(), dense.float(), atol=2e-2, rtol=2e-2)
    # independence of sequences: a row decoded alone gives what it gives inside the batch
    for b in (0, 17, 31):
        alone = fused_ops.run_paged_gqa_decode_fused(query=query[b:b + 1], key_pages=key_pages, value_pages=value_pages,
                                                     page_table=table[b:b + 1], visible_lengths=visible[b:b + 1],
                                                     scaling=dim ** -0.5)
        torch.testing.assert_close(alone.float(), paged[b:b + 1].float(), atol=2e-2, rtol=2e-2)


def test_config5_shard_full_size_packed_decode_agrees_with_dense_decode(cuda_device):
    """The per-GPU share of configuration 5: 64 sequences x 32768 tokens, 4-bit, 32 q / 8 kv heads, D=128, window 128."""
    torch.manual_seed(22)
    batch, heads, kv_heads, dim, context = 64, 32, 8, 128, 32768
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=16)
    cache = Qwen3DynamicCache(config, batch_size=batch, kv_cache_quantization="turboquant", kv_cache_quant_bits=4,
                              kv_cache_residual_len=128)
    cache.reserve_sequence_capacity(context)
    gen = torch.Generator(device=cuda_device).manual_seed(7)
    for _ in range(context // 4096):
        k = torch.randn(batch, kv_heads, 4096, dim, device=cuda_device, dtype=torch.bfloat16, generator=gen)
        v = torch.randn(batch, kv_heads, 4096, dim, device=cuda_device, dtype=torch.bfloat16, generator=gen)
        cache.update(k, v, 0, require_dense_cache=False)
        del k, v
    query = torch.randn(batch, heads, 1, dim, device=cuda_device, dtype=torch.bfloat16, generator=gen)
    packed = cache.turboquant_single_token_decode_attention(0, query, scaling=dim ** -0.5,
                                                            num_key_value_groups=heads // kv_heads)
    keys, values, visible = cache._gather_layer_cache(0)       # de-quantized prefix + exact window, one launch
    assert keys.shape == (batch, kv_heads, context, dim) and visible.tolist() == [context] * batch
    dense = fused_ops.run_gqa_decode_fused(query=query, key=keys, value=values, visible_lengths=visible.to(cuda_device),
                                           scaling=dim ** -0.5)
    assert torch.isfinite(packed).all()
    # same tolerance as the small TurboQuant cases against the oracle (the dense path rounds K-hat to bf16 first)
    torch.testing.assert_close(packed.float(), dense.float(), atol=4e-2, rtol=4e-2)
    pool = cache.allocator.turboquant_layers[0]
    assert pool.used_pages() == batch * ((context - 128 + 15) // 16)
    cache.release()
    assert pool.used_pages() == 0


# ---------------------------------------------------------------------------------------------------------------
# full shapes against the CPU oracle on a sample of rows (the oracle handles one row of 32768 tokens in seconds)


def _check_rows_against_oracle(cache, host_kv, sample_rows, query, *, bits, residual, heads, kv_heads, dim, page):
    """For each sampled row: feed the very K / V the GPU row received to an oracle row, compare the packed codes and
    metadata of three 16-token pages (first, middle, last) bit for bit, the block count, and the decode output."""
    import numpy as np

    import oracle
    from tests.helpers import TQ_ATOL, error_stats, packed_row_fields, to_np

    pool = cache.allocator.turboquant_layers[0]
    out = cache.turboquant_single_token_decode_attention(0, query, scaling=dim ** -0.5,
                                                         num_key_value_groups=heads // kv_heads)
    assert torch.isfinite(out).all()
    for b in sample_rows:
        keys, values = host_kv[b]
        orc = oracle.OracleTurboQuantRow(bits=bits, residual_len=residual, dtype=oracle.DTYPE_BF16, block_size=page,
                                         allocator=oracle.OracleLayerAllocator(), keep_decode_cache=True)
        orc.append(keys, values)
        row = cache.turboquant_rows[0][b]
        assert (row.length, row.quantized_length) == (orc.length, orc.quantized_length)
        assert len(row.block_table) == len(orc.block_table)
        lq = orc.quantized_length
        want_codes = oracle.pack_key_codes(orc.idx, orc.sign, bits)
        for first in sorted({0, (lq // 2) // page * page, max(0, (lq - 1) // page * page)}):
            last = min(lq, first + page)
            got = packed_row_fields(pool, row, first, last)
            np.testing.assert_array_equal(got["kcodes"], want_codes[:, first:last])
            np.testing.assert_array_equal(got["norms"].view(np.uint32), orc.norms[:, first:last].view(np.uint32))
            np.testing.assert_array_equal(got["rnorms"].view(np.uint32), orc.rnorms[:, first:last].view(np.uint32))
            np.testing.assert_array_equal(got["vdata"], orc.vdata[:, first:last])
            np.testing.assert_array_equal(got["vscales"].view(np.uint32), orc.vscales[:, first:last].view(np.uint32))
            np.testing.assert_array_equal(got["vzeros"].view(np.uint32), orc.vzeros[:, first:last].view(np.uint32))
        want = orc.decode_attention(to_np(query[b, :, 0]), scaling=dim ** -0.5, blas=True)
        max_abs, rel = error_stats(to_np(out[b, :, 0]), want)
        # 16-bit TurboQuant tolerance of the small-size tests (the reference's own, tests/test_fused_op_xpu.py:703)
        assert max_abs <= TQ_ATOL[torch.bfloat16] and rel <= TQ_ATOL[torch.bfloat16], (b, max_abs, rel)


def test_config5_shard_full_size_sampled_rows_match_oracle(cuda_device):
    """64 sequences x 32768 tokens, 4-bit, 32 q / 8 kv heads, D=128: two rows checked against the oracle."""
    from tests.helpers import to_np

    batch, heads, kv_heads, dim, context, page, bits, residual = 64, 32, 8, 128, 32768, 16, 4, 128
    sample_rows = (3, 61)
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=page)
    cache = Qwen3DynamicCache(config, batch_size=batch, kv_cache_quantization="turboquant", kv_cache_quant_bits=bits,
                              kv_cache_residual_len=residual)
    cache.reserve_sequence_capacity(context)
    gen = torch.Generator(device=cuda_device).manual_seed(31)
    host = {b: ([], []) for b in sample_rows}
    for _ in range(context // 4096):
        k = torch.randn(batch, kv_heads, 4096, dim, device=cuda_device, dtype=torch.bfloat16, generator=gen)
        v = torch.randn(batch, kv_heads, 4096, dim, device=cuda_device, dtype=torch.bfloat16, generator=gen)
        cache.update(k, v, 0, require_dense_cache=False)
        for b in sample_rows:
            host[b][0].append(to_np(k[b]))
            host[b][1].append(to_np(v[b]))
        del k, v
    import numpy as np

    host_kv = {b: (np.concatenate(ks, axis=1), np.concatenate(vs, axis=1)) for b, (ks, vs) in host.items()}
    query = torch.randn(batch, heads, 1, dim, device=cuda_device, dtype=torch.bfloat16, generator=gen)
    _check_rows_against_oracle(cache, host_kv, sample_rows, query, bits=bits, residual=residual, heads=heads,
                               kv_heads=kv_heads, dim=dim, page=page)
    cache.release()


def test_config3_full_size_ragged_rows_match_oracle(cuda_device):
    """64 sequences, contexts uniform in [4096, 32768], 2-bit, 16 q / 2 kv heads, D=256, window 128, per-channel
    log-normal scales (sigma 0.5): the shortest, the longest and one more row checked against the oracle."""
    import numpy as np

    from tests.helpers import to_np

    batch, heads, kv_heads, dim, page, bits, residual = 64, 16, 2, 256, 16, 2, 128
    lengths = torch.randint(4096, 32769, (batch,), generator=torch.Generator().manual_seed(41)).tolist()
    sample_rows = sorted({lengths.index(min(lengths)), lengths.index(max(lengths)), 29})
    config = KVCacheConfig(num_hidden_layers=1, cache_block_size=page)
    allocator = Qwen3PageAllocator(config)
    gen = torch.Generator(device=cuda_device).manual_seed(42)
    channel_scale = torch.exp(0.5 * torch.randn(kv_heads, 1, dim, device=cuda_device, generator=gen))
    rows, host_kv = [], {}
    for b, n in enumerate(lengths):
        row = Qwen3DynamicCache(config, allocator=allocator, batch_size=1, kv_cache_quantization="turboquant",
                                kv_cache_quant_bits=bits, kv_cache_residual_len=residual)
        k = (torch.randn(1, kv_heads, n, dim, device=cuda_device, generator=gen) * channel_scale).to(torch.bfloat16)
        v = (torch.randn(1, kv_heads, n, dim, device=cuda_device, generator=gen) * channel_scale).to(torch.bfloat16)
        row.update(k, v, 0, require_dense_cache=False)
        if b in sample_rows:
            host_kv[b] = (to_np(k[0]), to_np(v[0]))
        rows.append(row)
        del k, v
    cache = Qwen3DynamicCache.stack(rows, config, clone_turboquant_rows=False)
    assert cache.layer_lengths[0] == lengths
    query = torch.randn(batch, heads, 1, dim, device=cuda_device, dtype=torch.bfloat16, generator=gen)
    _check_rows_against_oracle(cache, host_kv, sample_rows, query, bits=bits, residual=residual, heads=heads,
                               kv_heads=kv_heads, dim=dim, page=page)
    # one more decode step on top: append a token per row, decode again, the sampled rows still agree
    k1 = (torch.randn(batch, kv_heads, 1, dim, device=cuda_device, generator=gen) * channel_scale).to(torch.bfloat16)
    v1 = (torch.randn(batch, kv_heads, 1, dim, device=cuda_device, generator=gen) * channel_scale).to(torch.bfloat16)
    cache.update(k1, v1, 0, require_dense_cache=False)
    host_kv = {b: (np.concatenate([kv[0], to_np(k1[b])], axis=1), np.concatenate([kv[1], to_np(v1[b])], axis=1))
               for b, kv in host_kv.items()}
    _check_rows_against_oracle(cache, host_kv, sample_rows, query, bits=bits, residual=residual, heads=heads,
                               kv_heads=kv_heads, dim=dim, page=page)
    cache.release()


def test_config4_prefill_chunk_over_long_context_matches_fp32_attention(cuda_device):
    """cfg4's prefill attention at a length the oracle does not finish in seconds: a 512-token chunk over 32 256 cached
    tokens (253 key tiles of the tensor-memory kernel, 16 q / 4 kv heads, D=128), ragged: the second row is 9 000 tokens
    long.  Floating-point kernel, so the check is a plain fp32 torch attention on the same bf16 inputs: 2e-2 absolute on
    bf16 outputs (values are N(0, 1); rows average thousands of them, so outputs are small and the bound is loose in
    relative terms) and 4e-3 relative L2: the output and P are each rounded to bf16 once (2^-9 / sqrt(3) = 1.1e-3 rms
    each, and on near-uniform rows the error of P does not average out against the output, which is itself a random
    walk over the values), measured 2.3e-3."""
    from anna_b200 import grouped_query_attention

    gen = torch.Generator(device=cuda_device).manual_seed(404)
    batch, heads, kv_heads, dim, q_len, key_len = 2, 16, 4, 128, 512, 32768
    lengths = torch.tensor([key_len, 9000], device=cuda_device)
    q = torch.randn(batch, heads, q_len, dim, device=cuda_device, generator=gen).to(torch.bfloat16)
    k = torch.randn(batch, kv_heads, key_len, dim, device=cuda_device, generator=gen).to(torch.bfloat16)
    v = torch.randn(batch, kv_heads, key_len, dim, device=cuda_device, generator=gen).to(torch.bfloat16)
    out = grouped_query_attention(q, k, v, scaling=dim ** -0.5, key_lengths=lengths, causal=True).float()
    groups = heads // kv_heads
    for b in range(batch):
        n = int(lengths[b])
        kk = k[b, :, :n].float().repeat_interleave(groups, 0)
        vv = v[b, :, :n].float().repeat_interleave(groups, 0)
        scores = q[b].float() @ kk.transpose(-1, -2) * dim ** -0.5                  # [heads, q_len, n]
        q_pos = n - q_len + torch.arange(q_len, device=cuda_device)
        hidden = torch.arange(n, device=cuda_device)[None, :] > q_pos[:, None]
        scores.masked_fill_(hidden[None], float("-inf"))
        want = torch.softmax(scores, dim=-1) @ vv
        diff = out[b] - want
        max_abs = float(diff.abs().max())
        rel_l2 = float(diff.pow(2).sum().sqrt() / want.pow(2).sum().sqrt())
        assert max_abs <= 2e-2 and rel_l2 <= 4e-3, (b, max_abs, rel_l2)
