"""GPU parity of the un-quantized decode ops against the CPU oracle.

Shapes follow the reference's kernel tests (tests/test_fused_op_xpu.py:490-944): dense decode with ragged visible
lengths, split-KV with strided K/V and fused gate, caller-owned workspace, paged decode with a block table.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from anna_b200 import fused_ops
from tests.helpers import ATOL, error_stats, reference_decode, to_np

pytestmark = pytest.mark.gpu


def _pack_paged_kv(key, value, *, block_size, permute_seed=None):
    batch, heads, key_len, dim = key.shape
    per_row = (key_len + block_size - 1) // block_size
    total = batch * per_row
    order = torch.arange(total)
    if permute_seed is not None:
        order = torch.randperm(total, generator=torch.Generator().manual_seed(permute_seed))
    key_pages = key.new_zeros((total, heads, block_size, dim))
    value_pages = value.new_zeros((total, heads, block_size, dim))
    table = torch.full((batch, per_row), -1, dtype=torch.int32, device=key.device)
    for b in range(batch):
        for blk in range(per_row):
            pid = int(order[b * per_row + blk])
            start = blk * block_size
            take = min(block_size, key_len - start)
            key_pages[pid, :, :take] = key[b, :, start:start + take]
            value_pages[pid, :, :take] = value[b, :, start:start + take]
            table[b, blk] = pid
    return key_pages, value_pages, table


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("heads,kv_heads,dim,key_len", [(8, 2, 64, 19), (16, 4, 256, 777), (8, 8, 128, 130),
                                                        (16, 2, 128, 300)])
def test_gqa_decode_fused_matches_oracle(cuda_device, dtype, heads, kv_heads, dim, key_len):
    torch.manual_seed(0)
    query = torch.randn(2, heads, 1, dim, device=cuda_device, dtype=dtype)
    key = torch.randn(2, kv_heads, key_len, dim, device=cuda_device, dtype=dtype)
    value = torch.randn(2, kv_heads, key_len, dim, device=cuda_device, dtype=dtype)
    visible = torch.tensor([key_len, max(1, key_len * 2 // 3)], device=cuda_device, dtype=torch.long)
    out = fused_ops.run_gqa_decode_fused(query=query, key=key, value=value, visible_lengths=visible,
                                         scaling=dim ** -0.5)
    expected = reference_decode(query, key, value, visible.tolist(), dim ** -0.5)
    assert out.shape == query.shape and out.dtype == dtype
    np.testing.assert_allclose(to_np(out), expected, atol=ATOL[dtype], rtol=ATOL[dtype])


def test_gqa_decode_fused_gate_layouts_agree(cuda_device):
    torch.manual_seed(11)
    batch, heads, dim = 2, 8, 64
    query = torch.randn(batch, heads, 1, dim, device=cuda_device, dtype=torch.bfloat16)
    key = torch.randn(batch, 2, 23, dim, device=cuda_device, dtype=torch.bfloat16)
    value = torch.randn_like(key)
    visible = torch.tensor([23, 17], device=cuda_device, dtype=torch.long)
    gate_3d = torch.randn(batch, 1, heads * dim, device=cuda_device, dtype=torch.bfloat16)
    gate_4d = gate_3d.view(batch, 1, heads, dim).transpose(1, 2)
    out_3d = fused_ops.run_gqa_decode_fused(query=query, key=key, value=value, visible_lengths=visible,
                                            scaling=dim ** -0.5, gate=gate_3d)
    out_4d = fused_ops.run_gqa_decode_fused(query=query, key=key, value=value, visible_lengths=visible,
                                            scaling=dim ** -0.5, gate=gate_4d)
    expected = reference_decode(query, key, value, visible.tolist(), dim ** -0.5, gate=gate_4d)
    assert torch.equal(out_3d, out_4d)
    np.testing.assert_allclose(to_np(out_4d), expected, atol=3e-2, rtol=3e-2)


def test_splitkv_accepts_strided_kv_and_fuses_gate(cuda_device):
    torch.manual_seed(20)
    heads, kv_heads, dim, key_len, capacity = 8, 2, 64, 257, 512
    query = torch.randn(1, heads, 1, dim, device=cuda_device, dtype=torch.bfloat16)
    key_storage = torch.empty(1, kv_heads, capacity, dim, device=cuda_device, dtype=torch.bfloat16)
    value_storage = torch.empty_like(key_storage)
    key_storage[:, :, :key_len].normal_()
    value_storage[:, :, :key_len].normal_()
    key, value = key_storage[:, :, :key_len], value_storage[:, :, :key_len]
    gate = torch.randn(1, 1, heads * dim, device=cuda_device, dtype=torch.bfloat16).view(1, 1, heads, dim).transpose(1, 2)
    assert not key.is_contiguous()
    out = fused_ops.run_gqa_decode_splitkv_fused(query=query, key=key, value=value, scaling=dim ** -0.5,
                                                 block_size=64, gate=gate)
    expected = reference_decode(query, key, value, [key_len], dim ** -0.5, gate=gate)
    np.testing.assert_allclose(to_np(out), expected, atol=3e-2, rtol=3e-2)


def test_splitkv_out_reuses_workspace_and_accepts_strided_query(cuda_device):
    torch.manual_seed(22)
    heads, kv_heads, dim, key_len, block = 8, 2, 64, 193, 64
    blocks = (key_len + block - 1) // block
    query = torch.randn(1, heads, 1, dim * 2, device=cuda_device, dtype=torch.bfloat16)[..., ::2]
    key = torch.randn(1, kv_heads, 256, dim, device=cuda_device, dtype=torch.bfloat16)[:, :, :key_len]
    value = torch.randn(1, kv_heads, 256, dim, device=cuda_device, dtype=torch.bfloat16)[:, :, :key_len]
    output = torch.empty_like(query)
    stats = torch.empty(1, heads, blocks + 2, 2, device=cuda_device, dtype=torch.float32)
    values = torch.empty(1, heads, blocks + 2, dim, device=cuda_device, dtype=torch.float32)
    assert not query.is_contiguous()
    returned = fused_ops.run_gqa_decode_splitkv_fused_out(query=query, key=key, value=value, output=output,
                                                          partial_stats=stats, partial_values=values,
                                                          scaling=dim ** -0.5, block_size=block)
    expected = reference_decode(query, key, value, [key_len], dim ** -0.5)
    assert returned.untyped_storage().data_ptr() == output.untyped_storage().data_ptr()
    np.testing.assert_allclose(to_np(output), expected, atol=3e-2, rtol=3e-2)


def test_splitkv_out_rejects_small_workspace(cuda_device):
    query = torch.randn(1, 8, 1, 64, device=cuda_device, dtype=torch.bfloat16)
    key = torch.randn(1, 2, 200, 64, device=cuda_device, dtype=torch.bfloat16)
    stats = torch.empty(1, 8, 2, 2, device=cuda_device, dtype=torch.float32)
    values = torch.empty(1, 8, 2, 64, device=cuda_device, dtype=torch.float32)
    with pytest.raises(RuntimeError, match="capacity"):
        fused_ops.run_gqa_decode_splitkv_fused_out(query=query, key=key, value=key.clone(),
                                                   output=torch.empty_like(query), partial_stats=stats,
                                                   partial_values=values, scaling=0.125, block_size=64)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("heads,kv_heads,dim,key_len,block", [(16, 4, 256, 4096, 32), (32, 8, 128, 1000, 16),
                                                             (8, 2, 64, 45, 16)])
def test_paged_decode_matches_oracle(cuda_device, dtype, heads, kv_heads, dim, key_len, block):
    torch.manual_seed(0)
    batch = 3
    query = torch.randn(batch, heads, 1, dim, device=cuda_device, dtype=dtype)
    key = torch.randn(batch, kv_heads, key_len, dim, device=cuda_device, dtype=dtype)
    value = torch.randn(batch, kv_heads, key_len, dim, device=cuda_device, dtype=dtype)
    key_pages, value_pages, table = _pack_paged_kv(key, value, block_size=block, permute_seed=5)
    visible = torch.tensor([key_len, key_len // 2 + 1, 1], device=cuda_device, dtype=torch.long)
    gate = torch.randn(batch, heads, 1, dim, device=cuda_device, dtype=dtype)
    out = fused_ops.run_paged_gqa_decode_fused(query=query, key_pages=key_pages, value_pages=value_pages,
                                               page_table=table, visible_lengths=visible, scaling=dim ** -0.5,
                                               gate=gate)
    expected = reference_decode(query, key, value, visible.tolist(), dim ** -0.5, gate=gate)
    max_abs, rel = error_stats(to_np(out), expected)
    assert max_abs <= ATOL[dtype] * 2 and rel <= ATOL[dtype], (max_abs, rel)


@pytest.mark.parametrize("heads,kv_heads,dim", [(32, 2, 128), (8, 4, 64), (4, 1, 256)])
def test_paged_decode_split_schedules_agree(cuda_device, heads, kv_heads, dim):
    """The three split schedules of the C entry point (even share of tiles per CTA with the in-kernel merge, fixed
    chunks with the in-kernel merge, fixed chunks with the separate merge launch) against the oracle, on ragged rows
    that include empty ones, groups wider than one 8-head tile and the smallest legal scratch."""
    from anna_b200 import _lib
    from anna_b200.fused_ops import dtype_code, on_device, ptr, stream_ptr

    torch.manual_seed(11)
    block, key_len = 16, 1500
    lengths = [key_len, 0, 1, 17, 640, 0, 1499, 256, 33]
    batch = len(lengths)
    query = torch.randn(batch, heads, 1, dim, device=cuda_device, dtype=torch.bfloat16)
    key = torch.randn(batch, kv_heads, key_len, dim, device=cuda_device, dtype=torch.bfloat16)
    value = torch.randn_like(key)
    key_pages, value_pages, table = _pack_paged_kv(key, value, block_size=block, permute_seed=2)
    visible = torch.tensor(lengths, device=cuda_device, dtype=torch.long)
    expected = reference_decode(query, key, value, lengths, dim ** -0.5)
    max_blocks = int(table.shape[1])
    _, plan_chunks = _lib.decode_plan(batch, kv_heads, max_blocks * block)
    fixed = 64
    fixed_chunks = (max_blocks * block + fixed - 1) // fixed
    group_tiles = (heads // kv_heads + 7) // 8

    def run(chunk_tokens, capacity, fused):
        stats = torch.empty(batch, heads, capacity, 2, device=cuda_device, dtype=torch.float32)
        values = torch.empty(batch, heads, capacity, dim, device=cuda_device, dtype=torch.float32)
        counters = torch.zeros(2 * batch * kv_heads * group_tiles, device=cuda_device, dtype=torch.int32)
        out = torch.full_like(query, float("nan"))
        for _ in range(2):  # the second call checks that the counters came back to zero
            with on_device(cuda_device):
                _lib.check(_lib.lib().anna_paged_gqa_decode(
                    ptr(query), query.stride(0), query.stride(1), ptr(key_pages), ptr(value_pages), ptr(table),
                    table.stride(0), ptr(visible), None, 0, 0, ptr(out), out.stride(0), out.stride(1), ptr(stats),
                    ptr(values), capacity, chunk_tokens, ptr(counters) if fused else None, batch, heads, kv_heads, dim,
                    block, int(key_pages.shape[0]), max_blocks, dim ** -0.5, dtype_code(query.dtype),
                    stream_ptr(cuda_device)), "anna_paged_gqa_decode")
        assert torch.count_nonzero(counters) == 0
        return to_np(out)

    results = {
        "even share": run(0, plan_chunks, True),
        "fixed chunks, merged in kernel": run(fixed, fixed_chunks, True),
        "fixed chunks, merge launch": run(fixed, fixed_chunks, False),
    }
    for label, got in results.items():
        assert np.isfinite(got).all(), label
        max_abs, rel = error_stats(got, expected)
        assert max_abs <= ATOL[torch.bfloat16] * 2 and rel <= ATOL[torch.bfloat16], (label, max_abs, rel)
        for row, length in enumerate(lengths):
            if length == 0:
                assert not got[row].any(), (label, row)


def test_paged_decode_even_share_respects_scratch_capacity(cuda_device):
    """Many short rows and one long one: an even share of tiles would cut the long row into more partials than the
    planned scratch (two slots per head here) holds, so the share must grow instead."""
    from anna_b200 import _lib
    from anna_b200.fused_ops import dtype_code, on_device, ptr, stream_ptr

    torch.manual_seed(12)
    batch, heads, kv_heads, dim, block, max_blocks = 512, 16, 8, 64, 16, 128
    chunk, capacity = _lib.decode_plan(batch, kv_heads, max_blocks * block)
    assert capacity == 2
    pages = max_blocks + batch
    key_pages = torch.randn(pages, kv_heads, block, dim, device=cuda_device, dtype=torch.bfloat16)
    value_pages = torch.randn_like(key_pages)
    table = torch.full((batch, max_blocks), -1, dtype=torch.int32, device=cuda_device)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(4)).to(torch.int32).to(cuda_device)
    long_row = 200
    table[long_row] = order[:max_blocks]
    others = [b for b in range(batch) if b != long_row]
    table[others, 0] = order[max_blocks:max_blocks + len(others)]
    lengths = torch.full((batch,), 16, dtype=torch.long)
    lengths[long_row] = max_blocks * block - 3
    lengths[7] = 0
    visible = lengths.to(cuda_device)
    query = torch.randn(batch, heads, 1, dim, device=cuda_device, dtype=torch.bfloat16)

    def run(chunk_tokens, slots, fused):
        stats = torch.empty(batch, heads, slots, 2, device=cuda_device, dtype=torch.float32)
        values = torch.empty(batch, heads, slots, dim, device=cuda_device, dtype=torch.float32)
        counters = torch.zeros(2 * batch * kv_heads, device=cuda_device, dtype=torch.int32)
        out = torch.full_like(query, float("nan"))
        with on_device(cuda_device):
            _lib.check(_lib.lib().anna_paged_gqa_decode(
                ptr(query), query.stride(0), query.stride(1), ptr(key_pages), ptr(value_pages), ptr(table),
                table.stride(0), ptr(visible), None, 0, 0, ptr(out), out.stride(0), out.stride(1), ptr(stats),
                ptr(values), slots, chunk_tokens, ptr(counters) if fused else None, batch, heads, kv_heads, dim, block,
                pages, max_blocks, dim ** -0.5, dtype_code(query.dtype), stream_ptr(cuda_device)),
                "anna_paged_gqa_decode")
        assert torch.count_nonzero(counters) == 0
        return to_np(out)

    even = run(0, capacity, True)
    fixed = run(256, max_blocks * block // 256, False)
    assert np.isfinite(even).all()
    np.testing.assert_allclose(even, fixed, atol=2e-2, rtol=2e-2)
    assert not even[7].any()


def test_paged_decode_skips_holes_and_zero_rows(cuda_device):
    """Entries < 0 are skipped and a row without visible keys gives zeros (.sycl:5310-5313, :5342)."""
    torch.manual_seed(3)
    heads, kv_heads, dim, block = 8, 2, 64, 16
    key = torch.randn(2, kv_heads, 64, dim, device=cuda_device, dtype=torch.bfloat16)
    value = torch.randn_like(key)
    query = torch.randn(2, heads, 1, dim, device=cuda_device, dtype=torch.bfloat16)
    key_pages, value_pages, table = _pack_paged_kv(key, value, block_size=block)
    table[0, 1] = -1
    visible = torch.tensor([64, 0], device=cuda_device, dtype=torch.long)
    out = fused_ops.run_paged_gqa_decode_fused(query=query, key_pages=key_pages, value_pages=value_pages,
                                               page_table=table, visible_lengths=visible, scaling=dim ** -0.5)
    keep = [t for t in range(64) if not (16 <= t < 32)]
    expected = reference_decode(query[:1], key[:1, :, keep], value[:1, :, keep], [len(keep)], dim ** -0.5)
    np.testing.assert_allclose(to_np(out[:1]), expected, atol=2e-2, rtol=2e-2)
    assert torch.count_nonzero(out[1]) == 0


def test_ops_reject_cpu_tensors_and_bad_shapes(cuda_device):
    query = torch.randn(1, 8, 1, 64)
    key = torch.randn(1, 2, 5, 64)
    with pytest.raises((RuntimeError, NotImplementedError)):
        fused_ops.run_gqa_decode_fused(query=query, key=key, value=key, visible_lengths=torch.tensor([5]), scaling=1.0)
    q = torch.randn(1, 6, 1, 64, device=cuda_device, dtype=torch.bfloat16)
    k = torch.randn(1, 4, 5, 64, device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="divisible"):
        fused_ops.run_gqa_decode_fused(query=q, key=k, value=k, visible_lengths=torch.tensor([5], device=cuda_device),
                                       scaling=1.0)


@pytest.mark.parametrize("value_bits", [2, 3, 4])
def test_splitkv_turboquant_out_matches_reference_case(cuda_device, value_bits):
    """The reference's own kernel test (tests/test_fused_op_xpu.py:647-703): Hq=8, Hkv=2, D=64, Lq=77, R=5, group 16,
    strided query, oversized workspace, fused gate; inputs and expected output come from the reference run on CPU."""
    from pathlib import Path

    data = np.load(Path(__file__).resolve().parent / "golden" / "splitkv_turboquant_case.npz")
    p = f"b{value_bits}_"
    bf = lambda name: torch.from_numpy(data[p + name]).to(cuda_device).to(torch.bfloat16)  # noqa: E731
    storage = torch.zeros(1, 8, 1, 128, device=cuda_device, dtype=torch.bfloat16)
    storage[..., ::2] = bf("query")
    query = storage[..., ::2]
    assert not query.is_contiguous()
    vdata = torch.from_numpy(data[p + "vdata"]).to(cuda_device).unsqueeze(0)
    output = torch.empty_like(query)
    blocks = (82 + 63) // 64
    stats = torch.empty(1, 8, blocks + 1, 2, device=cuda_device, dtype=torch.float32)
    values = torch.empty(1, 8, blocks + 1, 64, device=cuda_device, dtype=torch.float32)
    returned = fused_ops.run_gqa_decode_splitkv_turboquant_fused_out(
        query=query, quantized_key=bf("qkey"), value_data=vdata, value_scales=bf("vscales").unsqueeze(0),
        value_zeros=bf("vzeros").unsqueeze(0), residual_key=bf("rkey"), residual_value=bf("rvalue"), output=output,
        partial_stats=stats, partial_values=values, scaling=64 ** -0.5, value_bits=value_bits, value_group_size=16,
        block_size=64, gate=bf("gate"))
    assert returned.untyped_storage().data_ptr() == output.untyped_storage().data_ptr()
    np.testing.assert_allclose(to_np(output), data[p + "ref"], atol=4e-2, rtol=4e-2)
    assert fused_ops.gqa_decode_splitkv_turboquant_fused_out_is_available()
    via_torch_ops = torch.ops.anna.gqa_decode_splitkv_turboquant_fused_out(
        query, bf("qkey"), vdata, bf("vscales").unsqueeze(0), bf("vzeros").unsqueeze(0), bf("rkey"), bf("rvalue"),
        torch.empty_like(query), stats, values, 64 ** -0.5, value_bits, 16, 64, bf("gate"))
    assert torch.equal(via_torch_ops, output)
