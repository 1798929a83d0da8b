"""The ``anna::`` operator namespace: the reference's five decode schemas (gated_delta_fused_op.sycl:7621-7679) plus the
ops for the steps that are Python in the reference, each with a CUDA kernel, a Meta (shape-only) kernel and an autograd
fall-through (the reference's registration, .sycl:7916-7983).  The Meta kernels run here without a GPU; the CUDA
kernels are called through the dispatcher in the gpu-marked tests below."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import anna_b200
import oracle
from anna_b200 import _lib, fused_ops


@pytest.fixture(scope="module", autouse=True)
def registered():
    assert anna_b200.maybe_load_gated_delta_library()


def _meta(*shape, dtype=torch.bfloat16):
    return torch.empty(*shape, device="meta", dtype=dtype)


def test_every_schema_is_registered_with_the_reference_signature():
    for name, schema in {**fused_ops.SCHEMAS, **fused_ops.NEW_SCHEMAS}.items():
        op = getattr(torch.ops.anna, name)
        text = str(op.default._schema)
        assert text.startswith(f"anna::{name}(") and text.endswith(schema.split("->")[1].strip())
    # argument names and order of the five reference schemas
    args = [a.name for a in torch.ops.anna.gqa_decode_splitkv_turboquant_fused_out.default._schema.arguments]
    assert args == ["query", "quantized_key", "value_data", "value_scales", "value_zeros", "residual_key",
                    "residual_value", "output", "partial_stats", "partial_values", "scaling", "value_bits",
                    "value_group_size", "block_size", "gate"]
    args = [a.name for a in torch.ops.anna.paged_gqa_decode_fused.default._schema.arguments]
    assert args == ["query", "key_pages", "value_pages", "page_table", "visible_lengths", "scaling", "gate"]


def test_meta_kernels_give_shapes_and_alias_the_output_argument():
    q = _meta(2, 8, 1, 128)
    k = _meta(2, 2, 64, 128)
    lengths = _meta(2, dtype=torch.long)
    assert torch.ops.anna.gqa_decode_fused(q, k, k, lengths, 0.1).shape == q.shape
    assert torch.ops.anna.gqa_decode_splitkv_fused(q, k, k, 0.1, 16).shape == q.shape
    out, stats, values = _meta(2, 8, 1, 128), _meta(2, 8, 4, 2, dtype=torch.float32), _meta(2, 8, 4, 128, dtype=torch.float32)
    assert torch.ops.anna.gqa_decode_splitkv_fused_out(q, k, k, out, stats, values, 0.1, 16) is out
    vdata, vmeta = _meta(2, 2, 64, 64, dtype=torch.uint8), _meta(2, 2, 64, 4)
    resid = _meta(2, 2, 5, 128)
    assert torch.ops.anna.gqa_decode_splitkv_turboquant_fused_out(q, k, vdata, vmeta, vmeta, resid, resid, out, stats,
                                                                  values, 0.1, 4, 32, 16) is out
    pages, table = _meta(8, 2, 16, 128), _meta(2, 4, dtype=torch.int32)
    assert torch.ops.anna.paged_gqa_decode_fused(q, pages, pages, table, lengths, 0.1).shape == q.shape
    assert torch.ops.anna.paged_kv_write(k, k, pages, pages, table, lengths) is None
    packed, window = _meta(8, 2, 2432, dtype=torch.uint8), _meta(2, 2, 2, 128, 128)
    assert torch.ops.anna.tq_append(k, k, packed, table, window, lengths, lengths, 4, 128, 16, 32) is None
    assert torch.ops.anna.tq_paged_decode(q, packed, table, window, lengths, lengths, 0.1, 4, 128, 16, 32).shape == q.shape


@pytest.mark.gpu
def test_new_ops_through_the_dispatcher_match_the_oracle(cuda_device):
    """A TurboQuant history written and decoded only with torch.ops.anna.tq_append / tq_paged_decode on raw tensors,
    and an un-quantized one with paged_kv_write / paged_gqa_decode_fused, against the oracle."""
    from tests.helpers import outlier_kv, to_np

    gen = torch.Generator().manual_seed(77)
    batch, heads, kv_heads, dim, bits, window_len, page = 2, 8, 2, 128, 4, 8, 16
    layout = _lib.tq_page_layout(dim, bits, page, 2, 32)
    packed = torch.zeros(16, kv_heads, layout["chunk_bytes"], dtype=torch.uint8, device=cuda_device)
    window = torch.zeros(batch, 2, kv_heads, window_len, dim, dtype=torch.bfloat16, device=cuda_device)
    table = torch.tensor([[3, 1, 7, -1], [0, 9, 4, -1]], dtype=torch.int32, device=cuda_device)
    slots = torch.tensor([1, 0], dtype=torch.long, device=cuda_device)
    rows = [oracle.OracleTurboQuantRow(bits=bits, residual_len=window_len, dtype=oracle.DTYPE_BF16) for _ in range(batch)]
    lengths = torch.zeros(batch, dtype=torch.long, device=cuda_device)
    for tokens in (41, 1, 3):
        k, v = outlier_kv(gen, (batch, kv_heads, tokens, dim), torch.bfloat16), \
            outlier_kv(gen, (batch, kv_heads, tokens, dim), torch.bfloat16)
        torch.ops.anna.tq_append(k.to(cuda_device), v.to(cuda_device), packed, table, window, slots, lengths, bits,
                                 window_len, page, 32)
        lengths = lengths + tokens
        for b, row in enumerate(rows):
            row.append(to_np(k[b]), to_np(v[b]))
    query = torch.randn(batch, heads, 1, dim, generator=gen).to(torch.bfloat16)
    out = torch.ops.anna.tq_paged_decode(query.to(cuda_device), packed, table, window, slots, lengths, dim ** -0.5, bits,
                                         window_len, page, 32)
    want = np.stack([row.decode_attention(to_np(query[b, :, 0]), scaling=dim ** -0.5) for b, row in enumerate(rows)])
    np.testing.assert_allclose(to_np(out[:, :, 0]), want, atol=4e-2, rtol=4e-2)

    key_pages = torch.zeros(8, kv_heads, page, dim, dtype=torch.bfloat16, device=cuda_device)
    value_pages = torch.zeros_like(key_pages)
    table2 = torch.tensor([[5, 2], [6, 1]], dtype=torch.int32, device=cuda_device)
    past = torch.zeros(batch, dtype=torch.long, device=cuda_device)
    k = torch.randn(batch, kv_heads, 21, dim, generator=gen).to(torch.bfloat16)
    v = torch.randn(batch, kv_heads, 21, dim, generator=gen).to(torch.bfloat16)
    torch.ops.anna.paged_kv_write(k.to(cuda_device), v.to(cuda_device), key_pages, value_pages, table2, past)
    visible = past + 21
    out = torch.ops.anna.paged_gqa_decode_fused(query.to(cuda_device), key_pages, value_pages, table2, visible,
                                                dim ** -0.5)
    for b in range(batch):
        want = oracle.gqa_decode(to_np(query[b, :, 0]), to_np(k[b]), to_np(v[b]), dim ** -0.5)
        np.testing.assert_allclose(to_np(out[b, :, 0]), want, atol=2e-2, rtol=2e-2)


@pytest.mark.gpu
def test_reference_schemas_through_the_dispatcher(cuda_device):
    """gqa_decode_fused, gqa_decode_splitkv_fused and gqa_decode_splitkv_fused_out called as torch.ops.anna.* (the
    way Anna's wrappers call them, src/anna/model/fused_ops.py:451-609) against the oracle."""
    from tests.helpers import to_np

    gen = torch.Generator().manual_seed(78)
    batch, heads, kv_heads, dim, length = 2, 8, 2, 128, 75
    q = torch.randn(batch, heads, 1, dim, generator=gen).to(torch.bfloat16)
    k = torch.randn(batch, kv_heads, length, dim, generator=gen).to(torch.bfloat16)
    v = torch.randn(batch, kv_heads, length, dim, generator=gen).to(torch.bfloat16)
    visible = torch.tensor([length, 40], dtype=torch.long)
    qd, kd, vd = q.to(cuda_device), k.to(cuda_device), v.to(cuda_device)
    got = torch.ops.anna.gqa_decode_fused(qd, kd, vd, visible.to(cuda_device), dim ** -0.5)
    for b in range(batch):
        n = int(visible[b])
        want = oracle.gqa_decode(to_np(q[b, :, 0]), to_np(k[b, :, :n]), to_np(v[b, :, :n]), dim ** -0.5)
        np.testing.assert_allclose(to_np(got[b, :, 0]), want, atol=2e-2, rtol=2e-2)
    full = [oracle.gqa_decode(to_np(q[b, :, 0]), to_np(k[b]), to_np(v[b]), dim ** -0.5) for b in range(batch)]
    got = torch.ops.anna.gqa_decode_splitkv_fused(qd, kd, vd, dim ** -0.5, 32)
    np.testing.assert_allclose(to_np(got[:, :, 0]), np.stack(full), atol=3e-2, rtol=3e-2)
    blocks = (length + 31) // 32
    out = torch.empty_like(qd)
    stats = torch.empty(batch, heads, blocks, 2, device=cuda_device, dtype=torch.float32)
    values = torch.empty(batch, heads, blocks, dim, device=cuda_device, dtype=torch.float32)
    ret = torch.ops.anna.gqa_decode_splitkv_fused_out(qd, kd, vd, out, stats, values, dim ** -0.5, 32)
    assert ret.data_ptr() == out.data_ptr()
    np.testing.assert_allclose(to_np(out[:, :, 0]), np.stack(full), atol=3e-2, rtol=3e-2)
