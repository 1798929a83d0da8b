"""GPU parity of multi-token grouped-query attention (prefill / chunked prefill) against the CPU oracle and the
fixture computed by the reference's own grouped_query_attention (src/anna/model/ops.py:1552-1574)."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from anna_b200 import grouped_query_attention
from anna_b200 import attention as attention_module
from tests.helpers import ATOL, error_stats, to_np

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def _model_masks(lengths: torch.Tensor, q_len: int, key_len: int, causal: bool):
    """The masks Qwen3Attention builds (ops.py:1840-1852, :2008-2016) for a chunk that ends at each row's last key."""
    positions = torch.arange(key_len, device=lengths.device)[None, :]
    visible = positions < lengths[:, None]
    causal_mask = None
    if causal:
        q_positions = (lengths - q_len)[:, None] + torch.arange(q_len, device=lengths.device)[None, :]
        causal_mask = positions[:, None, :] > q_positions[:, :, None]
    return causal_mask, visible


def _oracle(q, k, v, lengths, causal):
    causal_mask, visible = _model_masks(lengths.cpu(), q.shape[2], k.shape[2], causal)
    return oracle.grouped_query_attention(to_np(q), to_np(k), to_np(v), q.shape[3] ** -0.5,
                                          causal_mask=None if causal_mask is None else causal_mask.numpy(),
                                          visible_mask=visible.numpy())


@pytest.mark.parametrize("dtype,heads,kv_heads,dim,q_len,key_len,lengths,causal", [
    (torch.bfloat16, 8, 2, 128, 70, 200, (200, 133), True),      # ragged chunk: 70 queries, not a multiple of 64
    (torch.bfloat16, 32, 8, 128, 256, 1100, (1100, 777), True),  # several key tiles and query tiles
    (torch.float16, 16, 2, 256, 48, 300, (300, 48, 129), True),  # head_dim 256 (32-key tiles), a row that is all chunk
    (torch.float16, 4, 4, 64, 33, 33, (33, 20), True),           # a row shorter than the chunk: queries without keys
    (torch.bfloat16, 6, 2, 128, 5, 90, (90, 64, 7), False),      # key padding only
    (torch.float32, 8, 2, 128, 16, 48, (48, 30), True),          # fp32 cache: row-by-row path through the decode kernel
    # head_dim 128 with 64 or more queries runs on tcgen05 / tensor memory (128-key tiles)
    (torch.float16, 8, 2, 128, 300, 900, (900, 411, 64), False),  # key padding only, a row shorter than one key tile
    (torch.bfloat16, 4, 1, 128, 130, 130, (130, 70), True),       # a row shorter than the chunk: queries without keys
    (torch.bfloat16, 8, 8, 128, 512, 3000, (3000, 1500), True),   # 24 key tiles: the running maximum moves, O is rescaled
    (torch.bfloat16, 16, 1, 128, 64, 64, (64, 1), True),          # 16 heads per KV head: 16 positions per CTA; one key tile
    (torch.float16, 3, 3, 128, 257, 400, (400, 257), True),       # one head per KV head, 256 positions per CTA + 1
    (torch.bfloat16, 6, 2, 128, 100, 333, (333, 0, 129), False),  # three heads per KV head (odd), a row without keys
    (torch.bfloat16, 8, 2, 128, 1024, 1024, (1024,), True),       # full prefill: every CTA ends on its diagonal tile
    # head_dim 256 with 64 or more queries: one 128-row query tile per CTA, 64-key tiles, two score buffers
    (torch.bfloat16, 16, 2, 256, 200, 700, (700, 333, 65), True),  # eight heads per KV head (16 positions per CTA)
    (torch.float16, 4, 4, 256, 130, 130, (130, 70), True),         # one head per KV head, queries without keys
    (torch.bfloat16, 6, 2, 256, 100, 333, (333, 0, 129), False),   # three heads per KV head, key padding only
    (torch.bfloat16, 16, 2, 256, 256, 2100, (2100, 1111), True),   # 33 key tiles
    # head_dim 64 with 64 or more queries: the same kernel template, two query tiles per CTA
    (torch.bfloat16, 8, 2, 64, 200, 700, (700, 333, 65), True),
    (torch.float16, 6, 2, 64, 100, 333, (333, 0, 129), False),
])
def test_prefill_matches_oracle(cuda_device, dtype, heads, kv_heads, dim, q_len, key_len, lengths, causal):
    gen = torch.Generator().manual_seed(heads * 1000 + q_len)
    batch = len(lengths)
    q = torch.randn(batch, heads, q_len, dim, generator=gen).to(dtype).to(cuda_device)
    k = torch.randn(batch, kv_heads, key_len, dim, generator=gen).to(dtype).to(cuda_device)
    v = torch.randn(batch, kv_heads, key_len, dim, generator=gen).to(dtype).to(cuda_device)
    n = torch.tensor(lengths, dtype=torch.long, device=cuda_device)
    causal_mask, visible = _model_masks(n, q_len, key_len, causal)
    out = grouped_query_attention(q, k, v, scaling=dim ** -0.5, causal_mask=causal_mask, visible_mask=visible,
                                  check_masks=True)
    assert out.shape == q.shape and out.dtype == dtype
    expected = _oracle(q, k, v, n, causal)
    max_abs, rel_l2 = error_stats(to_np(out), expected)
    assert max_abs <= ATOL[dtype], (max_abs, rel_l2)
    # the same call with the lengths given directly (no mask is read)
    again = grouped_query_attention(q, k, v, scaling=dim ** -0.5, key_lengths=n, causal=causal)
    assert torch.equal(again, out)


@pytest.mark.parametrize("dim,q_len", [(128, 200), (128, 40), (256, 48), (256, 200), (64, 200)])
def test_keys_behind_a_rows_length_may_hold_anything(cuda_device, dim, q_len):
    """K / V rows past key_lengths[b] are inside the tensors but not part of the row: NaNs there must not reach the
    output (the TMA-fed kernel reads them and zeroes the value rows of the boundary tile; the others never load them)."""
    gen = torch.Generator().manual_seed(dim + q_len)
    heads, kv_heads, key_len = 8, 2, 700
    lengths = (700, 333, q_len)
    batch = len(lengths)
    q = torch.randn(batch, heads, q_len, dim, generator=gen).to(torch.bfloat16).to(cuda_device)
    k = torch.randn(batch, kv_heads, key_len, dim, generator=gen).to(torch.bfloat16).to(cuda_device)
    v = torch.randn(batch, kv_heads, key_len, dim, generator=gen).to(torch.bfloat16).to(cuda_device)
    n = torch.tensor(lengths, dtype=torch.long, device=cuda_device)
    expected = _oracle(q, k, v, n, True)
    for b, length in enumerate(lengths):
        k[b, :, length:] = float("nan")
        v[b, :, length:] = float("nan")
    out = grouped_query_attention(q, k, v, scaling=dim ** -0.5, key_lengths=n, causal=True)
    assert bool(torch.isfinite(out).all())
    max_abs, rel_l2 = error_stats(to_np(out), expected)
    assert max_abs <= ATOL[torch.bfloat16], (max_abs, rel_l2)


@pytest.mark.parametrize("dtype,dim", [(torch.bfloat16, 128), (torch.float16, 128), (torch.bfloat16, 256)])
def test_scores_that_keep_growing_along_the_keys(cuda_device, dtype, dim):
    """Keys whose scale steps up every 80 positions: a row's running maximum moves by far more than the 2^8 the
    tensor-memory kernel tolerates without rescaling, inside key tiles (after part of P was stored) and between them
    (after O was accumulated), so its rescaling of O, of the row sum and of the stored part of P is what is compared."""
    gen = torch.Generator().manual_seed(77)
    batch, heads, kv_heads, q_len, key_len = 2, 8, 2, 192, 1000
    q = torch.randn(batch, heads, q_len, dim, generator=gen)
    k = torch.randn(batch, kv_heads, key_len, dim, generator=gen)
    v = torch.randn(batch, kv_heads, key_len, dim, generator=gen) * 0.25   # nearly one-hot rows: outputs are single values
    steps = (torch.arange(key_len) // 80).float()
    k = k * (1.0 + 3.0 * steps)[None, None, :, None]          # scores up to 38 times larger at the far end
    k[1, :, 500:] *= -1.0                                      # second row: they shrink again for queries that agree
    q, k, v = (t.to(dtype).to(cuda_device) for t in (q, k, v))
    n = torch.tensor((key_len, 901), dtype=torch.long, device=cuda_device)
    for causal in (True, False):
        out = grouped_query_attention(q, k, v, scaling=dim ** -0.5, key_lengths=n, causal=causal)
        expected = _oracle(q, k, v, n, causal)
        assert bool(torch.isfinite(out).all())
        max_abs, rel_l2 = error_stats(to_np(out), expected)
        assert max_abs <= ATOL[dtype], (causal, max_abs, rel_l2)


def test_tensor_memory_kernel_reported_no_expired_wait(cuda_device):
    """Runs after the cases above in this file: none of the bounded waits of the copy-engine / tensor-memory kernels may
    have run out."""
    import ctypes

    from anna_b200 import _lib

    q = torch.randn(1, 4, 128, 128, device=cuda_device, dtype=torch.bfloat16)
    k = torch.randn(1, 1, 256, 128, device=cuda_device, dtype=torch.bfloat16)
    out = grouped_query_attention(q, k, k, scaling=128 ** -0.5, key_lengths=torch.tensor([256], device=cuda_device),
                                  causal=True)
    assert bool(torch.isfinite(out).all())
    count = ctypes.c_int(-1)
    _lib.check(_lib.lib().anna_kv_device_faults(ctypes.byref(count)), "anna_kv_device_faults")
    assert count.value == 0


@pytest.mark.parametrize("case", ["chunk", "full", "padding_only"])
def test_prefill_matches_reference_fixture(cuda_device, case):
    data = np.load(GOLDEN / "prefill_attention.npz")
    q, k, v = (torch.from_numpy(data[f"{case}_{name}"]).to(cuda_device) for name in ("q", "k", "v"))  # fp16, exact
    n = torch.from_numpy(data[f"{case}_lengths"]).to(cuda_device)
    out = grouped_query_attention(q, k, v, scaling=q.shape[3] ** -0.5, key_lengths=n,
                                  causal=bool(data[f"{case}_causal"]))
    ref = data[f"{case}_ref"]
    hidden = ~np.isfinite(ref)
    got = to_np(out)
    assert float(np.abs(got[~hidden] - ref[~hidden]).max()) <= ATOL[torch.float16]
    assert not got[hidden].any()


def test_tensor_core_and_row_paths_agree_on_strided_views(cuda_device):
    """Both kernels on the same operands, K/V being views of a longer cache buffer (token stride > head_dim rows)."""
    gen = torch.Generator().manual_seed(5)
    batch, heads, kv_heads, dim, q_len, key_len = 2, 8, 2, 128, 40, 150
    q = torch.randn(batch, q_len, heads, dim, generator=gen).to(torch.bfloat16).to(cuda_device).transpose(1, 2)
    cache = torch.randn(2, batch, kv_heads, 256, dim, generator=gen).to(torch.bfloat16).to(cuda_device)
    k, v = cache[0, :, :, :key_len], cache[1, :, :, :key_len]
    n = torch.tensor([150, 97], dtype=torch.long, device=cuda_device)
    fast = attention_module._prefill_tensor_core(q, k, v, n, dim ** -0.5, True)
    slow = attention_module._prefill_by_rows(q, k, v, n, dim ** -0.5, True)
    assert float((fast.float() - slow.float()).abs().max()) <= ATOL[torch.bfloat16]


def test_masks_of_another_shape_are_rejected(cuda_device):
    q = torch.zeros(1, 2, 4, 64, dtype=torch.float16, device=cuda_device)
    k = torch.zeros(1, 2, 8, 64, dtype=torch.float16, device=cuda_device)
    holes = torch.tensor([[True, False, True, True, True, True, True, True]], device=cuda_device)
    with pytest.raises(ValueError, match="suffix"):
        grouped_query_attention(q, k, k, scaling=1.0, visible_mask=holes, check_masks=True)
    band = torch.zeros(1, 4, 8, dtype=torch.bool, device=cuda_device)
    with pytest.raises(ValueError, match="causal"):
        grouped_query_attention(q, k, k, scaling=1.0, causal_mask=band, check_masks=True)
    with pytest.raises(RuntimeError, match="CUDA"):
        grouped_query_attention(q.cpu(), k.cpu(), k.cpu(), scaling=1.0)


def test_chunked_prefill_over_turboquant_cache_matches_oracle(cuda_device):
    """The reference's prefill flow on a quantized cache (ops.py:2008-2025): update(require_dense_cache=True) hands back
    the de-quantized prefix + window + chunk as dense K/V, the chunk's queries attend to it causally.  Rows of different
    lengths, two chunks each; the expectation is the oracle row's materialize() followed by the oracle attention."""
    from tests.helpers import DTYPE_CODE, TQ_ATOL, TqPair

    dtype, heads, kv_heads, dim, bits, residual = torch.bfloat16, 8, 2, 128, 4, 16
    pair = TqPair(device=cuda_device, batch=2, kv_heads=kv_heads, head_dim=dim, bits=bits, residual_len=residual,
                  block_size=16, dtype=dtype)
    gen = torch.Generator().manual_seed(9)
    assert DTYPE_CODE[dtype] == oracle.DTYPE_BF16
    for chunk in (70, 45):
        k = torch.randn(2, kv_heads, chunk, dim, generator=gen).to(dtype)
        v = torch.randn(2, kv_heads, chunk, dim, generator=gen).to(dtype)
        q = torch.randn(2, heads, chunk, dim, generator=gen).to(dtype)
        keys, values, past = pair.cache.update(k.to(cuda_device), v.to(cuda_device), 0, require_dense_cache=True)
        for b, row in enumerate(pair.rows):
            row.append(to_np(k[b]), to_np(v[b]))
        visible = past + chunk
        out = grouped_query_attention(q.to(cuda_device), keys, values, scaling=dim ** -0.5, key_lengths=visible,
                                      causal=True)
        for b, row in enumerate(pair.rows):
            dense_k, dense_v = row.materialize()
            n = dense_k.shape[1]
            assert n == int(visible[b])
            positions = np.arange(n)[None, None, :]
            causal_mask = positions > (n - chunk + np.arange(chunk))[None, :, None]
            expected = oracle.grouped_query_attention(to_np(q[b:b + 1]), dense_k[None], dense_v[None], dim ** -0.5,
                                                      causal_mask=causal_mask)
            max_abs, _ = error_stats(to_np(out[b:b + 1]), expected)
            assert max_abs <= TQ_ATOL[dtype], (chunk, b, max_abs)
