"""Shared helpers of the parity tests: dtype plumbing between torch tensors and the numpy oracle."""
from __future__ import annotations

import numpy as np
import torch

import oracle

DTYPE_CODE = {torch.float32: oracle.DTYPE_F32, torch.float16: oracle.DTYPE_F16, torch.bfloat16: oracle.DTYPE_BF16}
# Attention-output tolerances per cache dtype, the same as the reference's kernel tests
# (tests/test_fused_op_xpu.py:513 dense/paged 2e-2, :561 split-KV 3e-2, :703 TurboQuant 4e-2).
ATOL = {torch.float32: 2e-4, torch.float16: 2e-2, torch.bfloat16: 2e-2}
TQ_ATOL = {torch.float32: 2e-3, torch.float16: 4e-2, torch.bfloat16: 4e-2}


def to_np(tensor: torch.Tensor) -> np.ndarray:
    return tensor.detach().float().cpu().numpy()


def outlier_kv(gen: torch.Generator, shape, dtype, *, outliers: int = 4, scale: float = 8.0) -> torch.Tensor:
    """N(0,1) with `outliers` random channels per head scaled up (shape [..., H, T, D])."""
    x = torch.randn(shape, generator=gen, dtype=torch.float32)
    heads, dim = shape[-3], shape[-1]
    for h in range(heads):
        idx = torch.randperm(dim, generator=gen)[:outliers]
        x[..., h, :, idx] *= scale
    return x.to(dtype)


def error_stats(actual: np.ndarray, expected: np.ndarray) -> tuple[float, float]:
    max_abs = float(np.abs(actual - expected).max()) if actual.size else 0.0
    denom = float(np.linalg.norm(expected.ravel())) or 1.0
    return max_abs, float(np.linalg.norm((actual - expected).ravel())) / denom


def reference_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, lengths, scaling: float, gate=None):
    """Oracle GQA decode for q [B, Hq, 1, D], k/v [B, Hkv, L, D] with per-row visible lengths -> [B, Hq, 1, D] fp32."""
    batch = q.shape[0]
    out = np.zeros((batch, q.shape[1], 1, q.shape[3]), dtype=np.float32)
    for b in range(batch):
        n = int(lengths[b])
        g = None if gate is None else to_np(gate[b]).reshape(q.shape[1], q.shape[3])
        out[b, :, 0] = oracle.gqa_decode(to_np(q[b, :, 0]), to_np(k[b, :, :n]), to_np(v[b, :, :n]), scaling, g)
    return out


# ---------------------------------------------------------------------------------------------------------------
# TurboQuant state: GPU cache next to oracle rows


def oracle_layout(pool) -> "oracle.PackedPageLayout":
    return oracle.PackedPageLayout(head_dim=pool.head_dim, bits=pool.bits, block_size=pool.block_size,
                                   dtype_bytes=4 if pool.dtype == torch.float32 else 2, group=pool.value_group)


def packed_row_fields(pool, row, first_token: int = 0, last_token: int | None = None) -> dict[str, np.ndarray]:
    """Per-token fields of quantized tokens [first_token, last_token) of one GPU row, read back from its packed pages
    and laid out like the oracle's arrays: kcodes / vdata uint8 [Hkv, n, bytes], norms / rnorms float32 [Hkv, n],
    vscales / vzeros float32 [Hkv, n, groups] (cache-dtype values widened to float32)."""
    layout = oracle_layout(pool)
    lq = row.quantized_length
    last_token = lq if last_token is None else min(int(last_token), lq)
    first_token = max(0, int(first_token))
    heads, s = pool.kv_heads, pool.block_size
    count = max(0, last_token - first_token)
    out = {
        "kcodes": np.zeros((heads, count, layout.key_bytes), np.uint8),
        "norms": np.zeros((heads, count), np.float32), "rnorms": np.zeros((heads, count), np.float32),
        "vdata": np.zeros((heads, count, layout.value_bytes), np.uint8),
        "vscales": np.zeros((heads, count, layout.groups), np.float32),
        "vzeros": np.zeros((heads, count, layout.groups), np.float32),
    }
    if count == 0:
        return out
    blk0, blk1 = first_token // s, (last_token + s - 1) // s
    ids = torch.tensor(row.block_table[blk0:blk1], device=pool.packed_pages.device)
    pages = pool.packed_pages[ids].cpu().numpy()  # [blocks, heads, chunk_bytes]
    blocks = pages.shape[0]
    lo, hi = first_token - blk0 * s, last_token - blk0 * s

    def tokens(offset: int, width: int) -> np.ndarray:
        """[heads, blocks * S, width] bytes of one per-token sub-array, cut to the asked token range."""
        sub = pages[:, :, offset:offset + s * width].reshape(blocks, heads, s, width)
        return np.ascontiguousarray(sub.transpose(1, 0, 2, 3).reshape(heads, blocks * s, width)[:, lo:hi])

    out["kcodes"] = tokens(layout.off_kcodes, layout.key_bytes)
    out["norms"] = tokens(layout.off_knorm, 4).view(np.float32)[..., 0]
    out["rnorms"] = tokens(layout.off_krnorm, 4).view(np.float32)[..., 0]
    out["vdata"] = tokens(layout.off_vdata, layout.value_bytes)
    for name, base in (("vscales", layout.off_vscale), ("vzeros", layout.off_vzero)):
        raw = tokens(base, layout.groups * layout.dtype_bytes)
        if pool.dtype == torch.float32:
            out[name] = raw.view(np.float32)
        elif pool.dtype == torch.float16:
            out[name] = raw.view(np.float16).astype(np.float32)
        else:  # bfloat16
            out[name] = (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32)
    return out


class TqPair:
    """A GPU Qwen3DynamicCache (one TurboQuant layer) driven in lock-step with per-row oracle rows."""

    def __init__(self, *, device, batch, kv_heads, head_dim, bits, residual_len, block_size, dtype):
        from anna_b200 import KVCacheConfig, Qwen3DynamicCache

        self.device, self.dtype = device, dtype
        self.batch, self.kv_heads, self.head_dim = batch, kv_heads, head_dim
        config = KVCacheConfig(num_hidden_layers=1, cache_block_size=block_size)
        self.cache = Qwen3DynamicCache(config, batch_size=batch, kv_cache_quantization="turboquant",
                                       kv_cache_quant_bits=bits, kv_cache_residual_len=residual_len)
        self.oracle_allocator = oracle.OracleLayerAllocator()
        self.rows = [oracle.OracleTurboQuantRow(bits=bits, residual_len=residual_len, dtype=DTYPE_CODE[dtype],
                                                block_size=block_size, allocator=self.oracle_allocator)
                     for _ in range(batch)]

    @property
    def pool(self):
        return self.cache.allocator.turboquant_layers[0]

    def append(self, keys: torch.Tensor, values: torch.Tensor) -> None:
        """keys/values [B, Hkv, T, D] in the cache dtype (CPU tensors)."""
        self.cache.update(keys.to(self.device), values.to(self.device), 0, require_dense_cache=False)
        for b, row in enumerate(self.rows):
            row.append(to_np(keys[b]), to_np(values[b]))

    def gpu_fields(self, b: int) -> dict[str, np.ndarray]:
        """Per-token fields of row b read back from the packed pages, in the oracle's array shapes."""
        return packed_row_fields(self.pool, self.cache.turboquant_rows[0][b])

    def assert_bit_exact(self) -> None:
        for b, orc in enumerate(self.rows):
            row = self.cache.turboquant_rows[0][b]
            assert row.length == orc.length
            assert row.quantized_length == orc.quantized_length
            assert row.residual_length == orc.residual_length
            assert row.block_table == orc.block_table, (row.block_table, orc.block_table)
            got = self.gpu_fields(b)
            if orc.quantized_length:
                want_codes = oracle.pack_key_codes(orc.idx, orc.sign, orc.bits)
                np.testing.assert_array_equal(got["kcodes"], want_codes)
                np.testing.assert_array_equal(got["norms"].view(np.uint32), orc.norms.view(np.uint32))
                np.testing.assert_array_equal(got["rnorms"].view(np.uint32), orc.rnorms.view(np.uint32))
                np.testing.assert_array_equal(got["vdata"], orc.vdata)
                np.testing.assert_array_equal(got["vscales"].view(np.uint32), orc.vscales.view(np.uint32))
                np.testing.assert_array_equal(got["vzeros"].view(np.uint32), orc.vzeros.view(np.uint32))
            # window ring: position p sits in slot p % R
            pool = self.pool
            lq, length = orc.quantized_length, orc.length
            if length > lq:
                ring = (torch.arange(lq, length) % pool.residual_len).to(pool.window.device)
                win_k = to_np(pool.window[row.slot, 0].index_select(1, ring))
                win_v = to_np(pool.window[row.slot, 1].index_select(1, ring))
                np.testing.assert_array_equal(win_k, orc.residual_keys)
                np.testing.assert_array_equal(win_v, orc.residual_values)
        assert int(self.pool.status.item()) == 0
