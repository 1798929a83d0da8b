"""TurboQuant paged decode against the oracle: packed prefix + window, batched, with and without gate."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from tests.helpers import TQ_ATOL, TqPair, error_stats, outlier_kv, to_np

pytestmark = pytest.mark.gpu


def _decode_and_compare(pair: TqPair, heads: int, seed: int, *, with_gate: bool, tol: float | None = None):
    """Runs one batched decode; checks |got - want| <= tol + tol * |want| (the reference's allclose form,
    tests/test_fused_op_xpu.py:703) and returns (max-abs, relative-L2) of the error."""
    gen = torch.Generator().manual_seed(seed)
    dim = pair.head_dim
    query = torch.randn(pair.batch, heads, 1, dim, generator=gen).to(pair.dtype)
    gate = torch.randn(pair.batch, heads, 1, dim, generator=gen).to(pair.dtype) if with_gate else None
    out = pair.cache.turboquant_single_token_decode_attention(
        0, query.to(pair.device), scaling=dim ** -0.5, num_key_value_groups=heads // pair.kv_heads,
        gate=None if gate is None else gate.to(pair.device))
    expected = np.stack([
        row.decode_attention(to_np(query[b, :, 0]), scaling=dim ** -0.5,
                             gate=None if gate is None else to_np(gate[b, :, 0]))
        for b, row in enumerate(pair.rows)])[:, :, None, :]
    assert out.shape == query.shape and out.dtype == pair.dtype
    if tol is not None:
        np.testing.assert_allclose(to_np(out), expected, atol=tol, rtol=tol)
    return error_stats(to_np(out), expected)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("heads,kv_heads,head_dim", [(8, 2, 64), (8, 2, 128), (16, 2, 256)])
def test_decode_matches_oracle(cuda_device, dtype, bits, heads, kv_heads, head_dim):
    pair = TqPair(device=cuda_device, batch=3, kv_heads=kv_heads, head_dim=head_dim, bits=bits, residual_len=5,
                  block_size=16, dtype=dtype)
    gen = torch.Generator().manual_seed(24 + bits)
    for tokens in (77, 1, 4):
        shape = (3, kv_heads, tokens, head_dim)
        pair.append(outlier_kv(gen, shape, dtype), outlier_kv(gen, shape, dtype))
    _, rel = _decode_and_compare(pair, heads, seed=5, with_gate=True, tol=TQ_ATOL[dtype])
    assert rel <= TQ_ATOL[dtype] / 2, rel


def test_decode_config1_every_step(cuda_device):
    """Config 1 (fp32): prefill 512, then 64 x (append 1, decode); outputs stay within 2e-3 of the oracle."""
    pair = TqPair(device=cuda_device, batch=2, kv_heads=2, head_dim=128, bits=4, residual_len=128, block_size=16,
                  dtype=torch.float32)
    gen = torch.Generator().manual_seed(1)
    shape = (2, 2, 512, 128)
    pair.append(outlier_kv(gen, shape, torch.float32), outlier_kv(gen, shape, torch.float32))
    worst = (0.0, 0.0)
    for step in range(64):
        shape = (2, 2, 1, 128)
        pair.append(outlier_kv(gen, shape, torch.float32), outlier_kv(gen, shape, torch.float32))
        stats = _decode_and_compare(pair, 8, seed=1000 + step, with_gate=False)
        worst = (max(worst[0], stats[0]), max(worst[1], stats[1]))
    assert worst[0] <= 2e-3 and worst[1] <= 2e-3, worst
    pair.assert_bit_exact()


def test_decode_window_only_and_empty_rows(cuda_device):
    """Rows shorter than the window never touch a page; a cache without tokens returns zeros."""
    pair = TqPair(device=cuda_device, batch=2, kv_heads=2, head_dim=128, bits=4, residual_len=16, block_size=16,
                  dtype=torch.bfloat16)
    query = torch.randn(2, 8, 1, 128, device=cuda_device, dtype=torch.bfloat16)
    zeros = pair.cache.turboquant_single_token_decode_attention(0, query, scaling=0.1, num_key_value_groups=4)
    assert torch.count_nonzero(zeros) == 0
    gen = torch.Generator().manual_seed(2)
    shape = (2, 2, 9, 128)
    pair.append(outlier_kv(gen, shape, torch.bfloat16), outlier_kv(gen, shape, torch.bfloat16))
    _, rel = _decode_and_compare(pair, 8, seed=6, with_gate=False, tol=2e-2)
    assert rel <= 2e-2, rel


def test_row_handle_matches_batched_cache(cuda_device):
    """TurboQuantKVRow.append / decode_attention / materialize on a single row (turboquant.py surface)."""
    from anna_b200 import TurboQuantKVRow
    import oracle

    gen = torch.Generator().manual_seed(4)
    row = TurboQuantKVRow(bits=4, residual_len=6)
    orc = oracle.OracleTurboQuantRow(bits=4, residual_len=6, dtype=oracle.DTYPE_BF16)
    for tokens in (9, 1, 20):
        keys = outlier_kv(gen, (2, tokens, 128), torch.bfloat16)
        values = outlier_kv(gen, (2, tokens, 128), torch.bfloat16)
        row.append(keys.to(cuda_device), values.to(cuda_device))
        orc.append(to_np(keys), to_np(values))
    assert (row.length, row.quantized_length, row.residual_length) == (30, 24, 6)
    keys, values = row.materialize()
    want_k, want_v = orc.materialize()
    assert keys.shape == (2, 30, 128)
    np.testing.assert_array_equal(to_np(values), want_v)
    np.testing.assert_allclose(to_np(keys), want_k, atol=4e-2, rtol=2e-2)
    np.testing.assert_array_equal(to_np(keys[:, 24:]), want_k[:, 24:])
    query = torch.randn(8, 1, 128, generator=gen).to(torch.bfloat16)
    out = row.decode_attention(query.to(cuda_device), scaling=128 ** -0.5, num_key_value_groups=4)
    want = orc.decode_attention(to_np(query[:, 0]), scaling=128 ** -0.5)
    np.testing.assert_allclose(to_np(out[:, 0]), want, atol=4e-2, rtol=4e-2)
    clone = row.clone()
    out2 = clone.decode_attention(query.to(cuda_device), scaling=128 ** -0.5, num_key_value_groups=4)
    assert torch.equal(out, out2)
    # copy-on-write: the clone maps the same packed pages until it writes into the partly filled last one
    assert clone.block_table == row.block_table
    keys = outlier_kv(gen, (2, 1, 128), torch.bfloat16)
    clone.append(keys.to(cuda_device), keys.to(cuda_device))
    assert clone.block_table[0] == row.block_table[0] and clone.block_table[1] != row.block_table[1]
    assert torch.equal(row.decode_attention(query.to(cuda_device), scaling=128 ** -0.5, num_key_value_groups=4), out)


def test_tensor_memory_decode_kernel_matches_oracle(cuda_device, tmp_path):
    """The opt-in tcgen05 kernel (ANNA_B200_TQ_UMMA=1, read once per process; head_dim 128, 3- / 4-bit, 4 query heads
    per kv head) against the oracle, in a child process: several 128-token steps, a ragged last step, a hole-free
    table, a gate, and a window-only row beside them; no bounded wait may have expired."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    script = r"""
import sys
import numpy as np, torch
from anna_b200 import _lib
from tests.helpers import TQ_ATOL, TqPair, outlier_kv, to_np
dev = torch.device("cuda:0")
for bits in (3, 4):
    pair = TqPair(device=dev, batch=3, kv_heads=2, head_dim=128, bits=bits, residual_len=16, block_size=16,
                  dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(50 + bits)
    for tokens in (700, 1, 37):
        shape = (3, 2, tokens, 128)
        pair.append(outlier_kv(gen, shape, torch.bfloat16), outlier_kv(gen, shape, torch.bfloat16))
    pair.assert_bit_exact()
    query = torch.randn(3, 8, 1, 128, generator=gen).to(torch.bfloat16)
    gate = torch.randn(3, 8, 1, 128, generator=gen).to(torch.bfloat16)
    out = pair.cache.turboquant_single_token_decode_attention(0, query.to(dev), scaling=128 ** -0.5,
                                                              num_key_value_groups=4, gate=gate.to(dev))
    want = np.stack([row.decode_attention(to_np(query[b, :, 0]), scaling=128 ** -0.5, gate=to_np(gate[b, :, 0]))
                     for b, row in enumerate(pair.rows)])[:, :, None, :]
    np.testing.assert_allclose(to_np(out), want, atol=TQ_ATOL[torch.bfloat16], rtol=TQ_ATOL[torch.bfloat16])
assert _lib.device_faults() == 0
print("ok")
"""
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, ANNA_B200_TQ_UMMA="1", PYTHONPATH=str(root))
    done = subprocess.run([sys.executable, "-c", script], env=env, capture_output=True, text=True, timeout=600,
                          cwd=str(root))
    assert done.returncode == 0 and "ok" in done.stdout, done.stderr[-3000:]
