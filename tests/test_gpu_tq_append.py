"""Bit-exact parity of the fused TurboQuant append (codes, metadata, block tables, window ring) with the oracle."""
from __future__ import annotations

import pytest
import torch

from tests.helpers import TqPair, outlier_kv

pytestmark = pytest.mark.gpu


def _run_schedule(pair: TqPair, schedule, seed: int) -> None:
    gen = torch.Generator().manual_seed(seed)
    for tokens in schedule:
        shape = (pair.batch, pair.kv_heads, tokens, pair.head_dim)
        keys = outlier_kv(gen, shape, pair.dtype)
        values = outlier_kv(gen, shape, pair.dtype)
        pair.append(keys, values)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("head_dim", [64, 128, 256])
def test_append_is_bit_exact_small_window(cuda_device, dtype, bits, head_dim):
    pair = TqPair(device=cuda_device, batch=2, kv_heads=2, head_dim=head_dim, bits=bits, residual_len=8,
                  block_size=16, dtype=dtype)
    # prefill below the window, cross it, single-token steps, a chunk larger than the window, more single steps
    _run_schedule(pair, [5, 1, 1, 1, 7, 1, 30, 1, 1, 1], seed=100 + bits)
    pair.assert_bit_exact()


def test_append_config1_prefill_and_decode_steps(cuda_device):
    """Benchmark configuration 1: fp32, 8q/2kv heads, D=128, S=16, 4-bit, R=128; prefill 512 then 64 single-token appends."""
    pair = TqPair(device=cuda_device, batch=2, kv_heads=2, head_dim=128, bits=4, residual_len=128, block_size=16,
                  dtype=torch.float32)
    _run_schedule(pair, [512] + [1] * 64, seed=1)
    pair.assert_bit_exact()
    assert pair.cache.turboquant_rows[0][0].quantized_length == 512 + 64 - 128


def test_append_edge_lengths_around_window_and_block(cuda_device):
    """L in {R-1, R, R+1} and quantized lengths in {S-1, S, S+1} (window 4, block 4)."""
    pair = TqPair(device=cuda_device, batch=1, kv_heads=2, head_dim=64, bits=4, residual_len=4, block_size=4,
                  dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(9)
    for _ in range(14):
        shape = (1, 2, 1, 64)
        pair.append(outlier_kv(gen, shape, torch.bfloat16), outlier_kv(gen, shape, torch.bfloat16))
        pair.assert_bit_exact()


def test_append_constant_and_zero_vectors(cuda_device):
    """Zero keys (norm 0) and constant values (max == min -> scale clamps to 1e-8) must not produce NaN codes."""
    pair = TqPair(device=cuda_device, batch=1, kv_heads=2, head_dim=128, bits=4, residual_len=2, block_size=16,
                  dtype=torch.bfloat16)
    keys = torch.zeros(1, 2, 6, 128, dtype=torch.bfloat16)
    values = torch.full((1, 2, 6, 128), 0.75, dtype=torch.bfloat16)
    keys[:, :, 1] = 1.0
    pair.append(keys, values)
    pair.assert_bit_exact()
