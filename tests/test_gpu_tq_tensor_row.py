"""GPU parity of the MSE-only tensor row (Gemma4's K / V history rows) against the CPU oracle.

Follows the reference's own checks of this row type (tests/test_gemma4_text_runtime.py:318-340: append in pieces, residual
tokens exact, reconstruction error bounded) and adds bit-exact index / norm parity with the oracle quantizer.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from anna_b200 import TurboQuantTensorRow
from tests.helpers import to_np

pytestmark = pytest.mark.gpu


def _unpack(codes: np.ndarray, dim: int, bits: int) -> np.ndarray:
    field = 2 if bits == 2 else 4
    per_byte = 8 // field
    out = np.zeros(codes.shape[:-1] + (dim,), dtype=np.uint8)
    for k in range(per_byte):
        out[..., k::per_byte] = (codes >> (field * k)) & ((1 << field) - 1)
    return out


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("dim,bits", [(64, 2), (128, 4), (256, 3), (512, 4), (512, 2)])
def test_tensor_row_matches_oracle(cuda_device, dtype, dim, bits):
    torch.manual_seed(dim + bits)
    heads, residual_len = 3, 8
    row = TurboQuantTensorRow(bits=bits, residual_len=residual_len)
    pieces = [torch.randn(heads, n, dim, device=cuda_device, dtype=dtype) * (1.0 + 0.1 * i)
              for i, n in enumerate((5, 1, 30, 1, 1, 19))]
    for piece in pieces:
        row.append(piece)
    full = torch.cat(pieces, dim=1)
    total = int(full.shape[1])
    assert row.length == total and row.quantized_length == total - residual_len

    # indices and norms: bit-exact against the oracle on the same (exactly widened) inputs
    lq = row.quantized_length
    idx, _, norms, _ = oracle.quantize_keys(to_np(full[:, :lq]), bits, "mse")
    got_idx = _unpack(row._codes[:, :lq].cpu().numpy(), dim, bits)
    assert np.array_equal(got_idx, idx)
    assert np.array_equal(row._norms[:, :lq].cpu().numpy(), norms)

    # materialize: de-quantized prefix (oracle arithmetic, rounded to the cache dtype) followed by the exact window
    dense = row.materialize()
    assert dense.shape == full.shape and dense.dtype == dtype
    assert torch.equal(dense[:, lq:], full[:, lq:])
    want = oracle.dequantize_keys(idx, None, norms, None, bits, "mse")
    want = torch.from_numpy(want).to(dtype).float().numpy()
    assert np.array_equal(to_np(dense[:, :lq]), want)
    mse = float(((dense[:, :lq].float() - full[:, :lq].float()) ** 2).mean())
    assert mse < 0.5  # the reference's own bound for this row type

    # clone is independent, fp32 materialisation on request
    twin = row.clone()
    row.append(torch.randn(heads, 4, dim, device=cuda_device, dtype=dtype))
    assert twin.length == total and row.length == total + 4
    assert torch.equal(twin.materialize(dtype=torch.float32), dense.float())


def test_tensor_row_rejects_bad_input(cuda_device):
    row = TurboQuantTensorRow(bits=4, residual_len=4)
    with pytest.raises(ValueError):
        row.append(torch.zeros(2, 128, device=cuda_device))
    with pytest.raises(RuntimeError):
        row.materialize()
    row.append(torch.zeros(2, 3, 128, device=cuda_device, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        row.append(torch.zeros(2, 3, 64, device=cuda_device, dtype=torch.bfloat16))
    with pytest.raises(RuntimeError):
        TurboQuantTensorRow(bits=4, residual_len=4).append(torch.zeros(2, 3, 128))
