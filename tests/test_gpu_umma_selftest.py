"""GPU: the tensor-memory matrix multiply primitives (tcgen05) against plain fp32 matrix products.

anna_kv_selftest_umma re-tiles row-major operands into the shared-memory layouts of the packed decode kernel and runs
both of its products: e4m3 x e4m3 with K-major operands (scores) and f16 x f16 with MN-major operands (values)."""
from __future__ import annotations

import ctypes

import pytest
import torch

from anna_b200 import _lib

pytestmark = pytest.mark.gpu


def test_umma_products_match_fp32_reference(cuda_device):
    gen = torch.Generator(device=cuda_device).manual_seed(11)
    # e4m3 operands: every value is exactly representable, so the fp32 reference is exact up to summation order
    a1 = (torch.randn(128, 128, device=cuda_device, generator=gen) * 2).to(torch.float8_e4m3fn)
    b1 = (torch.randn(16, 128, device=cuda_device, generator=gen) * 2).to(torch.float8_e4m3fn)
    a2 = torch.randn(128, 128, device=cuda_device, generator=gen).to(torch.float16)   # [K][rows]
    # the decode kernel feeds value codes as f16 subnormals (code * 2^-24, code * 2^-20): they must not be flushed
    codes = torch.randint(0, 16, (128, 64), device=cuda_device, generator=gen).to(torch.float32)
    a2[:, 0::4] = (codes[:, :32] * 2.0 ** -24).to(torch.float16)
    a2[:, 1::4] = (codes[:, 32:] * 2.0 ** -20).to(torch.float16)
    b2 = torch.randn(128, 16, device=cuda_device, generator=gen).to(torch.float16)    # [K][columns]
    d1 = torch.zeros(128, 16, device=cuda_device, dtype=torch.float32)
    d2 = torch.zeros(128, 16, device=cuda_device, dtype=torch.float32)
    status = ctypes.c_int(-1)
    with torch.cuda.device(cuda_device):
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        _lib.check(_lib.lib().anna_kv_selftest_umma(
            ctypes.c_void_p(a1.data_ptr()), ctypes.c_void_p(b1.data_ptr()), ctypes.c_void_p(a2.data_ptr()),
            ctypes.c_void_p(b2.data_ptr()), ctypes.c_void_p(d1.data_ptr()), ctypes.c_void_p(d2.data_ptr()),
            ctypes.byref(status), stream), "anna_kv_selftest_umma")
    assert status.value == 0
    want1 = a1.float() @ b1.float().t()
    want2 = a2.float().t() @ b2.float()
    torch.testing.assert_close(d1, want1, atol=1e-3, rtol=1e-4)
    torch.testing.assert_close(d2, want2, atol=1e-3, rtol=1e-4)
    # rows fed with subnormals only come out exactly (products of f16 values are exact, sums are small integers * 2^-k)
    sub_rows = a2.float().t()[0::4] @ b2.float()
    torch.testing.assert_close(d2[0::4], sub_rows, atol=0.0, rtol=2e-3)
    assert float(d2[0::4].abs().max()) > 0.0


def test_tma_fed_products_match_fp32_reference(cuda_device):
    """anna_kv_selftest_umma_tma: bf16 operands brought in by tiled TMA loads with the 128-byte swizzle and read through
    swizzled descriptors, K-major (the Q . K^T arrangement of the prefill kernel) and MN-major (its P . V one)."""
    gen = torch.Generator(device=cuda_device).manual_seed(12)
    a = torch.randn(128, 128, device=cuda_device, generator=gen).to(torch.bfloat16)
    b1 = torch.randn(128, 128, device=cuda_device, generator=gen).to(torch.bfloat16)
    b2 = torch.randn(128, 128, device=cuda_device, generator=gen).to(torch.bfloat16)
    d1 = torch.zeros(128, 128, device=cuda_device, dtype=torch.float32)
    d2 = torch.zeros(128, 128, device=cuda_device, dtype=torch.float32)
    status = ctypes.c_int(-1)
    with torch.cuda.device(cuda_device):
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        _lib.check(_lib.lib().anna_kv_selftest_umma_tma(
            ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b1.data_ptr()), ctypes.c_void_p(b2.data_ptr()),
            ctypes.c_void_p(d1.data_ptr()), ctypes.c_void_p(d2.data_ptr()), ctypes.byref(status), stream),
            "anna_kv_selftest_umma_tma")
    assert status.value == 0
    torch.testing.assert_close(d1, a.float() @ b1.float().t(), atol=1e-3, rtol=1e-4)
    torch.testing.assert_close(d2, a.float() @ b2.float(), atol=1e-3, rtol=1e-4)


def test_tensor_memory_operand_product_matches_fp32_reference(cuda_device):
    """anna_kv_selftest_umma_ts: the A operand packed into tensor memory by the threads (two bf16 values per column), B by
    TMA and MN-major -- the P . V arrangement of the prefill kernel."""
    gen = torch.Generator(device=cuda_device).manual_seed(13)
    a = torch.randn(128, 128, device=cuda_device, generator=gen).to(torch.bfloat16)
    b = torch.randn(128, 128, device=cuda_device, generator=gen).to(torch.bfloat16)
    d = torch.zeros(128, 128, device=cuda_device, dtype=torch.float32)
    status = ctypes.c_int(-1)
    with torch.cuda.device(cuda_device):
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        _lib.check(_lib.lib().anna_kv_selftest_umma_ts(
            ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()), ctypes.c_void_p(d.data_ptr()),
            ctypes.byref(status), stream), "anna_kv_selftest_umma_ts")
    assert status.value == 0
    torch.testing.assert_close(d, a.float() @ b.float(), atol=1e-3, rtol=1e-4)
