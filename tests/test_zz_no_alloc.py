"""GPU: the allocation-free paged decode entry point against the regular one, through the C ABI.

anna_paged_gqa_decode_noalloc serves hosts that may not allocate device memory (for example a plugin that lives
inside another engine's memory pool): it keeps its split-K scratch in a fixed array inside the library.  The array is
shared by all calls and keeps the previous call's contents, so the check runs twice in a row on different inputs.
"""
from __future__ import annotations

import ctypes

import numpy as np
import pytest
import torch

import oracle
from anna_b200 import _lib
from tests.helpers import to_np

pytestmark = pytest.mark.gpu


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _decode_both(device, seed, batch, heads, kv_heads, dim, block, max_blocks, dtype):
    gen = torch.Generator(device=device).manual_seed(seed)
    pages = batch * max_blocks
    key_pages = torch.randn(pages, kv_heads, block, dim, device=device, dtype=dtype, generator=gen)
    value_pages = torch.randn(pages, kv_heads, block, dim, device=device, dtype=dtype, generator=gen)
    query = torch.randn(batch, heads, 1, dim, device=device, dtype=dtype, generator=gen)
    gate = torch.randn(batch, heads, 1, dim, device=device, dtype=dtype, generator=gen)
    table = torch.randperm(pages, device=device, generator=gen).to(torch.int32).reshape(batch, max_blocks)
    table[0, 1] = -1  # a hole is skipped by both paths
    lengths = torch.randint(1, max_blocks * block + 1, (batch,), device=device, generator=gen)
    lengths[-1] = 0   # an empty row gives zeros
    lib = _lib.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    code = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}[dtype]

    chunk, chunks = _lib.decode_plan(batch, kv_heads, max_blocks * block)
    stats = torch.empty(batch, heads, chunks, 2, device=device, dtype=torch.float32)
    values = torch.empty(batch, heads, chunks, dim, device=device, dtype=torch.float32)
    counters = torch.zeros(2 * batch * kv_heads * ((heads // kv_heads + 7) // 8), device=device, dtype=torch.int32)
    want = torch.empty_like(query)
    _lib.check(lib.anna_paged_gqa_decode(
        _ptr(query), query.stride(0), query.stride(1), _ptr(key_pages), _ptr(value_pages), _ptr(table),
        table.stride(0), _ptr(lengths), _ptr(gate), gate.stride(0), gate.stride(1), _ptr(want), want.stride(0),
        want.stride(1), _ptr(stats), _ptr(values), chunks, 0, _ptr(counters), batch, heads, kv_heads, dim, block, pages,
        max_blocks, dim ** -0.5, code, stream), "anna_paged_gqa_decode")

    got = torch.empty_like(query)
    torch.cuda.synchronize(device)
    free_before = torch.cuda.mem_get_info(device)[0]
    _lib.check(lib.anna_paged_gqa_decode_noalloc(
        _ptr(query), query.stride(0), query.stride(1), _ptr(key_pages), _ptr(value_pages), _ptr(table),
        table.stride(0), _ptr(lengths), _ptr(gate), gate.stride(0), gate.stride(1), _ptr(got), got.stride(0),
        got.stride(1), batch, heads, kv_heads, dim, block, pages, max_blocks, dim ** -0.5, code, stream),
        "anna_paged_gqa_decode_noalloc")
    torch.cuda.synchronize(device)
    grew = free_before - torch.cuda.mem_get_info(device)[0]
    # the same rows through the CPU oracle: gather each row's pages (holes dropped), dense fp32 attention
    ref = np.zeros((batch, heads, 1, dim), dtype=np.float32)
    table_host, lengths_host = table.cpu().tolist(), lengths.cpu().tolist()
    kp, vp = to_np(key_pages), to_np(value_pages)
    for b in range(batch):
        n = int(lengths_host[b])
        if n == 0:
            continue
        keys, vals = [], []
        for blk in range((n + block - 1) // block):
            pid, take = table_host[b][blk], min(block, n - blk * block)
            if pid >= 0:
                keys.append(kp[pid][:, :take])
                vals.append(vp[pid][:, :take])
        if not keys:
            continue
        ref[b, :, 0] = oracle.gqa_decode(to_np(query[b, :, 0]), np.concatenate(keys, axis=1),
                                         np.concatenate(vals, axis=1), dim ** -0.5, to_np(gate[b, :, 0]))
    return got, want, grew, torch.from_numpy(ref)


def test_noalloc_decode_matches_regular_entry_point_twice(cuda_device):
    # same tolerance as the paged decode parity tests (tests/test_gpu_paged_decode.py)
    first = _decode_both(cuda_device, 1, batch=5, heads=32, kv_heads=8, dim=128, block=16, max_blocks=40,
                         dtype=torch.bfloat16)
    torch.testing.assert_close(first[0].float(), first[1].float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(first[0].float().cpu(), first[3], atol=2e-2, rtol=2e-2)  # and against the CPU oracle
    assert torch.count_nonzero(first[0][-1]) == 0
    # The first call on a device may load the library's device image (which contains the 16 MiB array); later calls
    # must not take any device memory at all.
    second = _decode_both(cuda_device, 2, batch=3, heads=8, kv_heads=2, dim=64, block=32, max_blocks=9,
                          dtype=torch.float32)
    torch.testing.assert_close(second[0], second[1], atol=2e-4, rtol=2e-4)
    torch.testing.assert_close(second[0].cpu(), second[3], atol=2e-4, rtol=2e-4)
    assert second[2] <= 0
    third = _decode_both(cuda_device, 3, batch=5, heads=32, kv_heads=8, dim=128, block=16, max_blocks=40,
                         dtype=torch.bfloat16)
    torch.testing.assert_close(third[0].float(), third[1].float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(third[0].float().cpu(), third[3], atol=2e-2, rtol=2e-2)
    assert third[2] <= 0


def test_noalloc_decode_rejects_problems_beyond_its_scratch(cuda_device):
    lib = _lib.lib()
    assert lib.anna_noalloc_scratch_bytes() == 16 << 20
    dummy = torch.zeros(16, device=cuda_device)
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda_device).cuda_stream)
    status = lib.anna_paged_gqa_decode_noalloc(
        _ptr(dummy), 0, 0, _ptr(dummy), _ptr(dummy), _ptr(dummy), 0, _ptr(dummy), None, 0, 0, _ptr(dummy), 0, 0,
        512, 64, 8, 256, 16, 1 << 20, 4096, 0.1, 2, stream)
    assert status == 4  # ANNA_ERR_WORKSPACE
    assert "built-in" in _lib.last_error() and "split-K scratch" in _lib.last_error()
    # a short context whose partials would fit, but with more (row, head-group) pairs than the counter region holds
    status = lib.anna_paged_gqa_decode_noalloc(
        _ptr(dummy), 0, 0, _ptr(dummy), _ptr(dummy), _ptr(dummy), 0, _ptr(dummy), None, 0, 0, _ptr(dummy), 0, 0,
        8200, 1, 1, 64, 16, 1 << 20, 1, 0.1, 2, stream)
    assert status == 4
    assert "merge counters" in _lib.last_error() and "8192" in _lib.last_error()


def test_bounded_copy_wait_gives_up_and_context_survives(cuda_device):
    """A wait on a barrier nothing completes must expire (not hang), and the GPU keeps working afterwards."""
    import ctypes

    from anna_b200 import _lib

    expired = ctypes.c_int(-1)
    with torch.cuda.device(cuda_device):
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib.lib().anna_kv_selftest_wait_expiry(ctypes.byref(expired), stream or None),
                   "anna_kv_selftest_wait_expiry")
    assert expired.value == 1
    probe = torch.arange(8, device=cuda_device).sum()
    assert int(probe) == 28 and _lib.device_faults() == 0
