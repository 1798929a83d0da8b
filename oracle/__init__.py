"""CPU oracle for the TurboQuant paged-KV path (numpy + a small C library).

TEST INFRASTRUCTURE ONLY.  Nothing under ``anna_b200/`` imports this package.  It is used by ``tests/``,
by ``__graft_entry__.smoke()`` and by ``bench.py`` (``cpu_baseline`` and ``--impl reference``) as the
checker and as the timed CPU baseline, never as a compute path of the product.

Parity status: the value quantizer, the window/flush bookkeeping, the page allocator policy and the decode
math restate code that lives in the reference tree and are pinned against outputs of the reference itself
(fixtures under ``tests/golden`` made by ``tests/golden/make_golden.py``).  The key quantizer restates the
published TurboQuant algorithm because the reference delegates it to the un-vendored ``turboquant`` package
(>=0.2,<0.3): key-code parity against that package is UNPINNED.

Arrays are numpy float32 holding values that are exactly representable in the cache dtype; the dtype itself
travels as a code (0 = float32, 1 = float16, 2 = bfloat16).
"""
from __future__ import annotations

import ctypes
import json
import math
import os
import struct
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libtq_oracle.so"
_LIB: ctypes.CDLL | None = None

DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2
QUANTIZER_SEED = 42  # turboquant.py:80, :90


def build(force: bool = False) -> Path:
    """Compile oracle/tq_oracle.c with the Makefile next to it."""
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < (_HERE / "tq_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE)], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        build()
        handle = ctypes.CDLL(str(_LIB_PATH))
        f32p = ctypes.POINTER(ctypes.c_float)
        u8p = ctypes.POINTER(ctypes.c_uint8)
        handle.tqo_signs.argtypes = [ctypes.c_int, ctypes.c_uint64, ctypes.c_int, f32p]
        handle.tqo_signs.restype = None
        handle.tqo_fwht.argtypes = [f32p, ctypes.c_int]
        handle.tqo_fwht.restype = None
        handle.tqo_quantize_keys.argtypes = [f32p, ctypes.c_int64, ctypes.c_int, ctypes.c_int, f32p, f32p, f32p, f32p,
                                             u8p, u8p, f32p, f32p]
        handle.tqo_dequantize_keys.argtypes = [u8p, u8p, f32p, f32p, ctypes.c_int64, ctypes.c_int, f32p, f32p, f32p,
                                               f32p]
        handle.tqo_rotate_queries.argtypes = [f32p, ctypes.c_int64, ctypes.c_int, f32p, f32p, f32p, f32p]
        handle.tqo_quantize_values.argtypes = [f32p, ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                               ctypes.c_int, u8p, f32p, f32p]
        handle.tqo_dequantize_values.argtypes = [u8p, f32p, f32p, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                                                 ctypes.c_int, f32p]
        handle.tqo_gqa_decode.argtypes = [f32p, f32p, f32p, f32p, ctypes.c_int, ctypes.c_int, ctypes.c_int64,
                                          ctypes.c_int, ctypes.c_float, f32p]
        handle.tqo_f32_to_bf16.argtypes = [ctypes.c_float]
        handle.tqo_f32_to_bf16.restype = ctypes.c_uint16
        handle.tqo_f32_to_f16.argtypes = [ctypes.c_float]
        handle.tqo_f32_to_f16.restype = ctypes.c_uint16
        _LIB = handle
    return _LIB


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _for_row_ranges(count: int, call) -> int:
    """Run ``call(first, rows) -> status`` over [0, count).  Vectors are independent, so large inputs are cut into one
    range per host core and run on threads (ctypes drops the GIL during the C call); the results do not depend on the
    cut.  Returns the first non-zero status."""
    workers = min(os.cpu_count() or 1, count // 2048)
    if workers <= 1:
        return call(0, count)
    from concurrent.futures import ThreadPoolExecutor

    step = (count + workers - 1) // workers
    ranges = [(first, min(step, count - first)) for first in range(0, count, step)]
    with ThreadPoolExecutor(max_workers=workers) as pool:
        for status in pool.map(lambda r: call(*r), ranges):
            if status != 0:
                return status
    return 0


def _p(a: np.ndarray, ctype):
    return a.ctypes.data_as(ctypes.POINTER(ctype))


# --------------------------------------------------------------------------------------------------
# dtype rounding (exact, vectorised)


def round_bf16(a) -> np.ndarray:
    a = _f32(a)
    bits = a.view(np.uint32)
    # round to nearest even on the 16 dropped bits; finite inputs cannot wrap (the largest finite float rounds to inf)
    rounded = (bits + (np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1)))) & np.uint32(0xFFFF0000)
    out = rounded.view(np.float32)
    nan = np.isnan(a)
    return np.where(nan, a, out) if nan.any() else out


def round_dtype(a, dtype: int) -> np.ndarray:
    if dtype == DTYPE_BF16:
        return round_bf16(a)
    if dtype == DTYPE_F16:
        return _f32(a).astype(np.float16).astype(np.float32)
    return _f32(a)


def dtype_size(dtype: int) -> int:
    return 4 if dtype == DTYPE_F32 else 2


# --------------------------------------------------------------------------------------------------
# key quantizer

_CODEBOOKS: dict[str, dict[str, list[str]]] | None = None


def codebook(dim: int, index_bits: int) -> tuple[np.ndarray, np.ndarray]:
    """Frozen Lloyd-Max centroids / boundaries (float32) for the scaled rotated coordinate."""
    global _CODEBOOKS
    if _CODEBOOKS is None:
        _CODEBOOKS = json.loads((_HERE / "tq_codebooks.json").read_text())["tables"]
    entry = _CODEBOOKS[f"d{dim}_m{index_bits}"]

    def dec(items: list[str]) -> np.ndarray:
        return np.array([struct.unpack(">f", bytes.fromhex(h))[0] for h in items], dtype=np.float32)

    return dec(entry["centroids"]), dec(entry["boundaries"])


def signs(dim: int, stream: int, seed: int = QUANTIZER_SEED) -> np.ndarray:
    out = np.empty(dim, dtype=np.float32)
    lib().tqo_signs(dim, seed, stream, _p(out, ctypes.c_float))
    return out


def fwht(v) -> np.ndarray:
    v = _f32(v).copy()
    flat = v.reshape(-1, v.shape[-1])
    for row in flat:
        lib().tqo_fwht(_p(row, ctypes.c_float), row.shape[0])
    return flat.reshape(v.shape)


def key_index_bits(bits: int, variant: str = "ip") -> int:
    """TurboQuantIP(bits=b) spends b-1 bits on the Lloyd-Max index and one on the QJL sign."""
    return bits - 1 if variant == "ip" else bits


def quantize_keys(x, bits: int, variant: str = "ip"):
    """x [..., D] -> (idx uint8 [..., D], sign uint8 [..., D] | None, norms [...], rnorms [...] | None)."""
    x = _f32(x)
    dim = x.shape[-1]
    flat = x.reshape(-1, dim)
    n = flat.shape[0]
    m = key_index_bits(bits, variant)
    cent, bnd = codebook(dim, m)
    s1, s2 = signs(dim, 0), signs(dim, 1)
    idx = np.zeros((n, dim), dtype=np.uint8)
    norms = np.zeros(n, dtype=np.float32)
    if variant == "ip":
        sign = np.zeros((n, dim), dtype=np.uint8)
        rnorms = np.zeros(n, dtype=np.float32)
    else:
        sign = rnorms = None
    fn = lib().tqo_quantize_keys

    def call(first: int, rows: int) -> int:
        sp = _p(sign[first:], ctypes.c_uint8) if sign is not None else ctypes.POINTER(ctypes.c_uint8)()
        rp = _p(rnorms[first:], ctypes.c_float) if rnorms is not None else ctypes.POINTER(ctypes.c_float)()
        return fn(_p(flat[first:], ctypes.c_float), rows, dim, m, _p(s1, ctypes.c_float), _p(s2, ctypes.c_float),
                  _p(cent, ctypes.c_float), _p(bnd, ctypes.c_float), _p(idx[first:], ctypes.c_uint8), sp,
                  _p(norms[first:], ctypes.c_float), rp)

    rc = _for_row_ranges(n, call)
    if rc != 0:
        raise ValueError(f"tqo_quantize_keys failed with status {rc} (dim={dim}, bits={bits})")
    lead = x.shape[:-1]
    return (idx.reshape(*lead, dim), None if sign is None else sign.reshape(*lead, dim), norms.reshape(lead),
            None if rnorms is None else rnorms.reshape(lead))


def dequantize_keys(idx, sign, norms, rnorms, bits: int, variant: str = "ip") -> np.ndarray:
    idx = np.ascontiguousarray(idx, dtype=np.uint8)
    dim = idx.shape[-1]
    flat = idx.reshape(-1, dim)
    n = flat.shape[0]
    m = key_index_bits(bits, variant)
    cent, _ = codebook(dim, m)
    s1, s2 = signs(dim, 0), signs(dim, 1)
    norms = _f32(norms).reshape(-1)
    out = np.zeros((n, dim), dtype=np.float32)
    with_sign = sign is not None and rnorms is not None
    if with_sign:
        sign = np.ascontiguousarray(sign, dtype=np.uint8).reshape(-1, dim)
        rnorms = _f32(rnorms).reshape(-1)
    fn = lib().tqo_dequantize_keys

    def call(first: int, rows: int) -> int:
        sp = _p(sign[first:], ctypes.c_uint8) if with_sign else ctypes.POINTER(ctypes.c_uint8)()
        rp = _p(rnorms[first:], ctypes.c_float) if with_sign else ctypes.POINTER(ctypes.c_float)()
        return fn(_p(flat[first:], ctypes.c_uint8), sp, _p(norms[first:], ctypes.c_float), rp, rows, dim,
                  _p(s1, ctypes.c_float), _p(s2, ctypes.c_float), _p(cent, ctypes.c_float),
                  _p(out[first:], ctypes.c_float))

    rc = _for_row_ranges(n, call)
    if rc != 0:
        raise ValueError(f"tqo_dequantize_keys failed with status {rc}")
    return out.reshape(idx.shape)


def qjl_matrix(dim: int) -> np.ndarray:
    """Dense S with S @ r == fwht(s2 * fwht(s1 * r)) / sqrt(D): the `quantizer.S` of turboquant.py:324."""
    s1, s2 = signs(dim, 0), signs(dim, 1)
    eye = np.eye(dim, dtype=np.float32)
    first = fwht(eye * s1[None, :])  # rows: fwht(s1 * e_j)  -> columns of H diag(s1)
    second = fwht(first * s2[None, :])
    return (second.T / np.float32(math.sqrt(dim))).astype(np.float32)


# --------------------------------------------------------------------------------------------------
# value quantizer (turboquant.py:157-252)


def resolve_value_group_size(head_dim: int) -> int:
    for candidate in (32, 16, 8, 4, 2, 1):
        if candidate <= head_dim and head_dim % candidate == 0:
            return candidate
    return 1


def quantize_values(x, bits: int, group: int, dtype: int):
    """x [..., D] float32 (exact in `dtype`) -> (data uint8 [..., D/per_byte], scales [..., D/group], zeros)."""
    x = _f32(x)
    dim = x.shape[-1]
    flat = x.reshape(-1, dim)
    n = flat.shape[0]
    per_byte = 4 if bits == 2 else 2
    data = np.zeros((n, dim // per_byte), dtype=np.uint8)
    scales = np.zeros((n, dim // group), dtype=np.float32)
    zeros = np.zeros((n, dim // group), dtype=np.float32)
    rc = lib().tqo_quantize_values(_p(flat, ctypes.c_float), n, dim, group, bits, dtype, _p(data, ctypes.c_uint8),
                                   _p(scales, ctypes.c_float), _p(zeros, ctypes.c_float))
    if rc != 0:
        raise ValueError(f"tqo_quantize_values failed with status {rc}")
    lead = x.shape[:-1]
    return data.reshape(*lead, -1), scales.reshape(*lead, -1), zeros.reshape(*lead, -1)


def dequantize_values(data, scales, zeros, bits: int, group: int) -> np.ndarray:
    data = np.ascontiguousarray(data, dtype=np.uint8)
    scales, zeros = _f32(scales), _f32(zeros)
    dim = scales.shape[-1] * group
    n = int(np.prod(scales.shape[:-1], dtype=np.int64))
    out = np.zeros((n, dim), dtype=np.float32)
    rc = lib().tqo_dequantize_values(_p(data, ctypes.c_uint8), _p(scales, ctypes.c_float), _p(zeros, ctypes.c_float),
                                     n, dim, group, bits, _p(out, ctypes.c_float))
    if rc != 0:
        raise ValueError(f"tqo_dequantize_values failed with status {rc}")
    return out.reshape(*scales.shape[:-1], dim)


# --------------------------------------------------------------------------------------------------
# decode attention (ops.py:1552-1574, turboquant.py:1275-1293)


def gqa_decode(q, k, v, scaling: float, gate=None) -> np.ndarray:
    """q [Hq, D], k/v [Hkv, L, D] (float32) -> [Hq, D]; softmax in fp32; L == 0 -> zeros."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    hq, dim = q.shape
    hkv, length = k.shape[0], k.shape[1]
    out = np.zeros((hq, dim), dtype=np.float32)
    gp = ctypes.POINTER(ctypes.c_float)()
    if gate is not None:
        gate = _f32(gate).reshape(hq, dim)
        gp = _p(gate, ctypes.c_float)
    rc = lib().tqo_gqa_decode(_p(q, ctypes.c_float), _p(k, ctypes.c_float), _p(v, ctypes.c_float), gp, hq, hkv,
                              length, dim, float(scaling), _p(out, ctypes.c_float))
    if rc != 0:
        raise ValueError(f"tqo_gqa_decode failed with status {rc}")
    return out


def gqa_decode_blas(q, k, v, scaling: float, gate=None) -> np.ndarray:
    """Same math through numpy matmul (multi-threaded BLAS); used for the timed CPU baseline.  k / v may be views of
    larger buffers (a decode cache with spare capacity): they are not copied."""
    q, k, v = _f32(q), np.asarray(k, dtype=np.float32), np.asarray(v, dtype=np.float32)
    hq, dim = q.shape
    hkv = k.shape[0]
    if k.shape[1] == 0:
        return np.zeros((hq, dim), dtype=np.float32)
    grouped = q.reshape(hkv, hq // hkv, dim)
    scores = np.matmul(grouped, k.transpose(0, 2, 1)) * np.float32(scaling)
    scores -= scores.max(axis=-1, keepdims=True)
    probs = np.exp(scores, dtype=np.float32)
    probs /= probs.sum(axis=-1, keepdims=True)
    out = np.matmul(probs, v).reshape(hq, dim)
    if gate is not None:
        out = out * (1.0 / (1.0 + np.exp(-_f32(gate).reshape(hq, dim))))
    return out.astype(np.float32)


def grouped_query_attention(q, k, v, scaling: float, *, causal_mask=None, visible_mask=None,
                            key_padding_mask=None) -> np.ndarray:
    """Multi-token attention with the reference's masks (ops.py:1552-1574), numpy fp32.

    q [B, Hq, T, D], k/v [B, Hkv, L, D]; causal_mask bool [B, T, L] (True = hidden), visible_mask and
    key_padding_mask bool [B, L] (True = visible).  softmax in fp32.  A query row with every key hidden gives NaN in
    the reference (softmax of all -inf); this restatement returns zeros there and the tests avoid comparing such rows
    with the reference itself."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    batch, hq, t, dim = q.shape
    hkv = k.shape[1]
    grouped = q.reshape(batch, hkv, hq // hkv, t, dim)
    scores = np.matmul(grouped, k[:, :, None].transpose(0, 1, 2, 4, 3)) * np.float32(scaling)
    hidden = np.zeros((batch, 1, 1, t, k.shape[2]), dtype=bool)
    if causal_mask is not None:
        hidden |= np.asarray(causal_mask, dtype=bool)[:, None, None, :, :]
    if visible_mask is not None:
        hidden |= ~np.asarray(visible_mask, dtype=bool)[:, None, None, None, :]
    if key_padding_mask is not None:
        hidden |= ~np.asarray(key_padding_mask, dtype=bool)[:, None, None, None, :]
    scores = np.where(hidden, -np.inf, scores).astype(np.float32)
    top = scores.max(axis=-1, keepdims=True)
    top = np.where(np.isfinite(top), top, 0.0)
    probs = np.exp(scores - top, dtype=np.float32)
    denom = probs.sum(axis=-1, keepdims=True)
    probs = np.divide(probs, denom, out=np.zeros_like(probs), where=denom > 0)
    out = np.matmul(probs, v[:, :, None])
    return out.reshape(batch, hq, t, dim).astype(np.float32)


from .kv_state import (  # noqa: E402
    OracleLayerAllocator,
    OracleTurboQuantRow,
    PackedPageLayout,
    pack_key_codes,
    unpack_key_codes,
    paged_blocks_needed,
)

__all__ = [
    "DTYPE_F32", "DTYPE_F16", "DTYPE_BF16", "build", "lib", "round_bf16", "round_dtype", "dtype_size", "codebook",
    "signs", "fwht", "key_index_bits", "quantize_keys", "dequantize_keys", "qjl_matrix", "resolve_value_group_size",
    "quantize_values", "dequantize_values", "gqa_decode", "gqa_decode_blas", "OracleLayerAllocator",
    "OracleTurboQuantRow", "PackedPageLayout", "pack_key_codes", "unpack_key_codes", "paged_blocks_needed",
]
