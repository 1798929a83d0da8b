"""ctypes binding of libanna_b200_kv.so (the C ABI declared in include/anna_b200_kv.h).

There is no CPU fallback: if the shared library is missing or fails to load, every call raises ``RuntimeError``
telling the user to build it (``python -m anna_b200.build``).
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libanna_b200_kv.so"

DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2
DEV_BAD_PAGE = 1

_LOCK = threading.Lock()
_LIB: ctypes.CDLL | None = None

c_i32 = ctypes.c_int
c_i64 = ctypes.c_int64
c_f32 = ctypes.c_float
c_ptr = ctypes.c_void_p
c_size = ctypes.c_size_t


class TqLayout(ctypes.Structure):
    _fields_ = [(name, ctypes.c_int32) for name in (
        "key_bytes", "value_bytes", "groups", "off_kcodes", "off_knorm", "off_krnorm", "off_vdata", "off_vscale",
        "off_vzero", "chunk_bytes")]

    def as_dict(self) -> dict[str, int]:
        return {name: int(getattr(self, name)) for name, _ in self._fields_}


# name -> (restype, argtypes); the order is the declaration order of include/anna_b200_kv.h
SIGNATURES: dict[str, tuple[object, list[object]]] = {
    "anna_kv_last_error": (ctypes.c_char_p, []),
    "anna_kv_abi_version": (c_i32, []),
    "anna_kv_device_faults": (c_i32, [ctypes.POINTER(c_i32)]),
    "anna_kv_selftest_wait_expiry": (c_i32, [ctypes.POINTER(c_i32), c_ptr]),
    "anna_kv_selftest_umma": (c_i32, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, ctypes.POINTER(c_i32), c_ptr]),
    "anna_decode_plan": (c_i32, [c_i32, c_i32, c_i64, ctypes.POINTER(c_i32), ctypes.POINTER(c_i32)]),
    "anna_paged_kv_write": (c_i32, [c_ptr, c_ptr, c_i64, c_i64, c_i64, c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_i32,
                                    c_i32, c_i32, c_i32, c_i32, c_i64, c_i64, c_i32, c_ptr, c_ptr]),
    "anna_block_table_patch": (c_i32, [c_ptr, c_i64, c_i64, c_i64, c_ptr, c_i32, c_ptr]),
    "anna_paged_kv_gather": (c_i32, [c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_i64, c_i32, c_i32,
                                     c_i32, c_i32, c_i64, c_i64, c_i64, c_i32, c_ptr]),
    "anna_paged_gqa_decode": (c_i32, [c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_i64, c_i64,
                                      c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_i32, c_i32, c_ptr, c_i32, c_i32, c_i32, c_i32,
                                      c_i32, c_i64, c_i64, c_f32, c_i32, c_ptr]),
    "anna_noalloc_scratch_bytes": (c_size, []),
    "anna_paged_gqa_decode_noalloc": (c_i32, [c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_i64,
                                              c_i64, c_ptr, c_i64, c_i64, c_i32, c_i32, c_i32, c_i32, c_i32, c_i64,
                                              c_i64, c_f32, c_i32, c_ptr]),
    "anna_gqa_decode": (c_i32, [c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_i64, c_i64, c_i64, c_ptr, c_ptr, c_i64, c_i64,
                                c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_i32, c_i32, c_ptr, c_i32, c_i32, c_i32, c_i64,
                                c_i32, c_f32, c_i32, c_ptr]),
    "anna_gqa_prefill": (c_i32, [c_ptr, c_i64, c_i64, c_i64, c_ptr, c_ptr, c_i64, c_i64, c_i64, c_ptr, c_ptr, c_i64,
                                 c_i64, c_i64, c_i32, c_i32, c_i32, c_i32, c_i64, c_i32, c_f32, c_i32, c_i32, c_ptr]),
    "anna_tq_page_layout": (c_i32, [c_i32, c_i32, c_i32, c_i32, c_i32, ctypes.POINTER(TqLayout)]),
    "anna_tq_append": (c_i32, [c_ptr, c_ptr, c_i64, c_i64, c_i64, c_ptr, c_ptr, c_i64, c_ptr, c_i64, c_ptr, c_ptr, c_ptr,
                               c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_i64,
                               c_i64, c_i32, c_ptr, c_ptr]),
    "anna_tq_paged_decode": (c_i32, [c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr,
                                     c_ptr, c_ptr, c_i64, c_i64, c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_i32, c_i32,
                                     c_ptr, c_ptr, c_size, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_i64,
                                     c_i64, c_f32, c_i32, c_ptr]),
    "anna_tq_paged_decode_peers": (c_i32, [c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr,
                                           c_ptr, c_ptr, c_i64, c_i64, c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_i32, c_i32,
                                           c_ptr, c_ptr, c_size, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32,
                                           c_i64, c_i64, c_f32, c_i32, c_ptr, c_i32, c_ptr]),
    "anna_peer_signal_wait": (c_i32, [c_ptr, c_i32, c_i32, c_i64, c_i64, c_ptr, c_ptr]),
    "anna_kv_selftest_umma_tma": (c_i32, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, ctypes.POINTER(c_i32), c_ptr]),
    "anna_kv_selftest_umma_ts": (c_i32, [c_ptr, c_ptr, c_ptr, ctypes.POINTER(c_i32), c_ptr]),
    "anna_tq_decode_plan": (c_i32, [c_i32, c_i32, c_i64, c_i32, c_i32, ctypes.POINTER(c_i32), ctypes.POINTER(c_i32)]),
    "anna_tq_query_scratch_bytes": (c_size, [c_i32, c_i32, c_i32, c_i32]),
    "anna_gqa_decode_turboquant_values": (c_i32, [c_ptr, c_i64, c_i64, c_ptr, c_i64, c_i64, c_i64, c_ptr, c_i64, c_i64,
                                                  c_i64, c_ptr, c_ptr, c_i64, c_i64, c_i64, c_ptr, c_ptr, c_i64, c_i64,
                                                  c_i64, c_ptr, c_i64, c_i64, c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_i32,
                                                  c_i32, c_i32, c_i32, c_i32, c_i64, c_i64, c_i32, c_i32, c_i32, c_f32,
                                                  c_i32, c_ptr]),
    "anna_tq_gather_dense": (c_i32, [c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64,
                                     c_i64, c_i64, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_i64, c_i64, c_i64,
                                     c_i32, c_ptr]),
    "anna_tq_tensor_row_bytes": (c_i32, [c_i32, c_i32]),
    "anna_tq_tensor_quantize": (c_i32, [c_ptr, c_i64, c_i64, c_ptr, c_ptr, c_i64, c_i64, c_i32, c_i32, c_i32, c_i32,
                                        c_ptr, c_ptr, c_i32, c_ptr]),
    "anna_tq_tensor_dequantize": (c_i32, [c_ptr, c_ptr, c_i64, c_i64, c_ptr, c_i64, c_i64, c_i32, c_i32, c_i32, c_i32,
                                          c_ptr, c_ptr, c_i32, c_ptr]),
    "anna_tq_materialize": (c_i32, [c_ptr, c_ptr, c_i64, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_i64,
                                    c_i32, c_i32, c_i32, c_i32, c_i32, c_i32, c_i64, c_i64, c_i64, c_i32, c_ptr]),
}


def library_path() -> Path:
    return LIB_PATH


def lib() -> ctypes.CDLL:
    """Load the shared library once; raise loudly when it is not there."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: the CUDA library of anna_b200 has not been built. "
                "Run `python -m anna_b200.build` (needs nvcc). There is no CPU fallback for this path.")
        try:
            handle = ctypes.CDLL(str(LIB_PATH))
        except OSError as exc:
            raise RuntimeError(f"failed to load {LIB_PATH}: {exc}. There is no CPU fallback for this path.") from exc
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                raise RuntimeError(f"{LIB_PATH} does not export {name}; rebuild it with `python -m anna_b200.build`.")
            fn.restype = restype
            fn.argtypes = argtypes
        _LIB = handle
    return _LIB


def device_faults() -> int:
    """Bounded in-kernel waits that expired on the current device (0 in a healthy run); synchronises the device."""
    count = c_i32(0)
    check(lib().anna_kv_device_faults(ctypes.byref(count)), "anna_kv_device_faults")
    return int(count.value)


def last_error() -> str:
    return lib().anna_kv_last_error().decode("utf-8", "replace")


def check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what} failed (status {status}): {last_error()}")


def decode_plan(batch: int, kv_heads: int, max_len: int) -> tuple[int, int]:
    chunk = c_i32(0)
    chunks = c_i32(0)
    check(lib().anna_decode_plan(batch, kv_heads, max_len, ctypes.byref(chunk), ctypes.byref(chunks)),
          "anna_decode_plan")
    return int(chunk.value), int(chunks.value)


def tq_decode_plan(batch: int, kv_heads: int, max_blocks: int, block_size: int, residual_len: int) -> tuple[int, int]:
    chunk = c_i32(0)
    chunks = c_i32(0)
    check(lib().anna_tq_decode_plan(batch, kv_heads, max_blocks, block_size, residual_len, ctypes.byref(chunk),
                                    ctypes.byref(chunks)), "anna_tq_decode_plan")
    return int(chunk.value), int(chunks.value)


def tq_page_layout(head_dim: int, bits: int, block_size: int, dtype_code: int, value_group: int) -> dict[str, int]:
    layout = TqLayout()
    check(lib().anna_tq_page_layout(head_dim, bits, block_size, dtype_code, value_group, ctypes.byref(layout)),
          "anna_tq_page_layout")
    return layout.as_dict()
