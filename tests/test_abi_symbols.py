"""CPU: the shared library loads, exports every symbol include/anna_b200_kv.h declares, and the ctypes signatures
agree with the header's parameter lists.  No compute call is made."""
from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest

from anna_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "anna_b200_kv.h"


def _declarations() -> dict[str, list[str]]:
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    text = re.sub(r"^\s*#.*$", "", text, flags=re.M)
    decls: dict[str, list[str]] = {}
    for match in re.finditer(r"([A-Za-z_][\w\s\*]*?)\b(anna_\w+)\s*\(([^;{}]*?)\)\s*;", text):
        params = match.group(3).strip()
        decls[match.group(2)] = [] if params in ("", "void") else [p.strip() for p in params.split(",")]
    return decls


@pytest.fixture(scope="module")
def library():
    if not _lib.library_path().exists():
        from anna_b200.build import build

        build()
    return _lib.lib()


def test_header_declares_the_expected_entry_points():
    names = set(_declarations())
    assert {"anna_kv_last_error", "anna_kv_abi_version", "anna_decode_plan", "anna_paged_kv_write",
            "anna_paged_gqa_decode", "anna_gqa_decode", "anna_gqa_prefill", "anna_tq_page_layout", "anna_tq_append",
            "anna_tq_paged_decode", "anna_tq_materialize", "anna_gqa_decode_turboquant_values",
            "anna_tq_decode_plan", "anna_kv_device_faults", "anna_tq_tensor_row_bytes",
            "anna_tq_tensor_quantize", "anna_tq_tensor_dequantize", "anna_tq_gather_dense", "anna_kv_selftest_wait_expiry", "anna_kv_selftest_umma",
            "anna_tq_query_scratch_bytes"} <= names


def test_library_exports_every_declared_symbol(library):
    for name in _declarations():
        assert hasattr(library, name), f"{name} is declared in the header but not exported"


def test_ctypes_signatures_match_header(library):
    decls = _declarations()
    assert set(decls) == set(_lib.SIGNATURES), set(decls) ^ set(_lib.SIGNATURES)

    def kind(param: str) -> str:
        if "*" in param or "anna_stream_t" in param:
            return "ptr"
        if "float" in param:
            return "f32"
        if "int64_t" in param:
            return "i64"
        if "size_t" in param:
            return "size"
        return "i32"

    ctype_kind = {ctypes.c_int: "i32", ctypes.c_int64: "i64", ctypes.c_float: "f32", ctypes.c_void_p: "ptr",
                  ctypes.c_size_t: "size"}
    for name, params in decls.items():
        _, argtypes = _lib.SIGNATURES[name]
        assert len(argtypes) == len(params), name
        for position, (param, ctype) in enumerate(zip(params, argtypes)):
            got = ctype_kind.get(ctype, "ptr")  # POINTER(...) types count as pointers
            assert got == kind(param), f"{name} argument {position} ({param!r}) bound as {got}"


def test_abi_version_and_plan_are_host_only_calls(library):
    assert library.anna_kv_abi_version() == 1
    chunk, chunks = _lib.decode_plan(32, 8, 8192)
    assert chunk >= 64 and chunks * chunk >= 8192
    chunk, chunks = _lib.decode_plan(1, 1, 0)
    assert chunks == 1
    with pytest.raises(RuntimeError, match="anna_decode_plan"):
        _lib.decode_plan(0, 8, 128)


def test_page_layout_matches_oracle_layout(library):
    import oracle

    for dim in (64, 128, 256):
        for bits in (2, 3, 4):
            for block in (4, 16, 32):
                for code, size in ((0, 4), (2, 2)):
                    got = _lib.tq_page_layout(dim, bits, block, code, 32)
                    want = oracle.PackedPageLayout(head_dim=dim, bits=bits, block_size=block, dtype_bytes=size, group=32)
                    for field in ("key_bytes", "value_bytes", "groups", "off_kcodes", "off_knorm", "off_krnorm",
                                  "off_vdata", "off_vscale", "off_vzero", "chunk_bytes"):
                        assert got[field] == getattr(want, field), (dim, bits, block, field)
    # algorithmic bytes per token-head of the benchmark configurations (D*b/8 + 8 for keys, D*sb/8 + 2*(D/32)*e for values)
    assert oracle.PackedPageLayout(128, 4, 16, 2, 32).bytes_per_token() == 152
    assert oracle.PackedPageLayout(256, 2, 16, 2, 32).bytes_per_token() == 168
    assert oracle.PackedPageLayout(128, 3, 16, 2, 32).bytes_per_token() == 136
    assert oracle.PackedPageLayout(128, 4, 16, 4, 32).bytes_per_token() == 168


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libanna_b200_kv.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.lib()
