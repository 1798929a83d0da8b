"""CPU: the oracle against fixtures produced by the reference itself (tests/golden/make_golden.py)."""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from tests.golden.make_golden import config1_inputs
from tests.helpers import to_np

GOLDEN = Path(__file__).resolve().parent / "golden"
DTYPES = {"bf16": oracle.DTYPE_BF16, "f16": oracle.DTYPE_F16, "f32": oracle.DTYPE_F32}


def _digest(array: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(array).tobytes()).hexdigest()


def test_value_quantizer_matches_reference_bit_for_bit():
    data = np.load(GOLDEN / "value_quantizer.npz")
    cases = sorted({key.rsplit("_", 1)[0] for key in data.files})
    assert len(cases) == 27
    for case in cases:
        dtype_name, bits, dim, group = case.split("_")
        bits, group = int(bits[1:]), int(group[1:])
        packed, scales, zeros = oracle.quantize_values(data[case + "_x"], bits, group, DTYPES[dtype_name])
        np.testing.assert_array_equal(packed, data[case + "_data"], err_msg=case)
        np.testing.assert_array_equal(scales.view(np.uint32), data[case + "_scales"].view(np.uint32), err_msg=case)
        np.testing.assert_array_equal(zeros.view(np.uint32), data[case + "_zeros"].view(np.uint32), err_msg=case)
        deq = oracle.dequantize_values(packed, scales, zeros, bits, group)
        np.testing.assert_array_equal(deq.view(np.uint32), data[case + "_deq"].view(np.uint32), err_msg=case)


def test_value_group_size_rule():
    # turboquant.py:157-161
    assert [oracle.resolve_value_group_size(d) for d in (256, 128, 64, 48, 24, 7)] == [32, 32, 32, 16, 8, 1]


def test_allocator_policy_matches_reference_trace():
    trace = json.loads((GOLDEN / "allocator_trace.json").read_text())
    alloc = oracle.OracleLayerAllocator()
    for entry in trace:
        op, arg = entry["op"], entry["arg"]
        if op == "allocate":
            assert alloc.allocate(arg) == entry["result"]
        elif op == "release":
            alloc.release_pages(arg)
        elif op == "ensure_capacity":
            assert alloc.ensure_capacity(arg) == entry["result"]
        elif op == "retain":
            alloc.retain_page(arg)
        elif op == "release_all":
            for ids in (trace[1]["result"], trace[3]["result"], trace[9]["result"]):
                alloc.release_pages(ids)
        elif op == "trim":
            assert alloc.trim() == entry["result"]
        assert alloc.capacity == entry["capacity"], entry
        assert alloc.free_pages == entry["free"], entry
        assert alloc.used_pages() == entry["used"], entry


def test_config1_rows_match_reference_run():
    """Config 1 through the reference's TurboQuantKVRow (key arithmetic supplied by the shim) == oracle rows."""
    golden = np.load(GOLDEN / "config1_turboquant.npz")
    digests = json.loads((GOLDEN / "config1_input_digests.json").read_text())
    prefill_k, prefill_v, steps = config1_inputs()
    assert _digest(prefill_k.numpy()) == digests["prefill_k"], "torch's CPU generator no longer reproduces the inputs"
    assert _digest(prefill_v.numpy()) == digests["prefill_v"]
    rows = [oracle.OracleTurboQuantRow(bits=4, residual_len=128, dtype=oracle.DTYPE_F32) for _ in range(2)]
    for b, row in enumerate(rows):
        row.append(to_np(prefill_k[b]), to_np(prefill_v[b]))
    for step, (k, v, q) in enumerate(steps):
        for b, row in enumerate(rows):
            row.append(to_np(k[b]), to_np(v[b]))
        if step in (0, 21, 42, 63):
            assert _digest(q.numpy()) == digests[f"q_step{step}"]
            got = np.stack([row.decode_attention(to_np(q[b, :, 0]), scaling=128 ** -0.5) for b, row in enumerate(rows)])
            np.testing.assert_allclose(got[:, :, None, :], golden[f"out_step{step}"], atol=2e-5, rtol=2e-5)
    for b, row in enumerate(rows):
        assert [row.length, row.quantized_length, row.residual_length] == golden[f"row{b}_lengths"].tolist()
        np.testing.assert_array_equal(row.idx, golden[f"row{b}_idx"])
        np.testing.assert_array_equal(np.packbits(row.sign, axis=-1, bitorder="little"), golden[f"row{b}_sign_bits"])
        np.testing.assert_array_equal(row.norms.view(np.uint32), golden[f"row{b}_norms"].view(np.uint32))
        np.testing.assert_array_equal(row.rnorms.view(np.uint32), golden[f"row{b}_rnorms"].view(np.uint32))
        np.testing.assert_array_equal(row.vdata, golden[f"row{b}_vdata"])
        np.testing.assert_array_equal(row.vscales.view(np.uint32), golden[f"row{b}_vscales"].view(np.uint32))
        np.testing.assert_array_equal(row.vzeros.view(np.uint32), golden[f"row{b}_vzeros"].view(np.uint32))


def test_decode_oracle_matches_reference_splitkv_case():
    """tests/test_fused_op_xpu.py:647-703 on CPU semantics: Hq=8, Hkv=2, D=64, Lq=77, R=5, group 16, bits 2/3/4."""
    data = np.load(GOLDEN / "splitkv_turboquant_case.npz")
    for bits in (2, 3, 4):
        p = f"b{bits}_"
        packed, scales, zeros = oracle.quantize_values(data[p + "dense_v"], bits, 16, oracle.DTYPE_BF16)
        np.testing.assert_array_equal(packed, data[p + "vdata"])
        deq = oracle.round_bf16(oracle.dequantize_values(packed, scales, zeros, bits, 16))
        keys = np.concatenate([data[p + "qkey"][0], data[p + "rkey"][0]], axis=1)
        values = np.concatenate([deq, data[p + "rvalue"][0]], axis=1)
        got = oracle.gqa_decode(data[p + "query"][0, :, 0], keys, values, 64 ** -0.5, gate=data[p + "gate"][0, :, 0])
        # the reference result carries bf16 matmul rounding; its own test allows 4e-2
        np.testing.assert_allclose(got, data[p + "ref"][0, :, 0], atol=4e-2, rtol=4e-2)
        assert np.abs(got - data[p + "ref"][0, :, 0]).max() < 2e-2


def test_key_quantizer_structure_and_quality():
    """Properties the reference's tests bound (tests/test_model_shapes.py:374-375 MSE < 1.0; estimator identity of
    turboquant.py:316-332): reconstruction error, un-biasedness of the inner-product estimate, exact identity between
    de-quantised scores and rotated-basis scores."""
    rng = np.random.default_rng(0)
    for dim in (64, 128, 256):
        for bits in (2, 3, 4):
            x = rng.standard_normal((400, dim)).astype(np.float32)
            idx, sign, norms, rnorms = oracle.quantize_keys(x, bits)
            assert idx.max() < (1 << (bits - 1)) and set(np.unique(sign)) <= {0, 1}
            np.testing.assert_allclose(norms, np.linalg.norm(x, axis=1), rtol=1e-5)
            k_hat = oracle.dequantize_keys(idx, sign, norms, rnorms, bits)
            assert float(((k_hat - x) ** 2).mean()) < 0.5
            q = rng.standard_normal((dim,)).astype(np.float32)
            est, true = k_hat @ q, x @ q
            assert abs(float((est - true).mean())) < 0.35 * float(np.abs(true).mean())
            cent, _ = oracle.codebook(dim, bits - 1)
            s1, s2 = oracle.signs(dim, 0), oracle.signs(dim, 1)
            q1 = oracle.fwht(s1 * q)
            q2 = oracle.fwht(s2 * q1)
            kappa = np.sqrt(np.pi / 2) / np.sqrt(dim)
            rotated = norms / dim * ((cent[idx] @ q1) + kappa * rnorms * ((2.0 * sign - 1.0) @ q2))
            np.testing.assert_allclose(rotated, est, rtol=2e-4, atol=2e-4)


def test_qjl_matrix_is_scaled_orthogonal_and_matches_transform():
    dim = 64
    S = oracle.qjl_matrix(dim)
    np.testing.assert_allclose(S @ S.T, dim * np.eye(dim), atol=1e-3)
    r = np.random.default_rng(1).standard_normal(dim).astype(np.float32)
    want = oracle.fwht(oracle.signs(dim, 1) * oracle.fwht(oracle.signs(dim, 0) * r)) / np.sqrt(dim)
    np.testing.assert_allclose(S @ r, want, atol=1e-4)


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_key_code_packing_round_trips(bits):
    rng = np.random.default_rng(bits)
    idx = rng.integers(0, 1 << (bits - 1), size=(2, 5, 128)).astype(np.uint8)
    sign = rng.integers(0, 2, size=(2, 5, 128)).astype(np.uint8)
    packed = oracle.pack_key_codes(idx, sign, bits)
    assert packed.shape == (2, 5, 128 * bits // 8)
    got_idx, got_sign = oracle.unpack_key_codes(packed, bits, 128)
    np.testing.assert_array_equal(got_idx, idx)
    np.testing.assert_array_equal(got_sign, sign)


def test_bf16_rounding_matches_torch():
    x = (torch.randn(4096) * 37).float()
    x[:4] = torch.tensor([0.0, -0.0, 1e-40, 3.4e38])
    np.testing.assert_array_equal(oracle.round_bf16(x.numpy()), x.to(torch.bfloat16).float().numpy())
    for value in x[:64].tolist():
        assert oracle.lib().tqo_f32_to_f16(value) == int(torch.tensor(value).half().view(torch.int16).item()) & 0xFFFF


@pytest.mark.parametrize("dim,bits", [(64, 2), (128, 3), (256, 4), (512, 4)])
def test_mse_variant_round_trip_quality(dim, bits):
    """The MSE-only quantizer of tensor rows (turboquant.py:75-82, :392-418): `bits` index bits, no sign plane; the
    reconstruction error of unit-scale data stays under the reference's own bound for this row type (< 0.5,
    tests/test_gemma4_text_runtime.py:339-340) and shrinks as bits grow."""
    rng = np.random.default_rng(dim + bits)
    x = rng.standard_normal((64, dim)).astype(np.float32)
    idx, sign, norms, rnorms = oracle.quantize_keys(x, bits, "mse")
    assert sign is None and rnorms is None and idx.max() < (1 << bits) and idx.dtype == np.uint8
    np.testing.assert_allclose(norms, np.linalg.norm(x, axis=-1), rtol=1e-5)
    recon = oracle.dequantize_keys(idx, None, norms, None, bits, "mse")
    mse = float(((recon - x) ** 2).mean())
    assert mse < 0.5
    coarse = oracle.dequantize_keys(*(lambda r: (r[0], None, r[2], None))(oracle.quantize_keys(x, 2, "mse")), 2, "mse")
    assert mse <= float(((coarse - x) ** 2).mean()) + 1e-6


def _masks(lengths: np.ndarray, q_len: int, key_len: int, causal: bool):
    positions = np.arange(key_len)[None, :]
    visible = positions < lengths[:, None]
    causal_mask = None
    if causal:
        q_positions = (lengths - q_len)[:, None] + np.arange(q_len)[None, :]
        causal_mask = positions[:, None, :] > q_positions[:, :, None]
    return causal_mask, visible


@pytest.mark.parametrize("case", ["chunk", "full", "padding_only"])
def test_grouped_query_attention_matches_reference(case):
    """oracle.grouped_query_attention against outputs of the reference's own function (ops.py:1552-1574) run with the
    masks the model builds."""
    data = np.load(GOLDEN / "prefill_attention.npz")
    q, k, v = (data[f"{case}_{n}"].astype(np.float32) for n in ("q", "k", "v"))
    lengths = data[f"{case}_lengths"]
    causal_mask, visible = _masks(lengths, q.shape[2], k.shape[2], bool(data[f"{case}_causal"]))
    out = oracle.grouped_query_attention(q, k, v, q.shape[3] ** -0.5, causal_mask=causal_mask, visible_mask=visible)
    ref = data[f"{case}_ref"]
    hidden = ~np.isfinite(ref)  # queries without a visible key: NaN in the reference, zeros here
    assert hidden.any() == (case == "full")
    np.testing.assert_allclose(out[~hidden], ref[~hidden], atol=2e-5, rtol=1e-5)
    assert not out[hidden].any()


def test_incremental_decode_cache_equals_full_rematerialisation():
    """The oracle row that extends its dense decode cache in place at every append (the reference's
    _KEEP_DECODE_CACHE, src/anna/model/turboquant.py:742-782, :1089-1140) sees exactly the keys and values of the row
    that de-quantizes its whole prefix at every call, across prefill, decode steps and a second chunk."""
    rng = np.random.default_rng(5)
    plain = oracle.OracleTurboQuantRow(bits=3, residual_len=8, dtype=oracle.DTYPE_BF16)
    cached = oracle.OracleTurboQuantRow(bits=3, residual_len=8, dtype=oracle.DTYPE_BF16, keep_decode_cache=True)
    for tokens in (5, 7, 1, 1, 40, 1):
        k = oracle.round_bf16(rng.standard_normal((2, tokens, 64), dtype=np.float32))
        v = oracle.round_bf16(rng.standard_normal((2, tokens, 64), dtype=np.float32))
        plain.append(k, v)
        cached.append(k, v)
        for got, want in zip(cached.materialize(), plain.materialize()):
            np.testing.assert_array_equal(got, want)
        for name in ("idx", "sign", "norms", "rnorms", "vdata", "vscales", "vzeros"):
            np.testing.assert_array_equal(getattr(cached, name), getattr(plain, name))
    q = rng.standard_normal((4, 64), dtype=np.float32)
    np.testing.assert_allclose(cached.decode_attention(q, scaling=0.125, blas=True),
                               plain.decode_attention(q, scaling=0.125), atol=1e-5, rtol=1e-5)
