"""Statistical properties of this build's key quantizer (CPU, oracle only).  The reference delegates the arithmetic to
the un-vendored `turboquant` package, so the bit-exact GPU parity tests pin the kernels to THIS definition; these tests
pin the definition itself to what the published algorithm promises: a Lloyd-Max codebook for the rotated coordinate and
an inner-product estimate that stays unbiased with the structured (sign-flip Walsh-Hadamard) projection, for which the
reference's scale sqrt(pi/2) / D (src/anna/model/turboquant.py:316-332) was derived with Gaussian rows."""
from __future__ import annotations

import math

import numpy as np
import pytest

import oracle


def _outlier_keys(rng, n: int, dim: int) -> np.ndarray:
    keys = rng.standard_normal((n, dim)).astype(np.float32)
    keys[:, rng.choice(dim, 4, replace=False)] *= 8.0  # BASELINE config 1: four outlier channels scaled by 8
    return keys


@pytest.mark.parametrize("dim,bits", [(128, 4), (128, 3), (128, 2), (256, 2), (64, 4)])
def test_inner_product_estimate_is_unbiased_with_the_structured_projection(dim, bits):
    """Slope of the estimated <q, k> against the true one over 6000 outlier keys: 1 within 1.5 % for the index + sign
    code; the index-only reconstruction of the same codes shrinks inner products (slope visibly below 1 at 2 bits)."""
    rng = np.random.default_rng(1000 * dim + bits)
    n = 6000
    keys = _outlier_keys(rng, n, dim)
    queries = rng.standard_normal((n, dim)).astype(np.float32)
    idx, sign, norms, rnorms = oracle.quantize_keys(keys, bits)
    full = oracle.dequantize_keys(idx, sign, norms, rnorms, bits)
    index_only = oracle.dequantize_keys(idx, None, norms, None, bits)
    true = np.einsum("nd,nd->n", queries, keys).astype(np.float64)
    est = np.einsum("nd,nd->n", queries, full).astype(np.float64)
    est_index = np.einsum("nd,nd->n", queries, index_only).astype(np.float64)
    slope = float(est @ true / (true @ true))
    slope_index = float(est_index @ true / (true @ true))
    assert abs(slope - 1.0) <= 0.015, slope
    assert slope_index < slope + 0.005
    if bits == 2:
        assert slope_index < 0.97, slope_index
    # and the residual error is not correlated with the query direction: its mean is zero within 4 standard errors
    err = est - true
    assert abs(err.mean()) <= 4.0 * err.std() / math.sqrt(n), (err.mean(), err.std())


def test_zero_residual_norms_give_the_index_only_reconstruction():
    """The reference asks for the index-only reconstruction by passing zero signs and zero residual norms
    (turboquant.py:318-320); with zero residual norms the sign term vanishes whatever the signs are."""
    rng = np.random.default_rng(7)
    keys = _outlier_keys(rng, 50, 128)
    idx, sign, norms, rnorms = oracle.quantize_keys(keys, 4)
    want = oracle.dequantize_keys(idx, None, norms, None, 4)
    got = oracle.dequantize_keys(idx, sign, norms, np.zeros_like(rnorms), 4)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("dim,index_bits", [(64, 1), (64, 3), (128, 1), (128, 2), (128, 3), (256, 1), (256, 3)])
def test_codebook_is_a_lloyd_max_fixed_point_of_the_rotated_coordinate(dim, index_bits):
    """The rotated, normalised coordinate times sqrt(D) has density (1 - x^2 / D)^((D - 3) / 2) on [-sqrt(D), sqrt(D)].
    Boundaries are midpoints of neighbouring centroids and every centroid is the mean of its cell (numerical
    integration on a fine grid)."""
    cent, bnd = oracle.codebook(dim, index_bits)
    cent = cent.astype(np.float64)
    bnd = bnd.astype(np.float64)
    assert len(cent) == 1 << index_bits and len(bnd) == len(cent) - 1
    np.testing.assert_allclose(bnd, (cent[:-1] + cent[1:]) / 2.0, atol=2e-6)
    np.testing.assert_allclose(cent, -cent[::-1], atol=2e-6)  # symmetric density
    limit = math.sqrt(dim)
    x = np.linspace(-limit, limit, 2_000_001)
    density = np.clip(1.0 - x * x / dim, 0.0, None) ** ((dim - 3) / 2.0)
    edges = np.concatenate([[-limit], bnd, [limit]])
    for i in range(len(cent)):
        cell = (x >= edges[i]) & (x <= edges[i + 1])
        mean = float((x[cell] * density[cell]).sum() / density[cell].sum())
        assert abs(mean - cent[i]) <= 2e-4, (i, mean, cent[i])
