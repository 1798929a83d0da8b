"""Generate the frozen Lloyd-Max codebooks used by the TurboQuant key quantizer.

A unit vector rotated by a random orthogonal matrix has coordinates whose marginal density is
f(y) ~ (1 - y^2)^((D-3)/2) on (-1, 1).  In the scaled variable w = sqrt(D) * y this is close to N(0, 1).
For every supported head_dim D and index width m (1..4 bits) this script runs Lloyd-Max on that exact
density (trapezoid integration on a fixed float64 grid) and stores the 2^m centroids and the 2^m - 1
decision boundaries (midpoints) as float32 bit patterns, so that every consumer (CUDA kernels, the CPU
oracle, the Python host code) compares against the same 32-bit constants.

Run:  python anna_b200/data/gen_tq_codebooks.py   (rewrites tq_codebooks.json next to this file)
"""
from __future__ import annotations

import json
import struct
from pathlib import Path

import numpy as np

HEAD_DIMS = (32, 64, 128, 256, 512)
INDEX_BITS = (1, 2, 3, 4)
GRID_POINTS = 400001
ITERATIONS = 400


def _f32_hex(value: float) -> str:
    return struct.pack(">f", np.float32(value)).hex()


def lloyd_max(dim: int, bits: int) -> tuple[np.ndarray, np.ndarray]:
    half = np.sqrt(float(dim))
    grid = np.linspace(-half, half, GRID_POINTS, dtype=np.float64)
    base = np.clip(1.0 - (grid * grid) / float(dim), 0.0, None)
    density = np.power(base, (dim - 3) / 2.0)
    step = grid[1] - grid[0]
    weight = density.copy()
    weight[0] *= 0.5
    weight[-1] *= 0.5
    weight *= step
    weight /= weight.sum()
    cdf = np.cumsum(weight)
    levels = 1 << bits
    # start from equal-probability cells
    targets = (np.arange(levels, dtype=np.float64) + 0.5) / levels
    centroids = np.interp(targets, cdf, grid)
    moment = weight * grid
    for _ in range(ITERATIONS):
        bounds = 0.5 * (centroids[1:] + centroids[:-1])
        cells = np.searchsorted(bounds, grid, side="left")
        mass = np.bincount(cells, weights=weight, minlength=levels)
        first = np.bincount(cells, weights=moment, minlength=levels)
        centroids = first / np.maximum(mass, 1e-300)
    # enforce exact odd symmetry, then freeze to float32
    centroids = 0.5 * (centroids - centroids[::-1])
    centroids32 = centroids.astype(np.float32)
    bounds32 = (0.5 * (centroids32[1:].astype(np.float64) + centroids32[:-1].astype(np.float64))).astype(np.float32)
    return centroids32, bounds32


def main() -> None:
    table: dict[str, dict[str, list[str]]] = {}
    for dim in HEAD_DIMS:
        for bits in INDEX_BITS:
            centroids, bounds = lloyd_max(dim, bits)
            table[f"d{dim}_m{bits}"] = {
                "centroids": [_f32_hex(v) for v in centroids],
                "boundaries": [_f32_hex(v) for v in bounds],
            }
    out = Path(__file__).with_name("tq_codebooks.json")
    out.write_text(json.dumps({"format": "float32 big-endian hex", "tables": table}, indent=1) + "\n")
    print(f"wrote {out} ({len(table)} tables)")


if __name__ == "__main__":
    main()
