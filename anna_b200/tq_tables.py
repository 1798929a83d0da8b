"""Constants of the TurboQuant key quantizer: sign vectors, Lloyd-Max codebooks, device-resident copies.

The reference builds one quantizer per ``(head_dim, bits, device)`` with ``seed=42`` and shares it between all
layers and heads (src/anna/model/turboquant.py:75-92); the same sharing rule applies here.  ``TurboQuantIP(bits=b)``
spends ``b - 1`` bits on the per-coordinate Lloyd-Max index and one bit on the QJL sign of the residual.
"""
from __future__ import annotations

import json
import math
import struct
import threading
from dataclasses import dataclass
from pathlib import Path

import torch

QUANTIZER_SEED = 42
_MASK64 = (1 << 64) - 1
_TABLE_PATH = Path(__file__).resolve().parent / "data" / "tq_codebooks.json"
_TABLES: dict[str, dict[str, list[str]]] | None = None
_LOCK = threading.Lock()


def sign_vector(dim: int, stream: int, seed: int = QUANTIZER_SEED) -> list[float]:
    """+1 / -1 per coordinate from a splitmix64 stream keyed by (seed, stream, dim)."""
    x = (seed ^ ((0xD1B54A32D192ED03 * (stream + 1)) & _MASK64) ^ ((dim * 0x9E3779B97F4A7C15) & _MASK64)) & _MASK64
    out: list[float] = []
    for _ in range(dim):
        x = (x + 0x9E3779B97F4A7C15) & _MASK64
        z = x
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK64
        z ^= z >> 31
        out.append(-1.0 if (z >> 63) else 1.0)
    return out


def codebook(dim: int, index_bits: int) -> tuple[list[float], list[float]]:
    """(centroids, boundaries) as Python floats that are exact float32 values."""
    global _TABLES
    if _TABLES is None:
        _TABLES = json.loads(_TABLE_PATH.read_text())["tables"]
    key = f"d{dim}_m{index_bits}"
    if key not in _TABLES:
        raise ValueError(f"no TurboQuant codebook for head_dim={dim}, index_bits={index_bits}")
    entry = _TABLES[key]

    def dec(items: list[str]) -> list[float]:
        return [struct.unpack(">f", bytes.fromhex(h))[0] for h in items]

    return dec(entry["centroids"]), dec(entry["boundaries"])


@dataclass(frozen=True)
class KeyQuantizerTables:
    head_dim: int
    bits: int
    index_bits: int
    signs1: torch.Tensor      # float32 [D]
    signs2: torch.Tensor      # float32 [D]
    centroids: torch.Tensor   # float32 [2^index_bits]
    boundaries: torch.Tensor  # float32 [2^index_bits - 1]

    @property
    def qjl_scale(self) -> float:
        return math.sqrt(math.pi / 2.0) / math.sqrt(self.head_dim)


_DEVICE_TABLES: dict[tuple[int, int, str, str], KeyQuantizerTables] = {}


def key_tables(*, head_dim: int, bits: int, device: torch.device | str, variant: str = "ip") -> KeyQuantizerTables:
    """Device-resident constants of the quantizer of (head_dim, bits): ``variant="ip"`` is the inner-product
    quantizer of KV rows (``bits - 1`` index bits + QJL sign), ``"mse"`` the plain one of tensor rows (``bits`` index
    bits, src/anna/model/turboquant.py:75-82)."""
    if variant not in ("ip", "mse"):
        raise ValueError(f"unknown TurboQuant variant {variant!r}")
    device = torch.device(device)
    key = (int(head_dim), int(bits), str(device), variant)
    tables = _DEVICE_TABLES.get(key)
    if tables is not None:
        return tables
    with _LOCK:
        tables = _DEVICE_TABLES.get(key)
        if tables is None:
            index_bits = int(bits) - (1 if variant == "ip" else 0)
            cent, bnd = codebook(int(head_dim), index_bits)
            tables = KeyQuantizerTables(
                head_dim=int(head_dim),
                bits=int(bits),
                index_bits=index_bits,
                signs1=torch.tensor(sign_vector(int(head_dim), 0), dtype=torch.float32, device=device),
                signs2=torch.tensor(sign_vector(int(head_dim), 1), dtype=torch.float32, device=device),
                centroids=torch.tensor(cent, dtype=torch.float32, device=device),
                boundaries=torch.tensor(bnd, dtype=torch.float32, device=device),
            )
            _DEVICE_TABLES[key] = tables
    return tables
