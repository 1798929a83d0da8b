"""Stand-in for the un-vendored ``turboquant.core`` module (PyPI ``turboquant`` >=0.2,<0.3).  Test infrastructure.

The reference imports ``TurboQuantMSE`` / ``TurboQuantIP`` from that package (src/anna/model/turboquant.py:45,
:57) and only uses this surface:

* ``TurboQuantMSE(dim=, bits=, device=, seed=42)`` (:80) with ``quantize(flat[N, D]) -> (indices, norms)`` (:393)
  and ``dequantize(indices[N, D], norms[N, 1]) -> [N, D]`` (:415-418);
* ``TurboQuantIP(dim=, bits=, device=, seed=42)`` (:90) with ``quantize(flat[N, D]) -> (mse_indices, norms,
  qjl_signs, residual_norms)`` (:265), ``dequantize(mse_indices, norms, qjl_signs, residual_norms)`` on
  ``[H, T, D]`` / ``[H, T, 1]`` shapes (:284, :320) and the attribute ``S`` ``[D, D]`` (:324).

``install()`` registers classes with exactly that surface, backed by the CPU oracle, so that the reference's own
``TurboQuantKVRow`` / ``Qwen3DynamicCache`` can be imported and run on CPU to produce golden fixtures.  The
arithmetic is this build's definition (oracle/tq_oracle.c), not the real package's: key-code parity is unpinned.
"""
from __future__ import annotations

import sys
import types

import numpy as np
import torch

import oracle


class TurboQuantMSE:
    variant = "mse"

    def __init__(self, dim: int, bits: int, device: str = "cpu", seed: int = 42) -> None:
        if int(seed) != oracle.QUANTIZER_SEED:
            raise ValueError("the oracle freezes the quantizer seed at 42")
        self.dim = int(dim)
        self.bits = int(bits)
        self.device = torch.device(device)

    def quantize(self, flat: torch.Tensor):
        idx, _, norms, _ = oracle.quantize_keys(flat.detach().float().cpu().numpy(), self.bits, "mse")
        return (torch.from_numpy(idx.reshape(-1)).to(self.device),
                torch.from_numpy(norms.reshape(-1)).to(self.device))

    def dequantize(self, indices: torch.Tensor, norms: torch.Tensor) -> torch.Tensor:
        idx = indices.detach().cpu().numpy().astype(np.uint8).reshape(-1, self.dim)
        out = oracle.dequantize_keys(idx, None, norms.detach().float().cpu().numpy().reshape(-1), None, self.bits,
                                     "mse")
        return torch.from_numpy(out).reshape(*indices.shape[:-1], self.dim).to(self.device)


class TurboQuantIP:
    variant = "ip"

    def __init__(self, dim: int, bits: int, device: str = "cpu", seed: int = 42) -> None:
        if int(seed) != oracle.QUANTIZER_SEED:
            raise ValueError("the oracle freezes the quantizer seed at 42")
        self.dim = int(dim)
        self.bits = int(bits)
        self.device = torch.device(device)
        self.S = torch.from_numpy(oracle.qjl_matrix(self.dim)).to(self.device)

    def quantize(self, flat: torch.Tensor):
        idx, sign, norms, rnorms = oracle.quantize_keys(flat.detach().float().cpu().numpy(), self.bits, "ip")
        return (torch.from_numpy(idx).to(self.device), torch.from_numpy(norms).to(self.device),
                torch.from_numpy(sign).to(self.device), torch.from_numpy(rnorms).to(self.device))

    def dequantize(self, mse_indices, norms, qjl_signs, residual_norms) -> torch.Tensor:
        shape = tuple(mse_indices.shape)
        idx = mse_indices.detach().cpu().numpy().astype(np.uint8).reshape(-1, self.dim)
        sign = qjl_signs.detach().cpu().numpy().astype(np.uint8).reshape(-1, self.dim)
        rn = residual_norms.detach().float().cpu().numpy().reshape(-1)
        # turboquant.py:318-320 asks for the index-only reconstruction by zeroing signs and residual norms: a zero
        # residual norm removes the sign term whatever the signs are, so no case analysis on the values is needed
        # (tests/test_quantizer_properties.py checks that both forms agree bit for bit)
        out = oracle.dequantize_keys(idx, sign, norms.detach().float().cpu().numpy().reshape(-1), rn, self.bits, "ip")
        return torch.from_numpy(out).reshape(shape).to(self.device)


def install() -> None:
    """Register ``turboquant`` / ``turboquant.core`` in ``sys.modules`` (idempotent)."""
    if "turboquant.core" in sys.modules and getattr(sys.modules["turboquant.core"], "_anna_b200_shim", False):
        return
    package = types.ModuleType("turboquant")
    core = types.ModuleType("turboquant.core")
    core.TurboQuantMSE = TurboQuantMSE
    core.TurboQuantIP = TurboQuantIP
    core._anna_b200_shim = True
    package.core = core
    sys.modules["turboquant"] = package
    sys.modules["turboquant.core"] = core
