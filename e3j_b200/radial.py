"""Radial basis, cutoff envelope and radial MLP feeding ``edge_scalars``.

These producers are not part of the reference tree (they live in downstream
model code); only the layout of their output is pinned there: a flat
``(E, S * C)`` matrix reshaped to ``(E, S, C)``, scalar-major / channel-minor
(tests/test_pallas_mosaic_tpu_convolution.py:858).  The definitions below are
the standard ones and are used identically by the GPU path and by the test
oracle:

  * Bessel basis  b_n(r) = sqrt(2 / r_c) sin(n pi r / r_c) / r,  n = 1..num_basis
  * polynomial envelope of order p (default 5)
        f(u) = 1 - (p+1)(p+2)/2 u^p + p(p+2) u^(p+1) - p(p+1)/2 u^(p+2),  u = r / r_c < 1
  * two-layer MLP with e3nn-style parametrisation: weights ~ N(0, 1), each
    layer divided by sqrt(fan_in), SiLU rescaled to unit second moment.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

# 1 / sqrt(E[silu(z)^2]) for z ~ N(0, 1)
SILU_2MOM = 1.6790176

def bessel_envelope_np(r: np.ndarray, r_cut: float, num_basis: int = 8, p: int = 5) -> np.ndarray:
    r = np.asarray(r, dtype=np.float64)
    n = np.arange(1, num_basis + 1, dtype=np.float64)
    b = math.sqrt(2.0 / r_cut) * np.sin(n[None, :] * math.pi * r[:, None] / r_cut) / r[:, None]
    u = r / r_cut
    f = 1 - (p + 1) * (p + 2) / 2 * u**p + p * (p + 2) * u ** (p + 1) - p * (p + 1) / 2 * u ** (p + 2)
    f = np.where(u < 1, f, 0.0)
    return b * f[:, None]


def bessel_envelope(r: torch.Tensor, r_cut: float, num_basis: int = 8, p: int = 5) -> torch.Tensor:
    n = torch.arange(1, num_basis + 1, dtype=r.dtype, device=r.device)
    b = math.sqrt(2.0 / r_cut) * torch.sin(n[None, :] * (math.pi / r_cut) * r[:, None]) / r[:, None]
    u = r / r_cut
    f = 1 - (p + 1) * (p + 2) / 2 * u**p + p * (p + 2) * u ** (p + 1) - p * (p + 1) / 2 * u ** (p + 2)
    f = torch.where(u < 1, f, torch.zeros_like(f))
    return b * f[:, None]


@dataclass
class RadialMLP:
    """``rbf (E, B) -> silu -> (E, S * C)``; weights are plain arrays."""

    w1: np.ndarray  # (B, H)
    w2: np.ndarray  # (H, S * C)

    @classmethod
    def init(cls, num_basis: int, hidden: int, num_out: int, seed: int = 0) -> "RadialMLP":
        rng = np.random.default_rng(seed)
        return cls(
            rng.standard_normal((num_basis, hidden)).astype(np.float32),
            rng.standard_normal((hidden, num_out)).astype(np.float32),
        )

    def forward_np(self, rbf: np.ndarray, dtype=np.float64) -> np.ndarray:
        h = rbf.astype(dtype) @ self.w1.astype(dtype) / math.sqrt(self.w1.shape[0])
        h = SILU_2MOM * h / (1 + np.exp(-h))
        return h @ self.w2.astype(dtype) / math.sqrt(self.w2.shape[0])

    def forward(self, rbf: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
        h = rbf @ w1 / math.sqrt(w1.shape[0])
        h = SILU_2MOM * torch.nn.functional.silu(h)
        return h @ w2 / math.sqrt(w2.shape[0])
