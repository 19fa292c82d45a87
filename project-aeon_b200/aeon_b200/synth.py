"""Host side of the synthetic-tensor generators: quantile tables and seeded small tensors.

The device fill kernels (aeon_b200_synth_fill_*) draw 16-bit values from a table of
quantiles, so the distribution is whatever the table encodes. The tables are computed here
in double precision with the standard library's inverse normal CDF, which is deterministic,
and uploaded once.
"""
from __future__ import annotations

from statistics import NormalDist

import numpy as np


def to_bits16(values, dtype: int) -> np.ndarray:
    """float64 array -> fp16 (dtype 0) or bf16 (dtype 1) bit patterns, round-to-nearest-even."""
    values = np.asarray(values, dtype=np.float64)
    if dtype == 0:
        return values.astype(np.float16).view(np.uint16)
    f = values.astype(np.float32).view(np.uint32)
    rounded = f + 0x7FFF + ((f >> 16) & 1)
    return (rounded >> 16).astype(np.uint16)


def from_bits16(bits, dtype: int) -> np.ndarray:
    bits = np.asarray(bits, dtype=np.uint16)
    if dtype == 0:
        return bits.view(np.float16).astype(np.float64)
    return (bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def half_normal_table(sigma: float, eps: float = 0.0, n: int = 4096, dtype: int = 0) -> np.ndarray:
    """Quantiles of |N(0, sigma)| + eps at (i + 0.5) / n, as 16-bit patterns."""
    nd = NormalDist()
    q = np.array([nd.inv_cdf(0.5 + 0.5 * (i + 0.5) / n) for i in range(n)], dtype=np.float64)
    return to_bits16(q * sigma + eps, dtype)


def normal_bits(rng: np.random.Generator, shape, sigma: float, dtype: int) -> np.ndarray:
    """Seeded N(0, sigma) tensor rounded to the 16-bit dtype (small tensors: activations, gate)."""
    return to_bits16(rng.standard_normal(shape) * sigma, dtype)
