"""bf16-weight GEMV oracle.  TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Restatement of model/bf16_gemv_metal.py:20-63 (the reference's kernel is Metal: "parity unpinned" for the order of
the fp32 additions): out[n] = sum_k f32(w[n, k]) * f32(x[k]).  The widening of a bf16 weight is exact, every product
of a bf16 weight and an fp32 activation is formed in at least fp32, and the sum is taken in float64 here, so a kernel
that accumulates in fp32 in any order must agree to a few ulp of the row's sum of magnitudes.
"""
from __future__ import annotations

import numpy as np


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bf16 bit patterns -> float32 (a shift)."""
    return (np.asarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def bf16_gemv_f32(x: np.ndarray, weight_bits: np.ndarray) -> np.ndarray:
    """x f32 [K] or [rows, K]; weight_bits u16 [N, K] -> float32 [N] or [rows, N] (float64 accumulation)."""
    w = bf16_to_f32(weight_bits).astype(np.float64)
    return (np.asarray(x, dtype=np.float32).astype(np.float64) @ w.T).astype(np.float32)


def bf16_gemv_bound(x: np.ndarray, weight_bits: np.ndarray) -> np.ndarray:
    """Per output, what fp32 accumulation in any order may differ by: K * 2**-24 * sum_k |w x| (generous)."""
    w = np.abs(bf16_to_f32(weight_bits).astype(np.float64))
    k = w.shape[1]
    return (np.abs(np.asarray(x, dtype=np.float64)) @ w.T) * k * 2.0 ** -24
