"""bfloat16 / float16 rounding helpers for the CPU oracle (test infrastructure)."""
from __future__ import annotations

import numpy as np


def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest bfloat16 (ties to even) -> float32.  NaN/Inf pass through."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    bits = x.view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    out = rounded.view(np.float32).reshape(x.shape)
    return np.where(np.isfinite(x), out, x)


def bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> uint16 bfloat16 bit pattern (round to nearest even)."""
    return (round_bf16(x).view(np.uint32) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.asarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_f16(x: np.ndarray) -> np.ndarray:
    return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)
