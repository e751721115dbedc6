"""MXFP4 activation quantisation oracle (E2M1 codes, one E8M0 scale per 32 along K).

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  The reference has this only in MLX
(src/cachalot/model/fp4_act_mlx.py), so it is a restatement ("parity unpinned" beyond the
rounding table): :12-16 amax floor 6*2**-126; :175-190 scale = 2**ceil(log2(amax/6));
:233-237 clip(x/scale, +-6); :19-98 nearest E2M1 with ties to even
(0.25->0, 0.75->1, 1.25->1, 1.75->2, 2.5->2, 3.5->4, 5->4), sign of zero kept.
"""
from __future__ import annotations

import numpy as np

from .fp4 import E2M1_VALUES

FP4_MAX = 6.0
MIN_AMAX = FP4_MAX * 2.0 ** -126


def round_e2m1_codes(v: np.ndarray) -> np.ndarray:
    """float32 in [-6, 6] -> E2M1 code 0..15 (bit 3 = sign), ties to even."""
    v = np.asarray(v, dtype=np.float32)
    a = np.abs(v)
    mag = np.select(
        [a <= 0.25, a < 0.75, a <= 1.25, a < 1.75, a <= 2.5, a < 3.5, a <= 5.0],
        [0, 1, 2, 3, 4, 5, 6],
        default=7,
    ).astype(np.uint8)
    return (mag | (np.signbit(v).astype(np.uint8) << 3)).astype(np.uint8)


def quantize_mxfp4(x: np.ndarray, block_size: int = 32):
    """x [..., K] -> (codes u8 [..., K] in 0..15, scale bytes u8 [..., K/block] raw E8M0)."""
    x = np.asarray(x, dtype=np.float32)
    k = x.shape[-1]
    if k % block_size:
        raise ValueError(f"last dimension {k} must be divisible by block_size={block_size}")
    blocks = x.reshape(x.shape[:-1] + (k // block_size, block_size))
    amax = np.maximum(np.max(np.abs(blocks), axis=-1), np.float32(MIN_AMAX)).astype(np.float32)
    exponent = np.ceil(np.log2((amax / np.float32(FP4_MAX)).astype(np.float32))).astype(np.int32)
    scale = np.exp2(exponent.astype(np.float64)).astype(np.float32)
    norm = np.clip((blocks / scale[..., None]).astype(np.float32), -FP4_MAX, FP4_MAX)
    codes = round_e2m1_codes(norm).reshape(x.shape)
    return codes, (exponent + 127).astype(np.uint8)


def dequantize_mxfp4(codes: np.ndarray, scale_bytes: np.ndarray, block_size: int = 32) -> np.ndarray:
    c = np.asarray(codes, dtype=np.uint8)
    s = np.exp2(np.asarray(scale_bytes, dtype=np.uint8).astype(np.float64) - 127).astype(np.float32)
    v = E2M1_VALUES[c].reshape(c.shape[:-1] + (-1, block_size))
    return (v * s[..., None]).reshape(c.shape).astype(np.float32)


def roundtrip(x: np.ndarray, block_size: int = 32) -> np.ndarray:
    codes, sb = quantize_mxfp4(x, block_size)
    return dequantize_mxfp4(codes, sb, block_size)
