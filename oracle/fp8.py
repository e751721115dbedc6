"""FP8 E4M3 trunk GEMV + act_quant oracle.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Follows the reference's
  src/cachalot/model/fp8_ref.py:27-92     act_quant: amax floor 1e-4, scale = 2**ceil(log2(amax/448)),
                                          clip to +-448, E4M3FN round-to-nearest-even
  src/cachalot/model/fp8_ref.py:95-231    GEMV: per K-block partial dot, times act scale, times weight
                                          scale[row // block, kblock]; fp32
  src/cachalot/model/fp8_fused_metal.py:33-74   in-kernel E4M3 encode / decode
  src/cachalot/model/fp8_gemv_metal.py:121-154  256-entry decode table; codes 0x7F / 0xFF decode to 0.0
  src/cachalot/model/wo_a_dequant.py:60-63      128x128 weight blocks as a legal block shape
Two scale rules: "e8m0" (reference: power-of-two act scale, E8M0 weight scale bytes, block 32) and
"f32" (configured variant: act scale = max(amax,1e-4)/448 kept in fp32, fp32 weight scales, block 128).
"""
from __future__ import annotations

import numpy as np

FP8_MAX = 448.0
MIN_AMAX = 1e-4


def _build_decode_table() -> np.ndarray:
    t = np.zeros(256, dtype=np.float32)
    for b in range(256):
        e, m = (b >> 3) & 0xF, b & 7
        if e == 0xF and m == 7:
            v = 0.0  # the two NaN codes are read as zero by the reference's kernels
        elif e == 0:
            v = m * 2.0 ** -9
        else:
            v = (1.0 + m / 8.0) * 2.0 ** (e - 7)
        t[b] = -v if b & 0x80 else v
    return t


E4M3_DECODE = _build_decode_table()


def e4m3_encode(x: np.ndarray) -> np.ndarray:
    """float32 (already clipped to +-448) -> E4M3FN byte, round to nearest even, signed zero kept."""
    x = np.asarray(x, dtype=np.float32)
    a = np.abs(x).astype(np.float64)
    sign = (np.signbit(x).astype(np.uint8) << 7)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.maximum(e, -6.0)
    quantum = np.exp2(e - 3.0)
    v = np.rint(a / quantum) * quantum  # np.rint rounds half to even
    v = np.minimum(v, FP8_MAX)
    ve = np.floor(np.log2(np.where(v > 0, v, 1.0)))
    sub = v < 2.0 ** -6
    ebits = np.where(sub, 0, ve + 7).astype(np.int64)
    mant = np.where(sub, np.rint(v * 512.0), np.rint((v / np.exp2(ve) - 1.0) * 8.0)).astype(np.int64)
    code = ((ebits << 3) | mant).astype(np.uint8)
    return np.where(a == 0, sign, sign | code).astype(np.uint8)


def quantize_activation_fp8(x, block_size: int = 32, scale_rule: str = "e8m0"):
    """x [K] or [B,K] -> (codes u8 same shape, scales f32 [..., K/block])."""
    x = np.asarray(x, dtype=np.float32)
    k = x.shape[-1]
    if k % block_size:
        raise ValueError(f"K={k} must be divisible by block_size={block_size}")
    blocks = x.reshape(x.shape[:-1] + (k // block_size, block_size))
    amax = np.maximum(np.max(np.abs(blocks), axis=-1), np.float32(MIN_AMAX)).astype(np.float32)
    raw = (amax / np.float32(FP8_MAX)).astype(np.float32)
    if scale_rule == "e8m0":
        scales = np.exp2(np.ceil(np.log2(raw))).astype(np.float32)
    elif scale_rule == "f32":
        scales = raw
    else:
        raise ValueError(f"unknown scale_rule {scale_rule!r}")
    norm = np.clip((blocks / scales[..., None]).astype(np.float32), -FP8_MAX, FP8_MAX)
    return e4m3_encode(norm).reshape(x.shape), scales


def decode_weight_scales(scale_raw, scale_rule: str) -> np.ndarray:
    if scale_rule == "e8m0":
        r = np.asarray(scale_raw, dtype=np.uint8).astype(np.int32) - 127
        return np.exp2(r.astype(np.float64)).astype(np.float32)
    return np.asarray(scale_raw, dtype=np.float32)


def fp8_gemv_quantized(codes, act_scales, weight_raw, scale_raw, *, block_size=32, scale_rule="e8m0"):
    """y[n] = sum_kb (sum_{j in kb} a_j w_nj) * act_scale[kb] * wscale[n // block, kb]; f32 [N] or [B,N]."""
    w = E4M3_DECODE[np.asarray(weight_raw, dtype=np.uint8)]
    n, k = w.shape
    nkb = k // block_size
    ws = decode_weight_scales(scale_raw, scale_rule)
    if ws.shape != (-(-n // block_size), nkb):
        raise ValueError(f"scale shape {ws.shape} != {(-(-n // block_size), nkb)}")
    a = E4M3_DECODE[np.asarray(codes, dtype=np.uint8)]
    single = a.ndim == 1
    a = np.atleast_2d(a).reshape(-1, nkb, block_size)
    s = np.atleast_2d(np.asarray(act_scales, dtype=np.float32))
    row_scale = ws[np.arange(n) // block_size]                      # [N, nkb]
    out = np.zeros((a.shape[0], n), dtype=np.float32)
    wb = w.reshape(n, nkb, block_size)
    for kb in range(nkb):
        partial = (a[:, kb, :] @ wb[:, kb, :].T).astype(np.float32)  # [B, N]
        out += partial * s[:, kb:kb + 1] * row_scale[None, :, kb]
    return out[0] if single else out


def fp8_linear(x, weight_raw, scale_raw, *, block_size=32, scale_rule="e8m0"):
    """act_quant then GEMV; float32 (the shipped op rounds this to bf16 afterwards)."""
    x = np.asarray(x, dtype=np.float32)
    if x.shape[-1] != np.shape(weight_raw)[1]:
        raise ValueError(f"x shape {x.shape} != ({np.shape(weight_raw)[1]},)")
    codes, scales = quantize_activation_fp8(x, block_size, scale_rule)
    return fp8_gemv_quantized(codes, scales, weight_raw, scale_raw, block_size=block_size, scale_rule=scale_rule)
