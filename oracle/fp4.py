"""FP4 (E2M1 codes, E8M0 per-32 scales) oracle: dequant and the routed-expert FFN.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Follows the reference's
  src/cachalot/model/fp4.py:5-109          table, E8M0 decode, nibble order, dequant
  src/cachalot/model/expert_metal.py:9-64  one expert: clamp, SwiGLU, router weight before w2
  src/cachalot/model/moe_metal.py:8-37     top-k = sum of the experts' outputs
  src/cachalot/model/moe_fused_metal.py:101-136,154-179  fused form, experts summed in order
"""
from __future__ import annotations

import numpy as np

# code -> value; bit 3 is the sign, code 8 is (negative) zero and decodes to 0.0
E2M1_VALUES = np.array(
    [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, 0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0],
    dtype=np.float32,
)
BLOCK = 32


def e8m0_to_f32(raw: np.ndarray) -> np.ndarray:
    """raw byte r -> 2**(r-127) as float32; no special case for 0 or 255 (fp4.py:28-41)."""
    r = np.asarray(raw, dtype=np.uint8).astype(np.int32) - 127
    return np.exp2(r.astype(np.float64)).astype(np.float32)


def unpack_codes(packed: np.ndarray) -> np.ndarray:
    """[..., K/2] bytes -> [..., K] codes 0..15; the low nibble is the even element (fp4.py:44-64)."""
    p = np.asarray(packed, dtype=np.uint8)
    codes = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.uint8)
    codes[..., 0::2] = p & 0x0F
    codes[..., 1::2] = p >> 4
    return codes


def pack_codes(codes: np.ndarray) -> np.ndarray:
    c = np.asarray(codes, dtype=np.uint8)
    return (c[..., 0::2] | (c[..., 1::2] << 4)).astype(np.uint8)


def dequantize_fp4_weight(packed: np.ndarray, scales: np.ndarray, block_size: int = BLOCK) -> np.ndarray:
    """packed u8 [N, K/2], scales u8 [N, K/block] -> f32 [N, K] = table[code] * 2**(scale-127)."""
    vals = E2M1_VALUES[unpack_codes(packed)]
    n, k = vals.shape
    if k % block_size:
        raise ValueError(f"K={k} must be divisible by block_size={block_size}")
    if tuple(scales.shape) != (n, k // block_size):
        raise ValueError(f"Scale shape {tuple(scales.shape)} does not match expected {(n, k // block_size)}")
    s = e8m0_to_f32(scales)
    return (vals.reshape(n, k // block_size, block_size) * s[:, :, None]).reshape(n, k)


def silu(g: np.ndarray) -> np.ndarray:
    """g / (1 + exp(-g)) in float32 (moe_fused_metal.py:133)."""
    g = np.asarray(g, dtype=np.float32)
    with np.errstate(over="ignore"):
        return (g / (np.float32(1.0) + np.exp(-g))).astype(np.float32)


def swiglu(gate: np.ndarray, up: np.ndarray, limit: float) -> np.ndarray:
    """up clamped both sides, gate clamped from above only, when limit > 0 (expert_metal.py:37-52)."""
    gate = np.asarray(gate, dtype=np.float32)
    up = np.asarray(up, dtype=np.float32)
    if limit > 0:
        up = np.clip(up, -np.float32(limit), np.float32(limit))
        gate = np.minimum(gate, np.float32(limit))
    return silu(gate) * up


def expert_forward(x, w1, s1, w2, s2, w3, s3, *, weight=None, swiglu_limit=10.0, acc=np.float32):
    """One routed expert on x [H] or [M, H] -> f32 [H] / [M, H].

    weight (scalar or [M]) multiplies the hidden activation BEFORE the down
    projection (expert_metal.py:54-56).  No bf16 rounding anywhere on this path.
    """
    xf = np.atleast_2d(np.asarray(x, dtype=np.float32)).astype(acc)
    g = (xf @ dequantize_fp4_weight(w1, s1).astype(acc).T).astype(np.float32)
    u = (xf @ dequantize_fp4_weight(w3, s3).astype(acc).T).astype(np.float32)
    h = swiglu(g, u, swiglu_limit)
    if weight is not None:
        h = h * np.asarray(weight, dtype=np.float32).reshape(-1, 1)
    y = (h.astype(acc) @ dequantize_fp4_weight(w2, s2).astype(acc).T).astype(np.float32)
    return y[0] if np.ndim(x) == 1 else y


def routed_topk_forward(x, experts, weights, *, swiglu_limit=10.0, acc=np.float32):
    """Sum over the routed experts, accumulated in routing order (moe_fused_metal.py:162-175).

    experts: sequence of dicts with w1.weight/w1.scale/w2.../w3... byte arrays
    already shaped [N, K/2] and [N, K/32].
    """
    if len(experts) != np.size(weights):
        raise ValueError(f"{len(experts)=} does not match {np.size(weights)=}")
    total = None
    for e, w in zip(experts, np.asarray(weights, dtype=np.float32).reshape(-1)):
        y = expert_forward(
            x, e["w1.weight"], e["w1.scale"], e["w2.weight"], e["w2.scale"], e["w3.weight"], e["w3.scale"],
            weight=w, swiglu_limit=swiglu_limit, acc=acc,
        )
        total = y if total is None else total + y
    return total


def fp4_to_affine8(packed: np.ndarray, scales: np.ndarray):
    """Exact 8-bit affine restatement of an FP4 matrix (fp4_affine8_metal.py:5-15):
    q = 2*v/1 + 12 in 0..24, scale = 0.5 * 2**e, bias = -6 * 2**e, so scale*q + bias == v * 2**e."""
    v = E2M1_VALUES[unpack_codes(packed)]
    q = (2.0 * v + 12.0).astype(np.uint8)
    s = e8m0_to_f32(scales)
    return q, (0.5 * s).astype(np.float32), (-6.0 * s).astype(np.float32)
