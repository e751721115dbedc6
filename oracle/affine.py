"""Affine-quantised expert bank oracle (2-bit group 128 is the configured case).

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

The matmul itself lives in MLX (`mx.quantized_matmul`, mlx>=0.32.2 per the
reference's pyproject.toml:30; not vendored, not installable here), so output
bits of the reference are "parity unpinned".  What the reference pins and this
file follows:
  benchmarks/quant_affine.py:60-105    bit layout: level i of a row occupies bits
                                       [i*bits, (i+1)*bits) of a little-endian stream of u32 words
  benchmarks/quant_affine.py:113-123   value = scale*q + bias, nearest level, clamp to 0..2**bits-1
  benchmarks/quant_affine.py:321-324   scale and bias are rounded to the storage dtype before use
  tests/test_quant_affine.py:171-180   3-bit known answer (level 10 = 7 -> words C0000000, 1, 0)
  src/cachalot/model/expert_affine.py:65-81,117-152  rounding points of the expert:
       x -> bf16; gate, up -> bf16 -> f32; (silu(g)*u*w) -> bf16; each W2 h -> bf16 -> f32;
       experts summed in f32 in routing order
"""
from __future__ import annotations

from math import gcd

import numpy as np

from .bf16 import round_bf16
from .fp4 import swiglu


def pack_bits(levels: np.ndarray, bits: int) -> np.ndarray:
    """[..., n] integer levels -> [..., n*bits/32] uint32 (little-endian bit stream, unpadded)."""
    q = np.asarray(levels).astype(np.uint64)
    n = q.shape[-1]
    if (n * bits) % 32:
        raise ValueError(f"group {n} at {bits} bits is not a whole number of uint32 words")
    chunk = 32 // gcd(bits, 32)
    if n % chunk:
        raise ValueError(f"group {n} is not a multiple of {chunk} at {bits} bits")
    n_words = n * bits // 32
    out = np.zeros(q.shape[:-1] + (n_words,), dtype=np.uint64)
    for i in range(n):  # pure loop over positions; vectorised over rows
        word, shift = divmod(i * bits, 32)
        out[..., word] |= (q[..., i] << shift) & 0xFFFFFFFF
        if shift + bits > 32:
            out[..., word + 1] |= q[..., i] >> (32 - shift)
    return out.astype(np.uint32)


def unpack_bits(words: np.ndarray, bits: int, n: int) -> np.ndarray:
    """Inverse of pack_bits: [..., n*bits/32] uint32 -> [..., n] uint8 levels."""
    w = np.asarray(words, dtype=np.uint32).astype(np.uint64)
    if bits in (2, 4, 8):
        per = 32 // bits
        shifts = (np.arange(per, dtype=np.uint64) * bits)
        lv = (w[..., :, None] >> shifts) & ((1 << bits) - 1)
        return lv.reshape(w.shape[:-1] + (-1,))[..., :n].astype(np.uint8)
    out = np.zeros(w.shape[:-1] + (n,), dtype=np.uint8)
    mask = (1 << bits) - 1
    for i in range(n):
        word, shift = divmod(i * bits, 32)
        v = w[..., word] >> shift
        if shift + bits > 32:
            v = v | (w[..., word + 1] << (32 - shift))
        out[..., i] = (v & mask).astype(np.uint8)
    return out


def dequantize_affine(words, scales, biases, *, bits: int, group_size: int) -> np.ndarray:
    """words u32 [N, K*bits/32]; scales/biases (f16 or bf16 values held in any float array), one
    per `group_size` consecutive elements of the flattened [N*K] matrix -- shaped [N, K/group]
    when the group divides K (the reference's layout) or flat [N*K/group] otherwise
    -> f32 [N, K] = f32(scale)*q + f32(bias), one float32 rounding (the product is exact)."""
    w = np.asarray(words)
    n, k = w.shape[0], w.shape[1] * 32 // bits
    s = np.asarray(scales).astype(np.float32).reshape(-1)
    b = np.asarray(biases).astype(np.float32).reshape(-1)
    if (n * k) % group_size or s.size != n * k // group_size or b.size != s.size:
        raise ValueError(f"{s.size} scales for a {n}x{k} matrix at group {group_size}")
    q = unpack_bits(w, bits, k).astype(np.float32).reshape(-1, group_size)
    return (s[:, None] * q + b[:, None]).astype(np.float32).reshape(n, k)


def quantize_affine_minmax(w: np.ndarray, *, bits: int, group_size: int, store=np.float16):
    """Simple min/max affine fit used only to build test banks: scale and bias are rounded to
    the storage dtype first, then levels are chosen against the rounded values
    (quant_affine.py:321-327)."""
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    g = w.reshape(n, k // group_size, group_size)
    lo, hi = g.min(-1), g.max(-1)
    levels = (1 << bits) - 1
    scale = np.maximum((hi - lo) / levels, 1e-8).astype(store).astype(np.float32)
    bias = lo.astype(store).astype(np.float32)
    q = np.clip(np.rint((g - bias[..., None]) / scale[..., None]), 0, levels).astype(np.uint8)
    return pack_bits(q.reshape(n, k), bits), scale.astype(store), bias.astype(store)


def _qmm(x, mats, proj, bits, group_size, acc):
    w = dequantize_affine(mats[f"{proj}.weight"], mats[f"{proj}.scales"], mats[f"{proj}.biases"],
                          bits=bits, group_size=group_size)
    return (x.astype(acc) @ w.astype(acc).T).astype(np.float32)


def affine_expert_forward(x, mats, *, bits, group_size, weight, swiglu_limit=10.0, acc=np.float32):
    """x [H] or [M,H]; weight scalar or [M] -> f32, rounding points of expert_affine.py:74-81."""
    xb = round_bf16(np.atleast_2d(np.asarray(x, dtype=np.float32)))
    g = round_bf16(_qmm(xb, mats, "w1", bits, group_size, acc))
    u = round_bf16(_qmm(xb, mats, "w3", bits, group_size, acc))
    h = swiglu(g, u, swiglu_limit) * np.asarray(weight, dtype=np.float32).reshape(-1, 1)
    h = round_bf16(h.astype(np.float32))
    y = round_bf16(_qmm(h, mats, "w2", bits, group_size, acc))
    return y[0] if np.ndim(x) == 1 else y


def affine_routed_experts(x, experts, weights, *, bits, group_size, swiglu_limit=10.0, acc=np.float32):
    """routed = 0; routed += expert_i(x) in routing order, float32 (expert_affine.py:134-152)."""
    total = np.zeros(np.shape(x), dtype=np.float32)
    for mats, w in zip(experts, np.asarray(weights, dtype=np.float32).reshape(-1)):
        total = total + affine_expert_forward(x, mats, bits=bits, group_size=group_size, weight=w,
                                              swiglu_limit=swiglu_limit, acc=acc)
    return total


def affine_routed_experts_plain(x, experts, weights, *, bits, group_size, swiglu_limit=10.0):
    """The same experts without any of the bf16 rounding points, accumulated in float64: the bound for a kernel
    run with its rounding points switched off (x is still the bf16 input)."""
    xv = np.asarray(x, dtype=np.float64)
    total = np.zeros(xv.shape, dtype=np.float64)
    for mats, w in zip(experts, np.asarray(weights, dtype=np.float32).reshape(-1)):
        m = {p: dequantize_affine(mats[f"{p}.weight"], mats[f"{p}.scales"], mats[f"{p}.biases"], bits=bits,
                                  group_size=group_size).astype(np.float64) for p in ("w1", "w2", "w3")}
        g, u = m["w1"] @ xv, m["w3"] @ xv
        total += m["w2"] @ (swiglu(g, u, swiglu_limit) * float(w))
    return total
