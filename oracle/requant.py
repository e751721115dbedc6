"""FP4 -> affine re-quantiser oracle: the fit that builds a 2-bit (or wider) affine bank from dense weights.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  Restatement in numpy ("parity unpinned": the reference runs it
through MLX) of
  benchmarks/quant_affine.py:113-123   nearest level, clamped; squared reconstruction error per group
  benchmarks/quant_affine.py:138-149   min/max fit: scale = max((hi - lo) / levels, 1e-8), bias = lo
  benchmarks/quant_affine.py:155-193   grid search over shrunk ranges (5 x 5), lowest error wins, ties keep the earlier
  benchmarks/quant_affine.py:213-251   least-squares refinement: assign levels, refit the line (closed form), scale and
                                       bias rounded to the storage dtype on every iteration, best iterate kept
  benchmarks/quant_affine.py:303-329   quantize_affine: levels against the rounded scale and bias; packed words
"""
from __future__ import annotations

import numpy as np

from .affine import pack_bits
from .bf16 import round_bf16

SHRINKS = (1.0, 0.925, 0.85, 0.775, 0.7)


def _store(v, store):
    return round_bf16(v.astype(np.float32)) if store == "bfloat16" else v.astype(np.float16).astype(np.float32)


def _quantize(w, scale, bias, levels):
    # a constant group whose 1e-8 scale rounds to 0 in f16 gives 0/0: level 0, as fmaxf(NaN, 0) gives on the GPU
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.rint((w - bias) / scale)
    return np.clip(np.nan_to_num(q, nan=0.0), 0, levels).astype(np.float32)


def _error(w, scale, bias, levels):
    q = _quantize(w, scale, bias, levels)
    return np.sum((scale * q + bias - w) ** 2, axis=-1, dtype=np.float32)


def fit_search(groups, bits=2, shrinks=SHRINKS):
    g = groups.astype(np.float32)
    levels = np.float32((1 << bits) - 1)
    lo, hi = g.min(-1, keepdims=True), g.max(-1, keepdims=True)
    mid = (lo + hi) / np.float32(2)
    best_s = np.maximum((hi - lo) / levels, np.float32(1e-8))
    best_b = lo.copy()
    best = _error(g, best_s, best_b, levels)
    for s_lo in shrinks:
        for s_hi in shrinks:
            if s_lo == 1.0 and s_hi == 1.0:
                continue
            new_lo = (mid + (lo - mid) * np.float32(s_lo)).astype(np.float32)
            new_hi = (mid + (hi - mid) * np.float32(s_hi)).astype(np.float32)
            scale = np.maximum((new_hi - new_lo) / levels, np.float32(1e-8))
            err = _error(g, scale, new_lo, levels)
            take = (err < best)[:, None]
            best_s, best_b = np.where(take, scale, best_s), np.where(take, new_lo, best_b)
            best = np.minimum(err, best)
    return best_s.astype(np.float32), best_b.astype(np.float32)


def refine_lsq(groups, scale, bias, bits=2, iters=4, store="float16"):
    g = groups.astype(np.float32)
    levels = np.float32((1 << bits) - 1)
    scale, bias = _store(scale, store), _store(bias, store)
    best_s, best_b = scale, bias
    best = _error(g, scale, bias, levels)
    n = np.float32(g.shape[-1])
    for _ in range(iters):
        q = _quantize(g, scale, bias, levels)
        sq, sqq = q.sum(-1, keepdims=True, dtype=np.float32), (q * q).sum(-1, keepdims=True, dtype=np.float32)
        sw, sqw = g.sum(-1, keepdims=True, dtype=np.float32), (q * g).sum(-1, keepdims=True, dtype=np.float32)
        den = n * sqq - sq * sq
        new_s = (n * sqw - sq * sw) / np.where(np.abs(den) < 1e-12, np.float32(1), den)
        new_b = (sw - new_s * sq) / n
        new_s, new_b = _store(new_s, store), _store(new_b, store)
        keep = (np.abs(den) < 1e-12) | (new_s <= 0)
        scale, bias = np.where(keep, scale, new_s), np.where(keep, bias, new_b)
        err = _error(g, scale, bias, levels)
        take = (err < best)[:, None]
        best_s, best_b = np.where(take, scale, best_s), np.where(take, bias, best_b)
        best = np.minimum(err, best)
    return best_s.astype(np.float32), best_b.astype(np.float32)


def quantize_affine(w, group_size=128, bits=2, store="float16", lsq=True):
    """w f32 [N, K] -> (words u32 [N, K*bits/32], scales, biases [N*K/group] in the storage dtype's values as f32,
    levels u8 [N, K]).  Groups run over the flattened matrix."""
    w = np.asarray(w, dtype=np.float32)
    n, k = w.shape
    g = w.reshape(-1, group_size)
    scale, bias = fit_search(g, bits)
    if lsq:
        scale, bias = refine_lsq(g, scale, bias, bits, store=store)
    scale, bias = _store(scale, store), _store(bias, store)
    q = _quantize(g, scale, bias, np.float32((1 << bits) - 1)).astype(np.uint8).reshape(n, k)
    return pack_bits(q, bits), scale.reshape(-1), bias.reshape(-1), q
