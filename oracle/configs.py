"""Seeded synthetic inputs with the shapes and value distributions of the five benchmark
configurations (sizes are parameters so tests can use small ones).

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  One numpy Generator per call,
`default_rng(seed)`, tensors drawn in the fixed order written in each function.
"""
from __future__ import annotations

import numpy as np

from .affine import pack_bits
from .bf16 import round_bf16


def fp4_matrix(rng, n, k, scale_lo=118, scale_hi=123):
    """codes uniform 0..15 packed two per byte along K (low nibble first); E8M0 bytes uniform in
    [scale_lo, scale_hi] = 2**-9 .. 2**-4 by default."""
    packed = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    scales = rng.integers(scale_lo, scale_hi + 1, (n, k // 32), dtype=np.uint8)
    return packed, scales


def fp4_expert(rng, hidden, inter):
    w1, s1 = fp4_matrix(rng, inter, hidden)
    w3, s3 = fp4_matrix(rng, inter, hidden)
    w2, s2 = fp4_matrix(rng, hidden, inter)
    return {"w1.weight": w1, "w1.scale": s1, "w2.weight": w2, "w2.scale": s2, "w3.weight": w3, "w3.scale": s3}


def config0(seed=0, hidden=4096, inter=2880):
    """Single FP4 expert, x bf16 [1,H] ~ N(0,1); no clamp, no router weight."""
    rng = np.random.default_rng(seed)
    x = round_bf16(rng.standard_normal((1, hidden)).astype(np.float32))
    return x, fp4_expert(rng, hidden, inter)


def affine_matrix(rng, n, k, bits=2, group=128):
    """codes uniform, fp16 scale ~U(0.002,0.02) and bias ~N(0,0.01) per `group` consecutive
    elements of the flattened matrix ([N, K/group] when the group divides K, else flat)."""
    levels = rng.integers(0, 1 << bits, (n, k), dtype=np.uint8)
    shape = (n, k // group) if k % group == 0 else (n * k // group,)
    scales = rng.uniform(0.002, 0.02, shape).astype(np.float16)
    biases = (rng.standard_normal(shape) * 0.01).astype(np.float16)
    return pack_bits(levels, bits), scales, biases


def affine_expert(rng, hidden, inter, bits=2, group=128):
    out = {}
    for proj, (n, k) in (("w1", (inter, hidden)), ("w2", (hidden, inter)), ("w3", (inter, hidden))):
        w, s, b = affine_matrix(rng, n, k, bits, group)
        out[f"{proj}.weight"], out[f"{proj}.scales"], out[f"{proj}.biases"] = w, s, b
    return out


def config1(seed=0, hidden=4096, inter=2880, n_experts=384, batch=1, materialise=None):
    """Decode layer over a 2-bit g128 bank: logits f32 [B,E] ~ N(0,1), x bf16 [B,H] ~ N(0,1).
    Only the experts in `materialise` (default: all) are generated, each from its own
    generator seeded (seed, expert) so any subset reproduces the same bytes."""
    rng = np.random.default_rng(seed)
    x = round_bf16(rng.standard_normal((batch, hidden)).astype(np.float32))
    logits = rng.standard_normal((batch, n_experts)).astype(np.float32)
    ids = range(n_experts) if materialise is None else materialise
    experts = {int(e): affine_expert(np.random.default_rng([seed, int(e)]), hidden, inter) for e in ids}
    return x, logits, experts


def config2(seed=0, hidden=4096, inter=2880, n_experts=384, layers=40, batch=1, materialise=None):
    """Decode over an FP4 bank: logits f32 [layers,B,E] ~ N(0,1) independent per token and layer."""
    rng = np.random.default_rng(seed)
    x = round_bf16(rng.standard_normal((batch, hidden)).astype(np.float32))
    logits = rng.standard_normal((layers, batch, n_experts)).astype(np.float32)
    ids = [(l, e) for l in range(layers) for e in range(n_experts)] if materialise is None else materialise
    experts = {(int(l), int(e)): fp4_expert(np.random.default_rng([seed, int(l), int(e)]), hidden, inter)
               for l, e in ids}
    return x, logits, experts


def zipf_routing(rng, tokens, n_experts, k, s=1.1):
    """k distinct experts per token drawn with p_i ~ 1/rank**s under a seeded rank permutation;
    gate weights = sigmoid of the drawn logits, renormalised to sum 1."""
    ranks = rng.permutation(n_experts) + 1
    p = 1.0 / ranks.astype(np.float64) ** s
    p /= p.sum()
    ids = np.empty((tokens, k), dtype=np.int32)
    # Gumbel top-k = sampling without replacement proportional to p
    g = rng.gumbel(size=(tokens, n_experts)) + np.log(p)[None, :]
    ids[:] = np.argsort(-g, axis=1, kind="stable")[:, :k]
    logits = rng.standard_normal((tokens, k)).astype(np.float32)
    sig = 1.0 / (1.0 + np.exp(-logits.astype(np.float64)))
    w = (sig / sig.sum(axis=1, keepdims=True)).astype(np.float32)
    return ids, w


def config3(seed=0, tokens=4096, hidden=4096, inter=2880, n_experts=384, k=6, materialise=None):
    rng = np.random.default_rng(seed)
    x = round_bf16(rng.standard_normal((tokens, hidden)).astype(np.float32))
    ids, w = zipf_routing(rng, tokens, n_experts, k)
    use = sorted(set(ids.reshape(-1).tolist())) if materialise is None else materialise
    experts = {int(e): fp4_expert(np.random.default_rng([seed, int(e)]), hidden, inter) for e in use}
    return x, ids, w, experts


_FINITE_E4M3 = np.array([b for b in range(256) if (b & 0x7F) != 0x7F], dtype=np.uint8)


def fp8_matrix(rng, n, k, block=128, scale_rule="f32"):
    codes = _FINITE_E4M3[rng.integers(0, _FINITE_E4M3.size, (n, k))]
    shape = (-(-n // block), k // block)
    if scale_rule == "f32":
        scales = rng.uniform(1e-3, 1e-2, shape).astype(np.float32)
    else:
        scales = rng.integers(120, 134, shape, dtype=np.uint8)
    return codes, scales


def config4(seed=0, shapes=((12288, 4096), (4096, 8192)), batch=1, block=128, scale_rule="f32"):
    rng = np.random.default_rng(seed)
    mats = []
    for n, k in shapes:
        w, s = fp8_matrix(rng, n, k, block, scale_rule)
        x = round_bf16(rng.standard_normal((batch, k)).astype(np.float32))
        mats.append((x, w, s))
    return mats
