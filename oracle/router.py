"""Router oracles: the DeepSeek sqrt-softplus router (R1) and the sigmoid routing tail (R2).

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  Both exist only as MLX / Metal code in
the reference, so this is a restatement ("parity unpinned" beyond the rules cited here).

R1 follows src/cachalot/model/router_mlx.py:16-118 (formula, stable argsort, last k taken,
i.e. ascending by selection score) and router_fused_metal.py:47-49 (stable softplus form),
:78-83 (tie: the larger index wins), :96-101 (normalise then scale).
R2 follows src/cachalot/minimax/gpu_select.py:80-115: sigmoid written as
y = 1/(1+exp(|x|)), s = x<0 ? y : 1-y; rank by -(s+bias) with ties to the lower index;
top-k in rank order (strongest first); weights = s/(sum+1e-20)*scale, sum taken in rank
order; slots looked up in an int32 [layers, E] table.
"""
from __future__ import annotations

import numpy as np

from .bf16 import round_bf16


def sqrt_softplus_scores(logits: np.ndarray, gate_temp: float = 1.0) -> np.ndarray:
    s = (np.asarray(logits, dtype=np.float32) / np.float32(gate_temp)).astype(np.float32)
    sp = np.maximum(s, np.float32(0)) + np.log(np.float32(1) + np.exp(-np.abs(s)))
    return np.sqrt(sp.astype(np.float32)).astype(np.float32)


def router_logits(x: np.ndarray, gate_weight: np.ndarray) -> np.ndarray:
    """[E,H] @ [H] (or rows [T,H]) with float64 accumulation, rounded once to float32."""
    x = np.asarray(x, dtype=np.float32).astype(np.float64)
    w = np.asarray(gate_weight, dtype=np.float32).astype(np.float64)
    return (x @ w.T).astype(np.float32)


def topk_from_scores_r1(scores, bias, *, topk=6, route_scale=1.5, norm_topk_prob=True):
    """scores f32 [E] -> (indices i32 [k] ascending by score+bias, weights f32 [k])."""
    scores = np.asarray(scores, dtype=np.float32)
    sel = (scores + np.asarray(bias, dtype=np.float32)).astype(np.float32)
    if not 1 <= topk <= scores.size:
        raise ValueError(f"Invalid topk={topk} for {scores.size} experts")
    order = np.argsort(sel, kind="stable")
    idx = order[-topk:].astype(np.int32)
    w = scores[idx].astype(np.float32)
    if norm_topk_prob and topk > 1:
        total = np.float32(0)
        for v in w:  # fixed order j = 0..k-1 (router_fused_metal.py:98)
            total = np.float32(total + v)
        w = (w / np.float32(total + np.float32(1e-20))).astype(np.float32)
    w = (w * np.float32(route_scale)).astype(np.float32)
    return idx, w


def route_topk(x, gate_weight, bias, *, topk=6, gate_temp=1.0, route_scale=1.5, norm_topk_prob=True):
    """R1 for one token; returns (indices, weights, scores)."""
    x = np.asarray(x)
    if x.ndim != 1:
        raise ValueError(f"x must be 1D, got {x.shape}")
    scores = sqrt_softplus_scores(router_logits(x, gate_weight), gate_temp)
    idx, w = topk_from_scores_r1(scores, bias, topk=topk, route_scale=route_scale, norm_topk_prob=norm_topk_prob)
    return idx, w, scores


def sigmoid_scores(raw: np.ndarray) -> np.ndarray:
    x = np.asarray(raw, dtype=np.float32)
    y = (np.float32(1) / (np.float32(1) + np.exp(np.abs(x)))).astype(np.float32)
    return np.where(x < 0, y, np.float32(1) - y).astype(np.float32)


def topk_from_scores_r2(s, bias, *, k=6, scale=1.0, weights_bf16=False):
    """s f32 [E] sigmoid scores -> (indices u32 [k] strongest first, weights f32 [k])."""
    s = np.asarray(s, dtype=np.float32)
    neg = (-(s + np.asarray(bias, dtype=np.float32))).astype(np.float32)
    order = np.argsort(neg, kind="stable")  # ascending -(s+b); ties keep the lower index first
    top = order[:k]
    total = s[top[0]]
    for r in range(1, k):
        total = np.float32(total + s[top[r]])
    den = np.float32(total + np.float32(1e-20))
    w = ((s[top] / den).astype(np.float32) * np.float32(scale)).astype(np.float32)
    if weights_bf16:
        w = round_bf16(w)
    return top.astype(np.uint32), w


def route_tail(raw, bias, table, layer, k, scale, *, weights_bf16=True):
    """R2 for one token: raw f32 [E] gate output -> (inds u32 [k], weights, slots i32 [k])."""
    raw = np.asarray(raw, dtype=np.float32).reshape(-1)
    inds, w = topk_from_scores_r2(sigmoid_scores(raw), bias, k=k, scale=scale, weights_bf16=weights_bf16)
    slots = np.asarray(table, dtype=np.int32).reshape(-1, raw.size)[layer, inds.astype(np.int64)]
    return inds, w, slots.astype(np.int32)
