"""Expert-major prefill oracle: row grouping, per-expert batched FFN, slot-ordered combine.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  Restatement ("parity unpinned" beyond the
ordering rules) of
  src/cachalot/model/moe_prefill_grouped.py:201-225  rows of an expert = its (token, route slot) pairs in
                                                     token-major, slot-minor order
  src/cachalot/glm/experts.py:301-303                the same as a stable argsort of the flattened ids
  src/cachalot/model/moe_prefill_grouped.py:464-467,526-530  results kept per route slot, summed slot 0..k-1
  src/cachalot/model/fp4_sgmm_metal.py:203-233,195   rounding points of the FP4 prefill expert:
       g,u -> bf16 -> f32; h = silu(g)*u*w -> bf16; down output -> bf16 -> f32
  src/cachalot/model/moe_prefill_batched.py:31-61    same contract for > 64 rows
"""
from __future__ import annotations

import numpy as np

from .bf16 import round_bf16
from .fp4 import dequantize_fp4_weight, swiglu
from .mxfp4 import roundtrip as mxfp4_roundtrip


def group_rows(expert_ids: np.ndarray, n_experts: int):
    """expert_ids [T,k] -> (perm i32 [T*k], offsets i32 [E+1]).

    perm lists flattened (token*k + slot) row ids sorted by expert id, stable, so each expert's
    rows are in token-major, slot-minor order; offsets[e]:offsets[e+1] is expert e's range."""
    flat = np.asarray(expert_ids).reshape(-1).astype(np.int64)
    perm = np.argsort(flat, kind="stable").astype(np.int32)
    counts = np.bincount(flat, minlength=n_experts)
    offsets = np.zeros(n_experts + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts)
    return perm, offsets


def fp4_expert_rows(x_rows, w1, s1, w2, s2, w3, s3, weights, *, swiglu_limit=10.0,
                    act="bf16", acc=np.float32):
    """x_rows [m,H] -> f32 [m,H].  act="bf16": the reference's numerics (bf16 activations);
    act="mxfp4": activations (x, and the hidden h) quantised per 32 to MXFP4 first, which is the
    configured prefill variant; act="f32": no activation rounding."""
    x = np.asarray(x_rows, dtype=np.float32)
    if act == "bf16":
        x = round_bf16(x)
    elif act == "mxfp4":
        x = mxfp4_roundtrip(x)
    g = (x.astype(acc) @ dequantize_fp4_weight(w1, s1).astype(acc).T).astype(np.float32)
    u = (x.astype(acc) @ dequantize_fp4_weight(w3, s3).astype(acc).T).astype(np.float32)
    if act != "f32":
        g, u = round_bf16(g), round_bf16(u)
    h = (swiglu(g, u, swiglu_limit) * np.asarray(weights, dtype=np.float32).reshape(-1, 1)).astype(np.float32)
    if act == "bf16":
        h = round_bf16(h)
    elif act == "mxfp4":
        h = mxfp4_roundtrip(h)
    y = (h.astype(acc) @ dequantize_fp4_weight(w2, s2).astype(acc).T).astype(np.float32)
    return round_bf16(y) if act != "f32" else y


def moe_prefill_fp4(x, expert_ids, weights, bank, *, n_experts, swiglu_limit=10.0, act="bf16", acc=np.float32):
    """x [T,H]; expert_ids/weights [T,k]; bank(e) -> dict of the six byte arrays.  Returns f32 [T,H]
    = sum over route slots 0..k-1 (in that order) of the expert outputs."""
    x = np.asarray(x, dtype=np.float32)
    t, k = np.shape(expert_ids)
    perm, offsets = group_rows(expert_ids, n_experts)
    slot_buffer = np.zeros((t, k, x.shape[1]), dtype=np.float32)
    wflat = np.asarray(weights, dtype=np.float32).reshape(-1)
    for e in range(n_experts):
        rows = perm[offsets[e]:offsets[e + 1]]
        if rows.size == 0:
            continue
        m = bank(e)
        y = fp4_expert_rows(x[rows // k], m["w1.weight"], m["w1.scale"], m["w2.weight"], m["w2.scale"],
                            m["w3.weight"], m["w3.scale"], wflat[rows], swiglu_limit=swiglu_limit, act=act, acc=acc)
        slot_buffer[rows // k, rows % k] = y
    out = slot_buffer[:, 0]
    for s in range(1, k):
        out = out + slot_buffer[:, s]
    return out
