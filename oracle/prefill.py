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


def fp4_expert_rows_bounds(x_rows, w1, s1, w2, s2, w3, s3, weights, *, swiglu_limit=10.0, eps_acc=2.0 ** -21, eps_fn=1e-5):
    """The mxfp4 variant of `fp4_expert_rows` together with what a correct fp32 implementation may
    deviate from it, element by element, so that a parity test needs no "most rows" clause.

    The MXFP4 quantiser of the hidden activation is discontinuous: an implementation whose fp32 sums differ
    from the float64 sums here in the last bits can round a value of g or u to the neighbouring bf16 number,
    and a value of h to the neighbouring E2M1 code.  For every element the function follows both candidates:
      g, u   in [exact -+ eps_acc * sum|x||w|]  ->  the one or two bf16 values that interval rounds to
      h      the range over those candidates, widened by eps_fn (exp and division in fast fp32 form)
      codes  the E2M1 codes of the two ends of h's range under the block's scale; `dev` = how far the decoded
             value can be from the nominal one (zero for all but the few elements that sit on a boundary)
    Returns a dict:
      y        f32 [m,H]  nominal output, rounded to bf16 (what `fp4_expert_rows(act="mxfp4")` gives with float64 sums)
      allow    f64 [m,H]  |W2| . dev + eps_acc * sum|h||w2|: admissible deviation of the unrounded output
      flip     bool [m,H] the unrounded output, within `allow`, may round to the other neighbouring bf16 value
      ulp      f32 [m,H]  that bf16 step
      scale_fragile bool [m]  a block maximum of h sits on a power-of-two boundary of the E8M0 scale: the whole
                              block may be coded on the other grid; such rows are to be exempted (and counted)
      n_boundary int [m]  elements of h with two candidate codes
    """
    from .mxfp4 import FP4_MAX, MIN_AMAX, round_e2m1_codes
    from .fp4 import E2M1_VALUES

    x = mxfp4_roundtrip(np.asarray(x_rows, dtype=np.float32)).astype(np.float64)
    W1 = dequantize_fp4_weight(w1, s1).astype(np.float64)
    W3 = dequantize_fp4_weight(w3, s3).astype(np.float64)
    W2 = dequantize_fp4_weight(w2, s2).astype(np.float64)
    wts = np.asarray(weights, dtype=np.float32).reshape(-1, 1)
    ax = np.abs(x)

    def bf16_range(M):
        v = x @ M.T
        e = eps_acc * (ax @ np.abs(M).T)
        return round_bf16((v - e).astype(np.float32)), round_bf16((v + e).astype(np.float32)), round_bf16(v.astype(np.float32))

    g_lo, g_hi, g_nom = bf16_range(W1)
    u_lo, u_hi, u_nom = bf16_range(W3)

    def hidden(g, u):
        return (swiglu(g, u, swiglu_limit) * wts).astype(np.float32).astype(np.float64)

    cands = [hidden(g, u) for g in (g_lo, g_hi) for u in (u_lo, u_hi)]
    h_nom = hidden(g_nom, u_nom)
    h_min = np.minimum.reduce(cands)
    h_max = np.maximum.reduce(cands)
    h_min = h_min - eps_fn * np.abs(h_min)
    h_max = h_max + eps_fn * np.abs(h_max)
    m, inter = h_nom.shape
    blk = lambda a: a.reshape(m, inter // 32, 32)
    abs_hi = np.maximum(np.abs(h_min), np.abs(h_max))
    abs_lo = np.where(np.sign(h_min) == np.sign(h_max), np.minimum(np.abs(h_min), np.abs(h_max)), 0.0)

    def exponent(amax):
        amax = np.maximum(amax.astype(np.float32), np.float32(MIN_AMAX))
        return np.ceil(np.log2((amax / np.float32(FP4_MAX)).astype(np.float32))).astype(np.int32)

    e_nom = exponent(blk(np.abs(h_nom)).max(-1))
    e_lo, e_hi = exponent(blk(abs_lo).max(-1)), exponent(blk(abs_hi).max(-1))
    scale_fragile = np.any((e_lo != e_nom) | (e_hi != e_nom), axis=1)
    scale = np.exp2(e_nom.astype(np.float64))[..., None]

    def decode(h):
        norm = np.clip((blk(h) / scale).astype(np.float32), -FP4_MAX, FP4_MAX)
        return (E2M1_VALUES[round_e2m1_codes(norm)].astype(np.float64) * scale).reshape(m, inter)

    q_nom, q_lo, q_hi = decode(h_nom), decode(h_min), decode(h_max)
    dev = np.maximum(np.abs(q_lo - q_nom), np.abs(q_hi - q_nom))
    aW2 = np.abs(W2)
    y64 = q_nom @ W2.T
    allow = dev @ aW2.T + eps_acc * (np.abs(q_nom) @ aW2.T)
    y = round_bf16(y64.astype(np.float32))
    lo, hi = round_bf16((y64 - allow).astype(np.float32)), round_bf16((y64 + allow).astype(np.float32))
    flip = lo != hi
    ulp = np.maximum(np.abs(hi - y), np.abs(y - lo)).astype(np.float32)
    return {"y": y, "allow": allow, "flip": flip, "ulp": ulp, "scale_fragile": scale_fragile,
            "n_boundary": np.count_nonzero(dev > 0, axis=1)}


def check_rows_against_bounds(got, b, tol):
    """got f32 [m,H] (bf16-rounded outputs of an implementation) against `fp4_expert_rows_bounds`'s dict.
    Returns (ok bool [m], exempt bool [m], worst float): a row is ok when every element is within
    tol * max|y| of the nominal value plus what the element's own boundary cases admit."""
    y = b["y"].astype(np.float64)
    ref = max(float(np.max(np.abs(y))), 1e-30)
    slack = tol * ref + b["allow"] + np.where(b["flip"], b["ulp"].astype(np.float64), 0.0)
    err = np.abs(np.asarray(got, np.float64) - y)
    ok = np.all(err <= slack, axis=1)
    worst = float(np.max((err - b["allow"] - np.where(b["flip"], b["ulp"], 0.0)) / ref))
    return ok, b["scale_fragile"], worst
