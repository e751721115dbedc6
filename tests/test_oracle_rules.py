"""Known answers the reference states in code: tie rules, rounding tables, packing, ordering."""
import numpy as np
import pytest

from oracle import affine, fp4, mxfp4, prefill, router
from oracle.bf16 import round_bf16


def test_affine_3bit_straddle_vector():
    lv = np.zeros((1, 32), dtype=np.uint32)
    lv[0, 10] = 7
    assert [int(v) for v in affine.pack_bits(lv, 3)[0]] == [0xC0000000, 0x1, 0]


def test_affine_2bit_low_field_first_and_roundtrip():
    lv = np.arange(16, dtype=np.uint32)[None, :] % 4
    word = int(affine.pack_bits(lv, 2)[0, 0])
    assert word == sum(int(v) << (2 * i) for i, v in enumerate(lv[0]))
    rng = np.random.default_rng(0)
    for bits in (2, 3, 4, 8):
        l = rng.integers(0, 1 << bits, (4, 256))
        assert (affine.unpack_bits(affine.pack_bits(l, bits), bits, 256) == l).all()
    with pytest.raises(ValueError):
        affine.pack_bits(np.zeros((2, 20)), 3)


def test_affine_dequant_formula_single_rounding():
    rng = np.random.default_rng(1)
    w, s, b = affine.quantize_affine_minmax(rng.standard_normal((8, 256)).astype(np.float32), bits=2, group_size=128)
    d = affine.dequantize_affine(w, s, b, bits=2, group_size=128)
    q = affine.unpack_bits(w, 2, 256).astype(np.float64).reshape(8, 2, 128)
    want = (s.astype(np.float64)[:, :, None] * q + b.astype(np.float64)[:, :, None]).astype(np.float32).reshape(8, 256)
    assert np.array_equal(d, want)


def test_router_r1_tie_goes_to_larger_index_and_output_ascends():
    scores = np.array([0.5, 0.9, 0.9, 0.1, 0.9, 0.3], dtype=np.float32)
    idx, w = router.topk_from_scores_r1(scores, np.zeros(6, np.float32), topk=2, route_scale=1.5)
    assert idx.tolist() == [2, 4]           # of the three 0.9s the two larger indices, ascending
    assert np.allclose(w, [0.75, 0.75])
    idx, _ = router.topk_from_scores_r1(scores, np.zeros(6, np.float32), topk=4)
    assert idx.tolist() == [0, 1, 2, 4]     # weakest first
    # bias moves selection but not the weights
    bias = np.array([0, 0, 0, 5, 0, 0], dtype=np.float32)
    idx, w = router.topk_from_scores_r1(scores, bias, topk=1, route_scale=2.0, norm_topk_prob=True)
    assert idx.tolist() == [3] and np.allclose(w, [0.2])


def test_router_r2_tie_goes_to_lower_index_strongest_first():
    raw = np.array([0.0, 2.0, 2.0, -1.0, 2.0, 0.5], dtype=np.float32)
    inds, w, slots = router.route_tail(raw, np.zeros(6, np.float32), np.arange(12, dtype=np.int32).reshape(2, 6) * 10,
                                       layer=1, k=3, scale=1.0, weights_bf16=False)
    assert inds.tolist() == [1, 2, 4]
    assert slots.tolist() == [70, 80, 100]
    assert abs(float(w.sum()) - 1.0) < 1e-6
    inds, w, _ = router.route_tail(raw, np.zeros(6, np.float32), np.arange(6, dtype=np.int32)[None], 0, 4, 1.0)
    assert inds.tolist() == [1, 2, 4, 5]
    assert np.array_equal(w, round_bf16(w))


def test_mxfp4_tie_table_and_signed_zero():
    v = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 0.26, 0.74, 5.01, -0.25, -0.75, -0.0, 6.0], dtype=np.float32)
    codes = mxfp4.round_e2m1_codes(v)
    vals = fp4.E2M1_VALUES[codes & 7] * np.where(codes & 8, -1, 1)
    assert vals.tolist() == [0, 1, 1, 2, 2, 4, 4, 0.5, 0.5, 6, 0, -1, 0, 6]
    assert codes[10] == 8 and codes[12] == 8          # negative values that round to zero keep the sign bit
    x = np.zeros((1, 32), dtype=np.float32)
    x[0, 0], x[0, 1] = 6.0, 3.0
    c, s = mxfp4.quantize_mxfp4(x)
    assert s[0, 0] == 127 and c[0, 0] == 7 and c[0, 1] == 5
    x[0, 0] = 6.5                                       # amax/6 just above 1 -> scale 2
    c, s = mxfp4.quantize_mxfp4(x)
    assert s[0, 0] == 128
    c, s = mxfp4.quantize_mxfp4(np.zeros((1, 32), np.float32))
    assert s[0, 0] == 1                                 # amax floor 6 * 2**-126


def test_group_rows_is_token_major_slot_minor():
    ids = np.array([[2, 0], [0, 2], [1, 0]], dtype=np.int32)
    perm, off = prefill.group_rows(ids, 4)
    assert off.tolist() == [0, 3, 4, 6, 6]
    assert perm.tolist() == [1, 2, 5, 4, 0, 3]


def test_fp4_affine8_identity():
    rng = np.random.default_rng(2)
    p = rng.integers(0, 256, (4, 32), dtype=np.uint8)
    s = rng.integers(110, 130, (4, 2), dtype=np.uint8)
    q, sc, bi = fp4.fp4_to_affine8(p, s)
    assert q.max() <= 24
    rebuilt = (sc[:, :, None] * q.reshape(4, 2, 32) + bi[:, :, None]).reshape(4, 64)
    assert np.array_equal(rebuilt, fp4.dequantize_fp4_weight(p, s))


def test_fused_topk_equals_per_expert_loop_and_weight_before_down():
    from oracle import configs
    rng = np.random.default_rng(3)
    experts = [configs.fp4_expert(rng, 64, 96) for _ in range(3)]
    x = rng.standard_normal(64).astype(np.float32)
    w = np.array([0.2, 0.5, 0.3], dtype=np.float32)
    total = fp4.routed_topk_forward(x, experts, w, swiglu_limit=10.0)
    loop = sum(fp4.expert_forward(x, e["w1.weight"], e["w1.scale"], e["w2.weight"], e["w2.scale"], e["w3.weight"],
                                  e["w3.scale"], weight=wi, swiglu_limit=10.0) for e, wi in zip(experts, w))
    assert np.allclose(total, loop, rtol=1e-6, atol=1e-6)
    e = experts[0]
    a = fp4.expert_forward(x, e["w1.weight"], e["w1.scale"], e["w2.weight"], e["w2.scale"], e["w3.weight"], e["w3.scale"],
                           weight=0.5, swiglu_limit=0.0)
    b = 0.5 * fp4.expert_forward(x, e["w1.weight"], e["w1.scale"], e["w2.weight"], e["w2.scale"], e["w3.weight"],
                                 e["w3.scale"], weight=None, swiglu_limit=0.0)
    assert np.allclose(a, b, rtol=1e-5, atol=1e-6)


def test_prefill_slot_order_equals_decode_per_row():
    from oracle import configs
    x, ids, w, experts = configs.config3(seed=5, tokens=6, hidden=64, inter=96, n_experts=8, k=3)
    out = prefill.moe_prefill_fp4(x, ids, w, lambda e: experts[e], n_experts=8, act="f32")
    for t in range(6):
        want = fp4.routed_topk_forward(x[t], [experts[int(e)] for e in ids[t]], w[t])
        assert np.allclose(out[t], want, rtol=1e-5, atol=1e-5)


def test_affine_expert_oracle_matches_dense_math_to_two_percent():
    """The reference's own check of a 2-bit g128 expert (tests/test_expert_bank.py:93-116) restated on the oracle:
    the quantised expert against dense matrices (the dequantised weights) with the same bf16 rounding points,
    within 2 % of the output's maximum; a row of a batch equals the same row alone within 2 %."""
    from oracle import affine
    from oracle.bf16 import round_bf16

    rng = np.random.default_rng(7)
    hidden, inter, bits, group = 256, 128, 2, 128
    mats, dense = {}, {}
    for proj, (n, k) in (("w1", (inter, hidden)), ("w3", (inter, hidden)), ("w2", (hidden, inter))):
        w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
        words, s, b = affine.quantize_affine_minmax(w, bits=bits, group_size=group)
        mats[f"{proj}.weight"], mats[f"{proj}.scales"], mats[f"{proj}.biases"] = words, s, b
        dense[proj] = affine.dequantize_affine(words, s, b, bits=bits, group_size=group).astype(np.float64)
    x = round_bf16(rng.standard_normal(hidden).astype(np.float32))
    got = affine.affine_expert_forward(x, mats, bits=bits, group_size=group, weight=0.7, swiglu_limit=10.0)
    xb = x.astype(np.float64)
    gate = np.minimum(round_bf16((dense["w1"] @ xb).astype(np.float32)), 10.0)
    up = np.clip(round_bf16((dense["w3"] @ xb).astype(np.float32)), -10.0, 10.0)
    h = round_bf16((gate / (1.0 + np.exp(-gate)) * up * 0.7).astype(np.float32))
    want = round_bf16((dense["w2"] @ h.astype(np.float64)).astype(np.float32))
    scale = float(np.abs(want).max())
    assert float(np.abs(got - want).max()) < 0.02 * scale
    xm = round_bf16(rng.standard_normal((4, hidden)).astype(np.float32))
    batched = affine.affine_expert_forward(xm, mats, bits=bits, group_size=group, weight=np.array([0.7, 0.1, 1.0, 0.3]))
    single = affine.affine_expert_forward(xm[1], mats, bits=bits, group_size=group, weight=0.1)
    assert float(np.abs(batched[1] - single).max()) < 0.02 * max(1e-6, float(np.abs(single).max()))


def test_bf16_gemv_oracle_widens_by_a_shift():
    """bf16 -> fp32 is a shift (model/bf16_gemv_metal.py:33-35): known bit patterns, and the product against
    hand-computed sums."""
    from oracle import bf16_gemv
    bits = np.array([[0x3F80, 0xBF80, 0x4000, 0x0000], [0x3F00, 0x3E80, 0xC040, 0x7F80]], dtype=np.uint16)
    assert bf16_gemv.bf16_to_f32(bits).tolist() == [[1.0, -1.0, 2.0, 0.0], [0.5, 0.25, -3.0, float("inf")]]
    x = np.array([1.0, 2.0, 3.0, 4.0], dtype=np.float32)
    assert bf16_gemv.bf16_gemv_f32(x, bits[:1]).tolist() == [1.0 - 2.0 + 6.0]
    assert bf16_gemv.bf16_gemv_f32(np.stack([x, 2 * x]), bits[:1]).tolist() == [[5.0], [10.0]]
