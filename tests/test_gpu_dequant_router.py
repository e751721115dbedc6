"""GPU parity: dequant tables and routing (bit-exact items)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import affine, configs, fp4, router  # noqa: E402
from oracle.bf16 import round_bf16  # noqa: E402


def _cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_fp4_dequant_every_code_and_scale():
    import cachalot_b200 as cb
    # all 256 byte values in every position of a 32-block, against every scale byte 0..254
    packed = np.tile(np.arange(256, dtype=np.uint8).reshape(16, 16), (16, 1))[:255]
    scales = np.arange(255, dtype=np.uint8).reshape(255, 1)
    got = cb.dequantize_fp4_weight(_cuda(packed), _cuda(scales)).cpu().numpy()
    with np.errstate(over="ignore"):
        want = fp4.dequantize_fp4_weight(packed, scales)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_fp4_dequant_golden_and_config_shape(golden):
    import cachalot_b200 as cb
    got = cb.dequantize_fp4_weight(_cuda(golden["fp4_packed"]), _cuda(golden["fp4_scales"])).cpu().numpy()
    assert np.array_equal(got, golden["fp4_dequant"])
    rng = np.random.default_rng(0)
    p, s = configs.fp4_matrix(rng, 2880, 4096)
    got = cb.dequantize_fp4_weight(_cuda(p), _cuda(s)).cpu().numpy()
    assert np.array_equal(got, fp4.dequantize_fp4_weight(p, s))


def test_fp4_dequant_errors():
    import cachalot_b200 as cb
    with pytest.raises(ValueError, match="Scale shape"):
        cb.dequantize_fp4_weight(torch.zeros(2, 16, dtype=torch.uint8, device="cuda"), torch.zeros(2, 2, dtype=torch.uint8, device="cuda"))
    with pytest.raises(ValueError, match="divisible"):
        cb.dequantize_fp4_weight(torch.zeros(2, 8, dtype=torch.uint8, device="cuda"), torch.zeros(2, 1, dtype=torch.uint8, device="cuda"))
    out = cb.dequantize_fp4_weight(torch.zeros(0, 16, dtype=torch.uint8, device="cuda"), torch.zeros(0, 1, dtype=torch.uint8, device="cuda"))
    assert tuple(out.shape) == (0, 32)


@pytest.mark.parametrize("dt", ["float16", "bfloat16"])
def test_affine_dequant_bit_exact(dt):
    import cachalot_b200 as cb
    rng = np.random.default_rng(1)
    n, k = 96, 512
    w, s, b = configs.affine_matrix(rng, n, k)
    if dt == "bfloat16":
        s32, b32 = round_bf16(s.astype(np.float32)), round_bf16(b.astype(np.float32))
        st, bt = torch.from_numpy(s32).cuda().to(torch.bfloat16), torch.from_numpy(b32).cuda().to(torch.bfloat16)
    else:
        s32, b32 = s.astype(np.float32), b.astype(np.float32)
        st, bt = _cuda(s), _cuda(b)
    got = cb.dequantize_affine(_cuda(w.view(np.int32)), st, bt, bits=2, group_size=128).cpu().numpy()
    want = affine.dequantize_affine(w, s32, b32, bits=2, group_size=128)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def _near_tie(scores_sorted_desc, k, ulps=8):
    a, b = scores_sorted_desc[k - 1], scores_sorted_desc[k]
    return abs(float(a) - float(b)) <= ulps * np.spacing(np.float32(max(abs(a), abs(b))))


def test_router_sigmoid_matches_oracle_and_slot_lookup():
    import cachalot_b200 as cb
    rng = np.random.default_rng(2)
    e, k, rows, layers = 384, 6, 64, 3
    raw = rng.standard_normal((rows, e)).astype(np.float32)
    bias = np.zeros(e, np.float32)
    table = rng.permutation(layers * e).astype(np.int32).reshape(layers, e)
    inds, w, slots = cb.route_tail(_cuda(raw), _cuda(bias), _cuda(table), 2, k, 1.0, weights_bf16=False)
    inds, w, slots = inds.cpu().numpy(), w.cpu().numpy(), slots.cpu().numpy()
    for r in range(rows):
        oi, ow, os_ = router.route_tail(raw[r], bias, table, 2, k, 1.0, weights_bf16=False)
        s = np.sort(router.sigmoid_scores(raw[r]))[::-1]
        if _near_tie(s, k):
            continue
        assert inds[r].tolist() == oi.tolist()
        assert slots[r].tolist() == os_.tolist()
        assert np.allclose(w[r], ow, rtol=2e-6, atol=0)
        assert abs(float(w[r].sum()) - 1.0) < 1e-6


def test_router_sigmoid_tie_rule_and_bf16_weights():
    import cachalot_b200 as cb
    raw = np.array([[0.0, 2.0, 2.0, -1.0, 2.0, 0.5, 2.0, -3.0]], dtype=np.float32)
    inds, w, slots = cb.route_tail(_cuda(raw), None, None, 0, 3, 1.0)
    assert inds.cpu().numpy()[0].tolist() == [1, 2, 4]            # ties -> lower index, strongest first
    assert slots.cpu().numpy()[0].tolist() == [1, 2, 4]
    wn = w.cpu().numpy()
    assert np.array_equal(wn, round_bf16(wn))


def test_router_sqrt_softplus_topk_bit_exact_on_gpu_scores():
    import cachalot_b200 as cb
    rng = np.random.default_rng(3)
    e, h, k = 384, 512, 6
    x = round_bf16(rng.standard_normal(h).astype(np.float32))
    gw = (rng.standard_normal((e, h)) * 0.05).astype(np.float32)
    bias = (rng.standard_normal(e) * 0.01).astype(np.float32)
    res = cb.route_topk_fused(_cuda(x).to(torch.bfloat16), _cuda(gw), _cuda(bias), topk=k, route_scale=1.5)
    scores = res.scores.cpu().numpy()
    # the selection and the weights are bit-exact given the scores the GPU computed
    oi, ow = router.topk_from_scores_r1(scores, bias, topk=k, route_scale=1.5)
    assert res.indices.cpu().numpy().tolist() == oi.tolist()
    assert np.allclose(res.weights.cpu().numpy(), ow, rtol=3e-7, atol=0)
    # and the scores agree with the float64-accumulated oracle
    _, _, oscores = router.route_topk(x, gw, bias, topk=k)
    assert np.max(np.abs(scores - oscores)) < 1e-5


def test_router_sqrt_softplus_tie_rule_rows():
    import cachalot_b200 as cb
    # identical gate rows give identical scores: ties go to the larger index, output ascends
    h, e = 64, 8
    gw = np.zeros((e, h), np.float32)
    gw[[1, 2, 4], 0] = 1.0
    gw[0, 0] = 0.5
    x = np.zeros((2, h), np.float32)
    x[:, 0] = 1.0
    res = cb.route_topk_rows(_cuda(x).to(torch.bfloat16), _cuda(gw), torch.zeros(e, device="cuda"), topk=2, route_scale=1.0)
    assert res.indices.cpu().numpy().tolist() == [[2, 4], [2, 4]]
    assert np.allclose(res.weights.cpu().numpy(), 0.5)
    with pytest.raises(ValueError, match="Invalid topk"):
        cb.route_topk_fused(_cuda(x[0]).to(torch.bfloat16), _cuda(gw), torch.zeros(e, device="cuda"), topk=9)
    with pytest.raises(ValueError, match="must be 1D"):
        cb.route_topk_fused(_cuda(x).to(torch.bfloat16), _cuda(gw), torch.zeros(e, device="cuda"))
