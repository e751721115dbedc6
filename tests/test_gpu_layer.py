"""GPU parity: the shared FP8 expert, the fused trunk projections and the whole decode MoE layer (router GEMV ->
routing -> routed experts -> shared expert -> sum -> bf16) against the oracle, through the reference-named entries."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import affine, configs, fp4, fp8, router, shared  # noqa: E402
from oracle.bf16 import round_bf16  # noqa: E402
from tests.helpers import bf16_tensor, make_bank, max_rel  # noqa: E402

TOL = 2e-3


def _cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _shared_weights(rng, hidden, inter, block, rule):
    w1, s1 = configs.fp8_matrix(rng, inter, hidden, block, rule)
    w3, s3 = configs.fp8_matrix(rng, inter, hidden, block, rule)
    w2, s2 = configs.fp8_matrix(rng, hidden, inter, block, rule)
    return w1, s1, w2, s2, w3, s3


def _bf16_steps(got, want, tol=TOL):
    """Elements outside tol * max|want|, and the largest error in units of max|want|: a bf16 output may sit one step
    (2**-8 of its own size) from the oracle's where the unrounded values straddle a rounding boundary."""
    ref = float(np.max(np.abs(want)))
    err = np.abs(np.asarray(got, np.float64) - want) / ref
    return int(np.count_nonzero(err >= tol)), float(err.max())


@pytest.mark.parametrize("hidden,inter,block,rule", [(4096, 2880, 32, "e8m0"), (5120, 2304, 32, "e8m0"), (5120, 2304, 128, "f32"),
                                                     (512, 384, 32, "f32")])
def test_shared_expert_matches_oracle(hidden, inter, block, rule):
    import cachalot_b200 as cb
    rng = np.random.default_rng(hidden + block)
    w1, s1, w2, s2, w3, s3 = _shared_weights(rng, hidden, inter, block, rule)
    sc = 0.05 if rule == "e8m0" else 1.0      # keeps the hidden activation in a sane range for either scale family
    x = round_bf16(rng.standard_normal((3, hidden)).astype(np.float32) * sc)
    want = shared.shared_expert_forward(x, w1, s1, w2, s2, w3, s3, block_size=block, scale_rule=rule)
    t = dict(w1=_cuda(w1), w1_scales=_cuda(s1), w2=_cuda(w2), w2_scales=_cuda(s2), w3=_cuda(w3), w3_scales=_cuda(s3))
    rows = cb.shared_expert_forward_batched(bf16_tensor(x), **t).float().cpu().numpy()
    moved, worst = _bf16_steps(rows, want)
    print(f"shared expert {hidden}x{inter} block {block} {rule}: {moved} of {want.size} elements one bf16 step away, max {worst:.2e}")
    assert worst < 2 ** -7 and moved <= max(2, want.size // 64)
    one = cb.shared_expert_forward(bf16_tensor(x)[0], **t)
    assert torch.equal(one.float().cpu(), torch.from_numpy(rows[0]))
    # w1 || w3 as one matrix: bit-identical to the two-GEMV form (the reference's test_shared_expert_fused.py:49)
    if inter % block == 0:
        w13, s13 = torch.cat([t["w1"], t["w3"]], 0), torch.cat([t["w1_scales"], t["w3_scales"]], 0)
        fused = cb.shared_expert_forward_fused(bf16_tensor(x)[0], w13=w13, w13_scales=s13, w2=t["w2"], w2_scales=t["w2_scales"])
        assert torch.equal(fused, one)
    with pytest.raises(ValueError):
        cb.shared_expert_forward(bf16_tensor(x), **t)          # decode entry takes one token


def test_fused_qr_kv_linear_equals_two_linears():
    """model/attention_qkv_fusion.py:46-68: one GEMV over the rows of both matrices, bit-identical to two calls."""
    import cachalot_b200 as cb
    rng = np.random.default_rng(3)
    k = 5120
    wq, sq = configs.fp8_matrix(rng, 1280, k, 32, "e8m0")
    wkv, skv = configs.fp8_matrix(rng, 512, k, 32, "e8m0")
    x = bf16_tensor(round_bf16(rng.standard_normal(k).astype(np.float32)))
    a, b = cb.fused_qr_kv_linear(x, _cuda(wq), _cuda(sq), _cuda(wkv), _cuda(skv))
    assert torch.equal(a, cb.fp8_linear(x, _cuda(wq), _cuda(sq))) and torch.equal(b, cb.fp8_linear(x, _cuda(wkv), _cuda(skv)))
    want = fp8.fp8_linear(x.float().cpu().numpy(), wq, sq)
    assert max_rel(a.float().cpu().numpy(), round_bf16(want)) < 2 ** -7


@pytest.mark.parametrize("kind,hidden,inter", [("fp4", 4096, 2880), ("fp4", 5120, 2304), ("affine", 4096, 2880)])
def test_moe_layer_forward_matches_oracle(kind, hidden, inter):
    """The reference's keyword signature end to end: gate GEMV in fp32, sqrt-softplus top-6 (indices bit-exact), routed
    experts over the bank, shared FP8 expert, (routed + shared.f32) -> bf16."""
    import cachalot_b200 as cb
    rng = np.random.default_rng(hidden)
    n_exp, k = 24, 6
    make = configs.fp4_expert if kind == "fp4" else configs.affine_expert
    fmt = cb.FP4_FORMAT if kind == "fp4" else cb.affine_format(hidden, inter)
    experts = [make(rng, hidden, inter) for _ in range(n_exp)]
    bank = make_bank(experts, fmt, hidden, inter)
    x = round_bf16(rng.standard_normal(hidden).astype(np.float32) * 0.05)
    gate_w = round_bf16(rng.standard_normal((n_exp, hidden)).astype(np.float32) * 0.3)
    gate_b = (rng.standard_normal(n_exp) * 0.05).astype(np.float32)
    w1, s1, w2, s2, w3, s3 = _shared_weights(rng, hidden, inter, 32, "e8m0")
    out, route = cb.moe_layer_forward(bf16_tensor(x), layer_id=0, gate_weight=bf16_tensor(gate_w), gate_bias=_cuda(gate_b),
                                      expert_index=None, expert_store=bank, shared_w1=_cuda(w1), shared_w1_scales=_cuda(s1),
                                      shared_w2=_cuda(w2), shared_w2_scales=_cuda(s2), shared_w3=_cuda(w3), shared_w3_scales=_cuda(s3),
                                      topk=k, gate_temp=1.0, route_scale=1.5, norm_topk_prob=True, swiglu_limit=10.0)
    o = router.route_topk(x, gate_w, gate_b, topk=k, gate_temp=1.0, route_scale=1.5, norm_topk_prob=True)
    o_idx, o_w = o[0], o[1]
    assert route.indices.cpu().numpy().tolist() == [int(i) for i in o_idx]
    assert np.allclose(route.weights.cpu().numpy(), o_w, rtol=1e-4)
    assert route.scores is not None and tuple(route.scores.shape) == (n_exp,)
    sel = [experts[int(i)] for i in o_idx]
    if kind == "fp4":
        routed = fp4.routed_topk_forward(x, sel, o_w, swiglu_limit=10.0, acc=np.float64)
    else:
        routed = affine.affine_routed_experts(x, sel, o_w, bits=2, group_size=128, swiglu_limit=10.0, acc=np.float64)
    sh = shared.shared_expert_forward(x, w1, s1, w2, s2, w3, s3)
    want = shared.close_layer(routed, sh)
    moved, worst = _bf16_steps(out.float().cpu().numpy(), want)
    print(f"layer {kind} {hidden}x{inter}: {moved} of {hidden} elements one bf16 step away, max {worst:.2e}")
    assert out.dtype == torch.bfloat16 and worst < 2 ** -7 and moved <= hidden // 32
    with pytest.raises(ValueError):
        cb.moe_layer_forward(bf16_tensor(x)[None], layer_id=0, gate_weight=bf16_tensor(gate_w), gate_bias=_cuda(gate_b),
                             expert_store=bank, shared_w1=_cuda(w1), shared_w1_scales=_cuda(s1), shared_w2=_cuda(w2),
                             shared_w2_scales=_cuda(s2), shared_w3=_cuda(w3), shared_w3_scales=_cuda(s3))


def test_reference_named_batched_expert_entries():
    """routed_expert_forward_batched / _sgmm (FP4) and affine_expert_forward_batched: rows through one expert with the
    prefill rounding points; SlabExperts keeps each expert's output apart."""
    import cachalot_b200 as cb
    from oracle import prefill
    rng = np.random.default_rng(17)
    hidden, inter, m = 512, 384, 10
    e = configs.fp4_expert(rng, hidden, inter)
    x = round_bf16(rng.standard_normal((m, hidden)).astype(np.float32))
    w = rng.uniform(0.1, 0.6, m).astype(np.float32)
    t = {k_: _cuda(v) for k_, v in e.items()}
    got = cb.routed_expert_forward_batched(bf16_tensor(x), w1_packed=t["w1.weight"], w1_scales=t["w1.scale"], w2_packed=t["w2.weight"],
                                           w2_scales=t["w2.scale"], w3_packed=t["w3.weight"], w3_scales=t["w3.scale"], weights=_cuda(w))
    want = prefill.fp4_expert_rows(x, e["w1.weight"], e["w1.scale"], e["w2.weight"], e["w2.scale"], e["w3.weight"], e["w3.scale"], w,
                                   act="bf16", acc=np.float64)
    moved, worst = _bf16_steps(got.cpu().numpy(), want)
    assert got.dtype == torch.float32 and worst < 2 ** -7 and moved <= want.size // 64
    assert cb.routed_expert_forward_sgmm is cb.routed_expert_forward_batched
    fmt = cb.affine_format(hidden, inter)
    ea = configs.affine_expert(rng, hidden, inter)
    ga = cb.affine_expert_forward_batched(bf16_tensor(x), {k_: _cuda(v.view(np.int32) if v.dtype == np.uint32 else v) for k_, v in ea.items()},
                                          fmt, _cuda(w))
    wa = affine.affine_expert_forward(x, ea, bits=2, group_size=128, weight=w, swiglu_limit=10.0, acc=np.float64)
    moved, worst = _bf16_steps(ga.cpu().numpy(), wa)
    assert worst < 2 ** -7 and moved <= wa.size // 64
    bank = make_bank([configs.fp4_expert(rng, hidden, inter) for _ in range(4)] + [e], cb.FP4_FORMAT, hidden, inter)
    slots = torch.tensor([4, 1, -1], dtype=torch.int32, device="cuda")
    per = cb.SlabExperts(bank)(bf16_tensor(x[:1]), slots, 10.0)
    assert tuple(per.shape) == (3, hidden) and float(per[2].abs().max()) == 0.0
    one = fp4.expert_forward(x[0], e["w1.weight"], e["w1.scale"], e["w2.weight"], e["w2.scale"], e["w3.weight"], e["w3.scale"],
                             weight=None, swiglu_limit=10.0, acc=np.float64)
    assert max_rel(per[0].float().cpu().numpy(), one) < 2 ** -7
