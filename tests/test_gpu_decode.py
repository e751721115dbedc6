"""GPU parity: routed-expert decode over FP4 and 2-bit affine banks (through the C ABI)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import affine, configs, fp4, router  # noqa: E402
from tests.helpers import bf16_tensor, expert_from_bank, make_bank, max_rel  # noqa: E402

TOL = 2e-3  # max relative error of layer outputs against the fp32-accumulated oracle


def _fp4_expert_out(x, e, w=None, limit=10.0):
    return fp4.expert_forward(x, e["w1.weight"], e["w1.scale"], e["w2.weight"], e["w2.scale"], e["w3.weight"], e["w3.scale"],
                              weight=w, swiglu_limit=limit, acc=np.float64)


def test_config0_single_fp4_expert_full_size():
    """x bf16 [1,4096], one FP4 expert 2880x4096, no clamp, no router weight, fp32 accumulation -> bf16."""
    import cachalot_b200 as cb
    x, e = configs.config0(seed=0)
    bank = make_bank([e], cb.FP4_FORMAT, 4096, 2880)
    slots = torch.zeros((1, 1), dtype=torch.int32, device="cuda")
    w = torch.ones((1, 1), dtype=torch.float32, device="cuda")
    got = cb.moe_forward(bf16_tensor(x), slots, w, bank, swiglu_limit=0.0).cpu().numpy()
    want = _fp4_expert_out(x, e, None, 0.0)
    assert max_rel(got, want) < TOL
    got_bf16 = cb.moe_forward(bf16_tensor(x), slots, w, bank, swiglu_limit=0.0, out_dtype=torch.bfloat16).float().cpu().numpy()
    assert max_rel(got_bf16, want) < 2 ** -8 + TOL
    # the loose-tensor entry of the reference gives the same numbers
    t = {k: torch.from_numpy(v).cuda() for k, v in e.items()}
    loose = cb.routed_expert_forward(bf16_tensor(x)[0], w1_packed=t["w1.weight"], w1_scales=t["w1.scale"], w2_packed=t["w2.weight"],
                                     w2_scales=t["w2.scale"], w3_packed=t["w3.weight"], w3_scales=t["w3.scale"], weight=None,
                                     swiglu_limit=0.0).cpu().numpy()
    assert np.array_equal(loose, got[0])


@pytest.mark.parametrize("rows", [1, 3, 8])
def test_fp4_topk_small_shapes_match_oracle(rows):
    import cachalot_b200 as cb
    rng = np.random.default_rng(10 + rows)
    hidden, inter, n_exp, k = 256, 192, 12, 6
    experts = [configs.fp4_expert(rng, hidden, inter) for _ in range(n_exp)]
    bank = make_bank(experts, cb.FP4_FORMAT, hidden, inter)
    x = configs.round_bf16(rng.standard_normal((rows, hidden)).astype(np.float32) * 4)
    ids = np.stack([rng.permutation(n_exp)[:k] for _ in range(rows)]).astype(np.int32)
    w = rng.uniform(0.05, 0.6, (rows, k)).astype(np.float32)
    got = cb.moe_forward(bf16_tensor(x), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), bank, swiglu_limit=10.0).cpu().numpy()
    want = np.stack([fp4.routed_topk_forward(x[t], [experts[i] for i in ids[t]], w[t], swiglu_limit=10.0, acc=np.float64) for t in range(rows)])
    assert max_rel(got, want) < TOL


def test_fused_routed_experts_reference_signature():
    import cachalot_b200 as cb
    rng = np.random.default_rng(4)
    hidden, inter = 128, 96
    experts = [configs.fp4_expert(rng, hidden, inter) for _ in range(6)]
    bank = make_bank(experts, cb.FP4_FORMAT, hidden, inter)
    x = configs.round_bf16(rng.standard_normal(hidden).astype(np.float32))
    w = np.full(6, 0.25, np.float32)
    res = [bank.expert(0, i) for i in (5, 0, 3, 1, 2, 4)]
    got = cb.fused_routed_experts(bf16_tensor(x), res, torch.from_numpy(w).cuda(), hidden_size=hidden, intermediate=inter).cpu().numpy()
    want = fp4.routed_topk_forward(x, [experts[i] for i in (5, 0, 3, 1, 2, 4)], w, acc=np.float64)
    assert max_rel(got, want) < TOL
    assert res[0].w1_weight.data_ptr() == bank.slab[5].data_ptr()       # views alias the slot
    with pytest.raises(ValueError):
        cb.fused_routed_experts(bf16_tensor(x), res, torch.from_numpy(w[:5]).cuda(), hidden_size=hidden, intermediate=inter)
    with pytest.raises(KeyError):
        bank.expert(0, 6)


def test_missing_slot_gives_zero_rows_and_leaves_the_others_alone():
    import cachalot_b200 as cb
    rng = np.random.default_rng(5)
    hidden, inter = 128, 96
    experts = [configs.fp4_expert(rng, hidden, inter) for _ in range(4)]
    bank = make_bank(experts, cb.FP4_FORMAT, hidden, inter)
    x = bf16_tensor(rng.standard_normal((1, hidden)).astype(np.float32))
    w = torch.full((1, 3), 0.3, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    full = cb.moe_forward(x, torch.tensor([[0, 1, 2]], dtype=torch.int32, device="cuda"), w, bank, status=status)
    two = cb.moe_forward(x, torch.tensor([[0, 2]], dtype=torch.int32, device="cuda"), w[:, :2], bank, status=status)
    holed = cb.moe_forward(x, torch.tensor([[0, -1, 2]], dtype=torch.int32, device="cuda"), w, bank, status=status)
    assert torch.equal(holed, two) and not torch.equal(holed, full)
    assert int(status.item()) == 0
    none = cb.moe_forward(x, torch.tensor([[-1, -1, -1]], dtype=torch.int32, device="cuda"), w, bank, status=status)
    assert float(none.abs().max()) == 0.0
    oob = cb.moe_forward(x, torch.tensor([[0, 4, 2]], dtype=torch.int32, device="cuda"), w, bank, status=status)
    assert torch.equal(oob, two) and int(status.item()) & 1


def test_config1_affine_layer_full_size():
    """2-bit g128 bank (fp16 scales/biases), sigmoid top-6 routing, batch 1, full shapes; only the
    routed experts are materialised (the rest of the 384 never enter the arithmetic)."""
    import cachalot_b200 as cb
    x, logits, _ = configs.config1(seed=0, materialise=[])
    inds, w, _ = router.route_tail(logits[0], np.zeros(384, np.float32), np.arange(384, dtype=np.int32)[None], 0, 6, 1.0, weights_bf16=False)
    ginds, gw, gslots = cb.route_tail(torch.from_numpy(logits).cuda(), None, None, 0, 6, 1.0, weights_bf16=False)
    assert ginds.cpu().numpy()[0].tolist() == inds.tolist()
    _, _, experts = configs.config1(seed=0, materialise=inds.tolist())
    fmt = cb.affine_format(4096, 2880)
    order = [int(i) for i in inds]
    bank = make_bank([experts[i] for i in order], fmt, 4096, 2880)
    slots = torch.arange(6, dtype=torch.int32, device="cuda")[None]
    got = cb.moe_forward(bf16_tensor(x), slots, gw, bank, swiglu_limit=10.0).cpu().numpy()
    want = affine.affine_routed_experts(x[0], [experts[i] for i in order], w, bits=2, group_size=128, swiglu_limit=10.0, acc=np.float64)
    assert max_rel(got[0], want) < TOL
    res = [cb.ResidentExpert(0, i, s, bank) for s, i in enumerate(order)]
    again = cb.affine_routed_experts(bf16_tensor(x)[0], res, fmt, gw[0], swiglu_limit=10.0).cpu().numpy()
    assert np.array_equal(again, got[0])


@pytest.mark.parametrize("group,dims", [(128, (256, 320)), (64, (128, 192))])
def test_affine_small_shapes_batch(group, dims):
    import cachalot_b200 as cb
    hidden, inter = dims       # 320 is 2.5 groups of 128: groups run over the flattened matrix
    rng = np.random.default_rng(20 + group)
    experts = []
    for _ in range(5):
        e = {}
        for proj, (n, kk) in (("w1", (inter, hidden)), ("w2", (hidden, inter)), ("w3", (inter, hidden))):
            lv = rng.integers(0, 4, (n, kk), dtype=np.uint8)
            e[f"{proj}.weight"] = affine.pack_bits(lv, 2)
            e[f"{proj}.scales"] = rng.uniform(0.002, 0.02, n * kk // group).astype(np.float16)
            e[f"{proj}.biases"] = (rng.standard_normal(n * kk // group) * 0.01).astype(np.float16)
        experts.append(e)
    bank = make_bank(experts, cb.affine_format(hidden, inter, 2, group), hidden, inter)
    rows, k = 4, 3
    x = configs.round_bf16(rng.standard_normal((rows, hidden)).astype(np.float32) * 3)
    ids = np.stack([rng.permutation(5)[:k] for _ in range(rows)]).astype(np.int32)
    w = rng.uniform(0.1, 0.5, (rows, k)).astype(np.float32)
    got = cb.moe_forward(bf16_tensor(x), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), bank).cpu().numpy()

    def dense(e, proj, n, kk):
        q = affine.unpack_bits(e[f"{proj}.weight"], 2, kk).astype(np.float32).reshape(-1)
        s = np.repeat(e[f"{proj}.scales"].astype(np.float32), group)
        b = np.repeat(e[f"{proj}.biases"].astype(np.float32), group)
        return (s * q + b).astype(np.float32).reshape(n, kk)

    from oracle.bf16 import round_bf16
    want = np.zeros((rows, hidden), np.float32)
    for t in range(rows):
        for j in range(k):
            e = experts[ids[t, j]]
            g = round_bf16((x[t].astype(np.float64) @ dense(e, "w1", inter, hidden).T.astype(np.float64)).astype(np.float32))
            u = round_bf16((x[t].astype(np.float64) @ dense(e, "w3", inter, hidden).T.astype(np.float64)).astype(np.float32))
            h = round_bf16((fp4.swiglu(g, u, 10.0) * w[t, j]).astype(np.float32))
            want[t] += round_bf16((h.astype(np.float64) @ dense(e, "w2", hidden, inter).T.astype(np.float64)).astype(np.float32))
    # bf16 numerics: a value on a rounding boundary may land one bf16 step (2**-8 relative) away from the float64
    # order of summation: such elements are counted and bounded by one step; all others meet 2e-3
    err = np.abs(got - want) / np.max(np.abs(want))
    assert err.max() < 2 ** -7 and np.count_nonzero(err >= TOL) <= max(2, err.size // 64)


def test_decode_full_size_properties():
    """Properties at the benchmark's shapes that need no oracle: a zero gate weight removes an expert,
    rows are independent (a row alone runs through the single-launch kernel, whose hidden operand is
    f16 per 32-element block, and in a batch through the grouped kernels: they agree to a few 1e-4),
    and a repeated call is bit-identical (fixed reduction order)."""
    import cachalot_b200 as cb
    g = torch.Generator(device="cuda").manual_seed(0)
    hidden, inter, n_slots, k = 4096, 2880, 12, 6
    bank = cb.SlabBank(cb.FP4_FORMAT, hidden, inter, n_slots)
    bank.slab.copy_(torch.randint(0, 256, bank.slab.shape, dtype=torch.uint8, device="cuda", generator=g))
    for name in ("w1.scale", "w2.scale", "w3.scale"):
        o, n = bank.offsets[name], bank.tensor_sizes[name]
        bank.slab[:, o:o + n] = torch.randint(118, 124, (n_slots, n), dtype=torch.uint8, device="cuda", generator=g)
    x = torch.randn((8, hidden), device="cuda", generator=g).to(torch.bfloat16)
    slots = torch.stack([torch.randperm(n_slots, device="cuda", generator=g)[:k] for _ in range(8)]).to(torch.int32)
    w = torch.rand((8, k), device="cuda", generator=g) * 0.3
    a = cb.moe_forward(x, slots, w, bank)
    b = cb.moe_forward(x, slots, w, bank)
    assert torch.equal(a, b) and bool(torch.isfinite(a).all())
    row3 = cb.moe_forward(x[3:4], slots[3:4], w[3:4], bank)
    assert float((row3[0] - a[3]).abs().max()) <= 5e-4 * float(a[3].abs().max())
    row3_again = cb.moe_forward(x[3:4], slots[3:4], w[3:4], bank)
    assert torch.equal(row3, row3_again)
    w0 = w.clone()
    w0[:, 2] = 0
    s_drop = slots.clone()
    s_drop[:, 2] = -1
    zero_w, dropped = cb.moe_forward(x, slots, w0, bank), cb.moe_forward(x, s_drop, w, bank)
    assert float((zero_w - dropped).abs().max()) <= 1e-5 * float(dropped.abs().max())


@pytest.mark.parametrize("kind,rows", [("fp4", 1), ("fp4", 5), ("fp4", 16), ("fp4", 80), ("affine", 1), ("affine", 7), ("affine", 64),
                                       ("affine", 72)])
def test_tensor_core_kernels_equal_simple_kernels(kind, rows):
    """The tensor-core decode kernels against the one-warp-per-output kernels on the same bank and
    routing, at the benchmark's shapes (the reference checks its fused kernels against the unfused
    loop the same way); up to 64 tokens run the single-launch kernel once per token, larger batches
    exercise the grouping of rows by expert (FP4 from eight tokens: the grouped tensor-core path)."""
    import cachalot_b200 as cb
    g = torch.Generator(device="cuda").manual_seed(rows)
    hidden, inter, n_slots, k = 4096, 2880, 40, 6
    fmt = cb.FP4_FORMAT if kind == "fp4" else cb.affine_format(hidden, inter)
    bank = cb.SlabBank(fmt, hidden, inter, n_slots)
    bank.fill_random(g)
    x = (torch.randn((rows, hidden), device="cuda", generator=g) * 2).to(torch.bfloat16)
    slots = torch.stack([torch.randperm(n_slots, device="cuda", generator=g)[:k] for _ in range(rows)]).to(torch.int32)
    if rows > 1:
        slots[1, 3] = -1
    w = torch.rand((rows, k), device="cuda", generator=g) * 0.3
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    fast = cb.moe_forward(x, slots, w, bank, status=status)
    slow = cb.moe_forward(x, slots, w, bank, simple=True)
    assert int(status.item()) == 0
    scale = float(slow.abs().max())
    # the single-launch kernel keeps the hidden operand as f16 per 32-element block, and from eight tokens up the FP4
    # bank runs on the block-scaled tensor cores with activations as four residual MXFP4 rows: a few 1e-4 either way
    assert float((fast - slow).abs().max()) / scale < (2e-3 if kind == "affine" else 5e-4)
    again = cb.moe_forward(x, slots, w, bank)
    assert torch.equal(fast, again)


@pytest.mark.parametrize("kind", ["fp4", "affine"])
@pytest.mark.parametrize("dims", [(256, 192), (512, 384), (1024, 320), (5120, 2304)])
def test_single_launch_kernel_matches_oracle(kind, dims):
    """One token through the single-launch kernel against the oracle: shapes with a partial last step
    (192, 320), the reference's own dimensions (5120 x 2304), an absent and an out-of-range slot, bf16
    output, and agreement with the two-launch kernels."""
    import cachalot_b200 as cb
    hidden, inter = dims
    rng = np.random.default_rng(hidden + inter)
    n_exp, k = 7, 6
    make = configs.fp4_expert if kind == "fp4" else configs.affine_expert
    fmt = cb.FP4_FORMAT if kind == "fp4" else cb.affine_format(hidden, inter)
    experts = [make(rng, hidden, inter) for _ in range(n_exp)]
    bank = make_bank(experts, fmt, hidden, inter)
    x = configs.round_bf16(rng.standard_normal((1, hidden)).astype(np.float32) * 3)
    ids = rng.permutation(n_exp)[:k].astype(np.int32)
    w = rng.uniform(0.05, 0.6, k).astype(np.float32)

    def oracle(sel):
        if kind == "fp4":
            return fp4.routed_topk_forward(x[0], [experts[i] for i in ids[sel]], w[sel], swiglu_limit=10.0, acc=np.float64)
        return affine.affine_routed_experts(x[0], [experts[i] for i in ids[sel]], w[sel], bits=2, group_size=128, swiglu_limit=10.0, acc=np.float64)

    def plain_affine(sel):
        """The same experts without the bf16 rounding points, accumulated in float64."""
        total = np.zeros(hidden, np.float64)
        for i, wi in zip(ids[sel], w[sel]):
            m = {p: affine.dequantize_affine(experts[i][f"{p}.weight"], experts[i][f"{p}.scales"], experts[i][f"{p}.biases"],
                                             bits=2, group_size=128).astype(np.float64) for p in ("w1", "w2", "w3")}
            g, u = m["w1"] @ x[0].astype(np.float64), m["w3"] @ x[0].astype(np.float64)
            total += m["w2"] @ (fp4.swiglu(g, u, 10.0) * float(wi))
        return total

    # With the affine op's rounding points (g, u, h and every expert's output go through bf16) two correct
    # accumulation orders can land on different sides of a rounding boundary: an output element then
    # moves by one bf16 ulp (2**-8 relative) of one expert's contribution, and two experts can do so at
    # the same element.  The arithmetic itself is held to TOL with the rounding points switched off.
    tol_op = TOL if kind == "fp4" else 2 ** -7
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    xs, ws = bf16_tensor(x), torch.from_numpy(w[None]).cuda()
    got = cb.moe_forward(xs, torch.from_numpy(ids[None]).cuda(), ws, bank, status=status).cpu().numpy()[0]
    assert int(status.item()) == 0
    want = oracle(np.arange(k))
    assert max_rel(got, want) < tol_op
    if kind == "affine":
        # ... and the elements that did move across a boundary are few, each by one bf16 step of one expert's output
        moved = int(np.count_nonzero(np.abs(got - want) >= TOL * np.max(np.abs(want))))
        print(f"affine {dims}: {moved} of {hidden} output elements on the other side of a bf16 boundary")
        assert moved <= max(2, hidden // 64)
        exact = cb.moe_forward(xs, torch.from_numpy(ids[None]).cuda(), ws, bank, numerics="f32").cpu().numpy()[0]
        assert max_rel(exact, plain_affine(np.arange(k))) < TOL
    two = cb.moe_forward(xs, torch.from_numpy(ids[None]).cuda(), ws, bank, unfused=True).cpu().numpy()[0]
    assert max_rel(got, two) < tol_op
    holed = ids.copy()
    holed[2], holed[4] = -1, n_exp + 3            # absent, and outside the bank (flagged, treated as absent)
    got_h = cb.moe_forward(xs, torch.from_numpy(holed[None]).cuda(), ws, bank, status=status).cpu().numpy()[0]
    assert int(status.item()) & 1
    assert max_rel(got_h, oracle(np.array([0, 1, 3, 5]))) < tol_op
    got_b = cb.moe_forward(xs, torch.from_numpy(ids[None]).cuda(), ws, bank, out_dtype=torch.bfloat16).float().cpu().numpy()[0]
    assert max_rel(got_b, got) < 2 ** -8


@pytest.mark.parametrize("kind", ["fp4", "affine"])
@pytest.mark.parametrize("router_mode", ["sigmoid", "sqrt_softplus"])
def test_layer_decode_one_launch_equals_route_then_experts(kind, router_mode):
    """Routing inside the expert kernel: indices equal the oracle's (bit-exact), weights and the layer output equal
    the two-step path (routing kernel, then the experts) bit for bit, including an expert that is not resident."""
    import cachalot_b200 as cb
    hidden, inter, n_exp, k = 1024, 704, 40, 6
    rng = np.random.default_rng(99)
    g = torch.Generator(device="cuda").manual_seed(5)
    fmt = cb.FP4_FORMAT if kind == "fp4" else cb.affine_format(hidden, inter)
    bank = cb.SlabBank(fmt, hidden, inter, n_exp, layers=1, n_experts=n_exp)
    bank.fill_random(g)
    logits = rng.standard_normal(n_exp).astype(np.float32)
    logits[7] = logits[3]                                   # a tie inside the candidate set
    bias = (rng.standard_normal(n_exp) * 0.1).astype(np.float32)
    x = bf16_tensor(rng.standard_normal(hidden).astype(np.float32))
    table = bank.slot_table.clone()
    scale = 1.5
    if router_mode == "sigmoid":
        want_idx, want_w, _ = router.route_tail(logits, bias, np.arange(n_exp, dtype=np.int32)[None], 0, k, scale, weights_bf16=False)
    else:
        want_idx, want_w = router.topk_from_scores_r1(router.sqrt_softplus_scores(logits, 1.0), bias, topk=k, route_scale=scale,
                                                      norm_topk_prob=True)
    table[0, int(want_idx[2])] = -1                          # the third selected expert is not resident
    lg, bs = torch.from_numpy(logits).cuda(), torch.from_numpy(bias).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, idx, w = cb.moe_layer_decode(x, lg, bank, layer=0, topk=k, bias=bs, table=table, router=router_mode, route_scale=scale,
                                      status=status, want_routing=True)
    assert int(status.item()) == 0
    assert idx.cpu().numpy().tolist() == [int(i) for i in want_idx]
    assert np.allclose(w.cpu().numpy(), want_w, rtol=2e-6, atol=0)
    # two-step path through the C ABI's routing kernel
    mode = cb.ops._lib.ROUTER_SIGMOID if router_mode == "sigmoid" else cb.ops._lib.ROUTER_SQRT_SOFTPLUS
    idx2, w2, slots2, _ = cb.ops._route(lg[None], bs, table, 0, k, mode, 1.0, scale, True, False, False)
    assert torch.equal(idx2[0], idx) and torch.equal(w2[0], w)
    two = cb.moe_forward(x[None], slots2, w2, bank)[0]
    assert torch.equal(two, out)


def test_fp4_scale_window_and_calibration():
    """Block scales far from the default centre: the grouped (two-launch) kernels hold scales relative to
    a centre in f16; `SlabBank.write_expert` keeps the centre on the bytes the bank holds, and a descriptor whose
    centre is off raises the status bit.  The single-launch kernel applies every E8M0 scale in fp32 and does not
    depend on the centre."""
    import cachalot_b200 as cb
    rng = np.random.default_rng(9)
    hidden, inter = 256, 192
    e = configs.fp4_expert(rng, hidden, inter)
    for name in ("w1.scale", "w2.scale", "w3.scale"):
        e[name] = rng.integers(90, 100, e[name].shape, dtype=np.uint8)       # 2**-37 .. 2**-28
    bank = make_bank([e], cb.FP4_FORMAT, hidden, inter)
    x = configs.round_bf16(rng.standard_normal((1, hidden)).astype(np.float32) * 1e6)
    slots = torch.zeros((1, 1), dtype=torch.int32, device="cuda")
    w = torch.ones((1, 1), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    want = _fp4_expert_out(x, e, None, 0.0)
    got = cb.moe_forward(bf16_tensor(x), slots, w, bank, swiglu_limit=0.0, status=status).cpu().numpy()
    assert int(status.item()) == 0 and max_rel(got, want) < TOL               # single launch: any scale
    assert 90 <= bank.desc.fp4_scale_centre <= 100                             # set while the expert was written
    bank.desc.fp4_scale_centre = 121                                          # a host that passes the default
    cb.moe_forward(bf16_tensor(x), slots, w, bank, swiglu_limit=0.0, status=status, unfused=True)
    assert int(status.item()) & 4                                             # centre 121 does not cover them
    assert 90 <= bank.calibrate_scale_centre() <= 100
    status.zero_()
    got = cb.moe_forward(bf16_tensor(x), slots, w, bank, swiglu_limit=0.0, status=status, unfused=True).cpu().numpy()
    assert int(status.item()) == 0
    assert max_rel(got, want) < TOL


@pytest.mark.parametrize("kind", ["fp4", "affine"])
@pytest.mark.parametrize("rows", [8, 64])
def test_config2_batches_at_full_dims_meet_the_oracle(kind, rows):
    """Batches of 8 and 64 tokens at hidden 4096 / inter 2880, tokens sharing experts (48 slots for up to 384 routed
    rows): three sampled tokens against the oracle through every kernel family -- whatever cachalot_moe_decode picks,
    the two-launch kernels that group rows by expert (`unfused`) and the one-warp-per-output kernels (`simple`).
    FP4 runs in its own numerics (fp32 throughout): 2e-3.  The 2-bit bank is held to 2e-3 with the rounding points
    off, and with them on (g, u, h and each expert's output through bf16) an output element may land on the other side
    of a bf16 rounding boundary of one expert's contribution: those elements are counted, and bounded by one step."""
    import cachalot_b200 as cb
    hidden, inter, n_slots, k = 4096, 2880, 48, 6
    g = torch.Generator(device="cuda").manual_seed(100 + rows)
    fmt = cb.FP4_FORMAT if kind == "fp4" else cb.affine_format(hidden, inter)
    bank = cb.SlabBank(fmt, hidden, inter, n_slots)
    bank.fill_random(g)
    x = torch.randn((rows, hidden), device="cuda", generator=g).to(torch.bfloat16)
    slots = torch.stack([torch.randperm(n_slots, device="cuda", generator=g)[:k] for _ in range(rows)]).to(torch.int32)
    slots[rows // 2, 4] = -1                                   # one absent expert among the sampled rows
    w = torch.rand((rows, k), device="cuda", generator=g) * 0.3 + 0.02
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    outs = {"default": cb.moe_forward(x, slots, w, bank, status=status),
            "unfused": cb.moe_forward(x, slots, w, bank, status=status, unfused=True),
            "simple": cb.moe_forward(x, slots, w, bank, status=status, simple=True)}
    exact = {name: cb.moe_forward(x, slots, w, bank, status=status, numerics="f32", **kw)
             for name, kw in (("default", {}), ("unfused", {"unfused": True}), ("simple", {"simple": True}))} if kind == "affine" else {}
    assert int(status.item()) == 0
    xh, sh, wh = x.float().cpu().numpy(), slots.cpu().numpy(), w.cpu().numpy()
    cache = {}

    def expert(slot):
        if slot not in cache:
            cache[slot] = expert_from_bank(bank, int(slot))
        return cache[slot]

    for t in (0, rows // 2, rows - 1):
        sel = [j for j in range(k) if sh[t, j] >= 0]
        ex, wt = [expert(sh[t, j]) for j in sel], wh[t, sel]
        if kind == "fp4":
            want = fp4.routed_topk_forward(xh[t], ex, wt, swiglu_limit=10.0, acc=np.float64)
            for name, o in outs.items():
                assert max_rel(o[t].cpu().numpy(), want) < TOL, (name, t)
            continue
        want = affine.affine_routed_experts(xh[t], ex, wt, bits=2, group_size=128, swiglu_limit=10.0, acc=np.float64)
        plain = affine.affine_routed_experts_plain(xh[t], ex, wt, bits=2, group_size=128, swiglu_limit=10.0)
        ref = float(np.max(np.abs(want)))
        for name, o in outs.items():
            err = np.abs(o[t].cpu().numpy().astype(np.float64) - want) / ref
            outside = int(np.count_nonzero(err >= TOL))
            print(f"{kind} rows={rows} token {t} {name}: {outside} of {hidden} elements moved across a bf16 boundary, max {err.max():.2e}")
            assert err.max() < 2 ** -7 and outside <= hidden // 64, (name, t, outside)
            assert max_rel(exact[name][t].cpu().numpy(), plain) < TOL, (name, t)


def test_self_check_passes_and_a_nan_weight_sets_its_status_bit():
    import cachalot_b200 as cb
    from cachalot_b200 import _lib
    assert cb.self_check() is True and cb.ops.FORCE_SIMPLE_KERNELS is False
    hidden, inter, n_slots, k = 4096, 2880, 8, 6
    bank = cb.SlabBank(cb.FP4_FORMAT, hidden, inter, n_slots)
    bank.fill_random(torch.Generator(device="cuda").manual_seed(1))
    for rows in (1, 8):          # the single-launch kernel, and the grouped tensor-core path
        x = torch.randn((rows, hidden), device="cuda").to(torch.bfloat16)
        slots = torch.arange(k, dtype=torch.int32, device="cuda").repeat(rows, 1)
        w = torch.full((rows, k), 0.2, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        cb.moe_forward(x, slots, w, bank, status=status)
        assert int(status.item()) == 0
        w[rows - 1, 2] = float("nan")
        cb.moe_forward(x, slots, w, bank, status=status)
        assert int(status.item()) & _lib.STATUS_BAD_WEIGHT


def test_two_streams_decode_small_banks_concurrently():
    """Small banks leave most of an SM's shared memory unused, yet the single-launch kernel always takes a whole SM per
    CTA: launches from two streams cannot overlap on the shared hidden rows, and both streams get the right answers."""
    import cachalot_b200 as cb
    hidden, inter, n_slots, k = 512, 384, 12, 6
    bank = cb.SlabBank(cb.affine_format(hidden, inter), hidden, inter, n_slots)
    bank.fill_random(torch.Generator(device="cuda").manual_seed(4))
    g = torch.Generator(device="cuda").manual_seed(5)
    xs = [torch.randn((1, hidden), device="cuda", generator=g).to(torch.bfloat16) for _ in range(2)]
    slots = [torch.randperm(n_slots, device="cuda", generator=g)[:k].to(torch.int32)[None] for _ in range(2)]
    w = torch.full((1, k), 0.15, device="cuda")
    want = [cb.moe_forward(xs[i], slots[i], w, bank, simple=True) for i in range(2)]
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    ws = [torch.empty(1 << 20, dtype=torch.uint8, device="cuda") for _ in range(2)]
    outs = [[], []]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for it in range(30):
        for i, st in enumerate(streams):
            with torch.cuda.stream(st):
                outs[i].append(cb.moe_forward(xs[i], slots[i], w, bank, workspace=ws[i], status=status))
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for i in range(2):
        scale = float(want[i].abs().max())
        for o in outs[i]:
            assert torch.equal(o, outs[i][0])
            assert float((o - want[i]).abs().max()) <= 2 ** -7 * scale


def test_float32_activations_are_rounded_to_bf16():
    """The kernels take bf16 activations: a float32 x gives exactly what its bf16 rounding gives (documented on
    `moe_forward`; the reference's op would read the float32 values unrounded)."""
    import cachalot_b200 as cb
    rng = np.random.default_rng(21)
    hidden, inter = 256, 192
    bank = make_bank([configs.fp4_expert(rng, hidden, inter)], cb.FP4_FORMAT, hidden, inter)
    x32 = torch.from_numpy(rng.standard_normal((1, hidden)).astype(np.float32)).cuda()
    slots = torch.zeros((1, 1), dtype=torch.int32, device="cuda")
    w = torch.ones((1, 1), device="cuda")
    a = cb.moe_forward(x32, slots, w, bank)
    b = cb.moe_forward(x32.to(torch.bfloat16), slots, w, bank)
    assert torch.equal(a, b)
