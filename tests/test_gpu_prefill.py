"""GPU parity: expert-major grouping (bit-exact), MXFP4 activation quant (bit-exact), prefill FFN."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import configs, mxfp4, prefill  # noqa: E402
from oracle.bf16 import round_bf16  # noqa: E402
from tests.helpers import within_bf16_flips, bf16_tensor, check_prefill_rows, expert_from_bank, make_bank, max_rel  # noqa: E402

TOL = 2e-3


def test_group_rows_bit_exact_config3_routing():
    import cachalot_b200 as cb
    rng = np.random.default_rng(0)
    ids, _ = configs.zipf_routing(rng, 4096, 384, 6)
    perm, off = cb.group_rows(torch.from_numpy(ids).cuda(), 384)
    operm, ooff = prefill.group_rows(ids, 384)
    assert np.array_equal(off.cpu().numpy(), ooff)
    assert np.array_equal(perm.cpu().numpy(), operm)


def test_group_rows_edges():
    import cachalot_b200 as cb
    # an expert with no rows, one expert taking everything, ragged tail, out-of-range ids dropped
    ids = np.array([[3, 3], [3, 3], [3, 0]], dtype=np.int32)
    perm, off = cb.group_rows(torch.from_numpy(ids).cuda(), 5)
    assert off.cpu().numpy().tolist() == [0, 1, 1, 1, 6, 6]
    assert perm.cpu().numpy().tolist() == [5, 0, 1, 2, 3, 4]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    bad = np.array([[1, 7], [-2, 0]], dtype=np.int32)
    perm, off = cb.group_rows(torch.from_numpy(bad).cuda(), 4, status)
    assert off.cpu().numpy().tolist() == [0, 1, 2, 2, 2]
    assert perm.cpu().numpy()[:2].tolist() == [3, 0] and int(status.item()) & 2
    perm, off = cb.group_rows(torch.zeros((0, 6), dtype=torch.int32, device="cuda"), 4)
    assert off.cpu().numpy().tolist() == [0] * 5 and perm.numel() == 0


def test_mxfp4_act_quant_bit_exact():
    import cachalot_b200 as cb
    rng = np.random.default_rng(1)
    x = rng.standard_normal((64, 4096)).astype(np.float32)
    x[1] *= 1e-30
    x[2] *= 1e20
    x[3, :64] = 0.0
    x[4] = np.round(x[4] * 4) / 4          # lands on E2M1 midpoints
    x[5, ::2] *= -1
    x = round_bf16(x)
    codes, scales = cb.quantize_mxfp4(bf16_tensor(x))
    oc, os_ = mxfp4.quantize_mxfp4(x)
    assert np.array_equal(scales.cpu().numpy(), os_)
    from oracle.fp4 import pack_codes
    assert np.array_equal(codes.cpu().numpy(), pack_codes(oc))
    # gathered rows
    src = torch.tensor([5, 5, 0, 63], dtype=torch.int32, device="cuda")
    c2, s2 = cb.quantize_mxfp4(bf16_tensor(x), src)
    assert np.array_equal(c2.cpu().numpy(), pack_codes(oc)[[5, 5, 0, 63]])
    assert np.array_equal(s2.cpu().numpy(), os_[[5, 5, 0, 63]])


@pytest.mark.parametrize("mx", [False, True])
def test_prefill_small_matches_oracle(mx):
    import cachalot_b200 as cb
    tokens, hidden, inter, n_exp, k = 48, 256, 192, 16, 6
    x, ids, w, experts = configs.config3(seed=2, tokens=tokens, hidden=hidden, inter=inter, n_experts=n_exp, k=k,
                                         materialise=range(n_exp))
    bank = make_bank([experts[e] for e in range(n_exp)], cb.FP4_FORMAT, hidden, inter)
    got = cb.moe_prefill_grouped(bf16_tensor(x), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), bank,
                                 swiglu_limit=10.0, mxfp4_act=mx).cpu().numpy()
    want = prefill.moe_prefill_fp4(x, ids, w, lambda e: experts[e], n_experts=n_exp, swiglu_limit=10.0,
                                   act="mxfp4" if mx else "bf16", acc=np.float64)
    if not mx:
        # bf16 activations run on the tensor cores as four residual MXFP4 terms (2.4e-4 of the activation), so a g, u,
        # h or y that sat on a bf16 rounding boundary may move one step: counted and bounded; the per-row kernels, which
        # take the bf16 values as they are, meet the plain tolerance
        assert within_bf16_flips(got, want, TOL)
        xt, it, wt = bf16_tensor(x), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
        exact = cb.moe_forward(xt, it, wt, bank, numerics="bf16", simple=True).cpu().numpy()
        assert max_rel(exact, want) < TOL
        return
    # The MXFP4 quantiser of the hidden activation is discontinuous, so the comparison is made per routed row with
    # the deviation each element's own boundary cases admit (an element of g or u within rounding noise of a bf16
    # midpoint, an element of h within it of an E2M1 threshold); everything else must meet the tolerance.
    xt, it, wt = bf16_tensor(x), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    y, perm, offsets, inv = check_prefill_rows(bank, lambda e: experts[e], xt, it, wt, n_experts=n_exp, k=k, tol=TOL)
    # the whole call is the slot-ordered sum of exactly those rows
    assert torch.equal(cb.combine_rows(y, inv, tokens, k), torch.from_numpy(got).cuda())


def test_prefill_equals_decode_row_by_row():
    """Expert-major execution keeps decode's per-token result: slot-ordered sum of the same experts."""
    import cachalot_b200 as cb
    tokens, hidden, inter, n_exp, k = 32, 256, 192, 16, 6
    x, ids, w, experts = configs.config3(seed=3, tokens=tokens, hidden=hidden, inter=inter, n_experts=n_exp, k=k,
                                         materialise=range(n_exp))
    bank = make_bank([experts[e] for e in range(n_exp)], cb.FP4_FORMAT, hidden, inter)
    xt, it, wt = bf16_tensor(x), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    pre = cb.moe_prefill_grouped(xt, it, wt, bank)
    fast = cb.moe_forward(xt, it, wt, bank, numerics="bf16")
    assert torch.equal(pre, fast)          # the same kernels, rows grouped by expert either way
    # the one-warp-per-output kernels take the bf16 activations as they are; the tensor-core path takes them as four
    # MXFP4 terms, so a value on a bf16 rounding boundary may move one step
    dec = cb.moe_forward(xt, it, wt, bank, numerics="bf16", simple=True)
    assert within_bf16_flips(pre.cpu().numpy(), dec.cpu().numpy())


@pytest.mark.parametrize("tokens,hidden,inter,n_exp", [(48, 256, 192, 16), (300, 512, 320, 12), (64, 1024, 2880 // 5, 40), (8, 256, 192, 40)])
def test_prefill_tensor_core_path_matches_oracle_row_by_row(tokens, hidden, inter, n_exp):
    """mxfp4_act=1 (block-scaled FP4 MMAs, weights as the M side) against the oracle, every routed row, with an absent
    expert; the last case has more experts than routed rows (a short chunk of layer-major prefill).  The per-row
    kernels (mxfp4_act=2: the same arithmetic in a fixed summation order) must agree with the same sum to the bound
    that rounding-boundary cases allow."""
    import cachalot_b200 as cb
    k = 6
    x, ids, w, experts = configs.config3(seed=5, tokens=tokens, hidden=hidden, inter=inter, n_experts=n_exp, k=k,
                                         materialise=range(n_exp))
    bank = make_bank([experts[e] for e in range(n_exp)], cb.FP4_FORMAT, hidden, inter)
    bank.slot_table[0, 3] = -1  # an absent expert contributes zeros on both paths
    xt, it, wt = bf16_tensor(x), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    y, perm, offsets, inv = check_prefill_rows(bank, lambda e: experts[e], xt, it, wt, n_experts=n_exp, k=k, tol=TOL)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tc = cb.moe_prefill_grouped(xt, it, wt, bank, mxfp4_act=1, status=status)
    assert int(status.item()) == 0
    assert torch.equal(tc, cb.combine_rows(y, inv, tokens, k))
    plain = cb.moe_prefill_grouped(xt, it, wt, bank, mxfp4_act=2)
    err = (tc - plain).abs().amax(dim=1) / plain.abs().max()
    assert float(err.max()) < 5e-2   # a cross-check only: the rows above are held to the oracle


def test_prefill_rows_and_combine_equal_the_whole_call():
    """The two halves an expert-parallel rank runs (rows-level GEMMs, slot-ordered combine) reproduce
    cachalot_moe_prefill bit for bit when fed the same grouping, also with an absent expert."""
    import cachalot_b200 as cb
    tokens, hidden, inter, n_exp, k = 200, 512, 320, 10, 6
    x, ids, w, experts = configs.config3(seed=8, tokens=tokens, hidden=hidden, inter=inter, n_experts=n_exp, k=k,
                                         materialise=range(n_exp))
    bank = make_bank([experts[e] for e in range(n_exp)], cb.FP4_FORMAT, hidden, inter)
    bank.slot_table[0, 2] = -1
    xt, it, wt = bf16_tensor(x), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    whole = cb.moe_prefill_grouped(xt, it, wt, bank, mxfp4_act=1)
    perm, offsets = cb.group_rows(it, n_exp)
    codes, scales = cb.quantize_mxfp4(xt, perm // k)
    row_w = wt.reshape(-1)[perm.long()]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = cb.moe_prefill_rows(codes, scales, row_w, offsets, bank.slot_table[0], bank, status=status)
    inv = torch.empty(tokens * k, dtype=torch.int32, device="cuda")
    inv[perm.long()] = torch.arange(tokens * k, dtype=torch.int32, device="cuda")
    got = cb.combine_rows(y, inv, tokens, k)
    assert int(status.item()) == 0
    assert torch.equal(got, whole)
    lo, hi = int(offsets[2]), int(offsets[3])
    assert hi > lo and float(y[lo:hi].abs().max()) == 0.0


def _ep_prefill_worker(rank, world, port, results):
    import os

    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import cachalot_b200 as cb
    from cachalot_b200 import ep
    tokens, hidden, inter, n_exp, k = 256, 512, 320, 10, 6
    x, ids, w, experts = configs.config3(seed=9, tokens=tokens, hidden=hidden, inter=inter, n_experts=n_exp, k=k,
                                         materialise=range(n_exp))
    full = make_bank([experts[e] for e in range(n_exp)], cb.FP4_FORMAT, hidden, inter, device=dev)
    lo, hi = ep.local_range(n_exp, rank, world)
    shard = make_bank([experts[e] for e in range(lo, hi)], cb.FP4_FORMAT, hidden, inter, device=dev)
    shard.slot_table = ep.local_slot_table(1, n_exp, rank, world).to(dev)
    mine = slice(rank * tokens // world, (rank + 1) * tokens // world)
    xt, it, wt = bf16_tensor(x[mine]).to(dev), torch.from_numpy(ids[mine]).to(dev), torch.from_numpy(w[mine]).to(dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    got = ep.ep_moe_prefill(xt, it, wt, shard, n_experts=n_exp, status=status)
    want = cb.moe_prefill_grouped(xt, it, wt, full, mxfp4_act=1)
    torch.cuda.synchronize(dev)
    results[rank] = bool(torch.equal(got, want)) and int(status.item()) == 0
    os._exit(0 if results[rank] else 1)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_expert_parallel_prefill_on_two_gpus_equals_one_gpu():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_ep_prefill_worker, args=(r, 2, 29621, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
    assert all(p.exitcode == 0 for p in procs) and all(results.get(r) for r in range(2))


def test_prefill_tensor_core_path_at_full_layer_dims():
    """hidden 4096, inter 2880 (partial last 128-row tile, K tail of the down projection, scale rows of 90 bytes):
    routed rows against the oracle, sampled where the tiling has its edges: the first and last row of every expert
    and both sides of every 96-row unit boundary (one expert has more rows than a unit holds)."""
    import cachalot_b200 as cb
    tokens, hidden, inter, n_exp, k = 160, 4096, 2880, 8, 6
    rng = np.random.default_rng(11)
    bank = cb.SlabBank(cb.FP4_FORMAT, hidden, inter, n_exp)
    bank.fill_random(torch.Generator(device="cuda").manual_seed(3))
    x = bf16_tensor(round_bf16(rng.standard_normal((tokens, hidden)).astype(np.float32)))
    ids = np.stack([rng.permutation(n_exp)[:k] for _ in range(tokens)]).astype(np.int32)   # ~120 rows per expert
    w = rng.uniform(0.05, 0.3, (tokens, k)).astype(np.float32)
    it, wt = torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    counts = np.bincount(ids.reshape(-1), minlength=n_exp)
    starts = np.concatenate([[0], np.cumsum(counts)])
    sample = []
    for e in range(n_exp):
        sample += [starts[e], starts[e + 1] - 1]
        sample += [starts[e] + p for p in (95, 96, 97) if p < counts[e]]
        sample += [starts[e] + int(p) for p in rng.integers(0, counts[e], 2)]
    y, perm, offsets, inv = check_prefill_rows(bank, lambda e: expert_from_bank(bank, e), x, it, wt, n_experts=n_exp, k=k,
                                               sample=sample, tol=TOL)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tc = cb.moe_prefill_grouped(x, it, wt, bank, mxfp4_act=1, status=status)
    assert int(status.item()) == 0
    assert torch.equal(tc, cb.combine_rows(y, inv, tokens, k))
    plain = cb.moe_prefill_grouped(x, it, wt, bank, mxfp4_act=2)
    err = (tc - plain).abs().amax(dim=1) / plain.abs().max()
    assert float(err.max()) < 5e-2


def test_config3_full_size_sampled_rows_match_oracle():
    """Config 3 itself: 4096 tokens, 384 experts, Zipf(1.1) popularity, hidden 4096, inter 2880.  The whole call
    equals the slot-ordered sum of the rows-level outputs bit for bit, and sampled routed rows (all six rows of
    four tokens; the edges of the heaviest expert's 96-row units; the lightest experts) meet the oracle."""
    import cachalot_b200 as cb
    tokens, hidden, inter, n_exp, k = 4096, 4096, 2880, 384, 6
    rng = np.random.default_rng(0)
    ids, w = configs.zipf_routing(rng, tokens, n_exp, k)
    x = bf16_tensor(round_bf16(rng.standard_normal((tokens, hidden)).astype(np.float32)))
    bank = cb.SlabBank(cb.FP4_FORMAT, hidden, inter, n_exp)
    bank.fill_random(torch.Generator(device="cuda").manual_seed(7))
    it, wt = torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    flat = ids.reshape(-1)
    counts = np.bincount(flat, minlength=n_exp)
    starts = np.concatenate([[0], np.cumsum(counts)])
    order = np.argsort(flat, kind="stable")
    where = np.empty_like(order)
    where[order] = np.arange(order.size)             # grouped position of routed row (token*k + slot)
    sample = [int(where[t * k + j]) for t in (0, 1777, 4095) for j in range(k)]
    heavy = int(np.argmax(counts))
    sample += [int(starts[heavy] + p) for p in (0, 95, 96, 191, 192, counts[heavy] - 1)]
    for e in np.argsort(counts)[:3]:
        if counts[e]:
            sample.append(int(starts[e]))
    y, perm, offsets, inv = check_prefill_rows(bank, lambda e: expert_from_bank(bank, e), x, it, wt, n_experts=n_exp, k=k,
                                               sample=sample, tol=TOL)
    assert np.array_equal(perm.cpu().numpy(), order)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    whole = cb.moe_prefill_grouped(x, it, wt, bank, mxfp4_act=1, status=status)
    assert int(status.item()) == 0
    assert torch.equal(whole, cb.combine_rows(y, inv, tokens, k))


@pytest.mark.parametrize("case", ["one_token", "one_expert_many_rows", "all_absent", "k1", "empty"])
def test_prefill_tensor_core_path_edges(case):
    """Ragged and degenerate groupings through the block-scaled MMAs: a single token, every row on one expert
    (several 96-row units of the same weights), no expert resident (zeros), top-1 routing, an empty chunk."""
    import cachalot_b200 as cb
    hidden, inter, n_exp = 256, 192, 6
    rng = np.random.default_rng(31)
    experts = [configs.fp4_expert(rng, hidden, inter) for _ in range(n_exp)]
    bank = make_bank(experts, cb.FP4_FORMAT, hidden, inter)
    tokens, k = {"one_token": (1, 3), "one_expert_many_rows": (250, 2), "all_absent": (9, 3), "k1": (40, 1), "empty": (0, 3)}[case]
    x = round_bf16(rng.standard_normal((tokens, hidden)).astype(np.float32))
    ids = np.stack([rng.permutation(n_exp)[:k] for _ in range(tokens)]).astype(np.int32) if tokens else np.zeros((0, k), np.int32)
    if case == "one_expert_many_rows":
        ids[:, 0] = 4
        ids[:, 1] = np.where(ids[:, 1] == 4, 5, ids[:, 1])
    if case == "all_absent":
        bank.slot_table[0, :] = -1
    w = rng.uniform(0.1, 0.5, (tokens, k)).astype(np.float32)
    xt, it, wt = bf16_tensor(x), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    tc = cb.moe_prefill_grouped(xt, it, wt, bank, mxfp4_act=1, status=status)
    assert int(status.item()) == 0 and tuple(tc.shape) == (tokens, hidden)
    if case == "empty":
        return
    plain = cb.moe_prefill_grouped(xt, it, wt, bank, mxfp4_act=2)
    if case == "all_absent":
        assert float(tc.abs().max()) == 0.0 and float(plain.abs().max()) == 0.0
        return
    err = (tc - plain).abs().amax(dim=1) / plain.abs().max()
    assert float(err.max()) < 5e-2
    y, perm, offsets, inv = check_prefill_rows(bank, lambda e: experts[e], xt, it, wt, n_experts=n_exp, k=k, tol=TOL, max_exempt=0.5)
    assert torch.equal(tc, cb.combine_rows(y, inv, tokens, k))


def test_prefill_over_a_two_bit_bank_matches_oracle():
    """model/expert_affine.py:84-99 through the grouped prefill entry: a 2-bit g128 bank, the affine op's rounding points
    (g, u, h and each expert's output through bf16), results summed in slot order."""
    import cachalot_b200 as cb
    from oracle import affine
    tokens, hidden, inter, n_exp, k = 20, 256, 384, 6, 3
    rng = np.random.default_rng(41)
    experts = [configs.affine_expert(rng, hidden, inter) for _ in range(n_exp)]
    bank = make_bank(experts, cb.affine_format(hidden, inter), hidden, inter)
    bank.slot_table[0, 4] = -1
    x = round_bf16(rng.standard_normal((tokens, hidden)).astype(np.float32))
    ids = np.stack([rng.permutation(n_exp)[:k] for _ in range(tokens)]).astype(np.int32)
    w = rng.uniform(0.1, 0.5, (tokens, k)).astype(np.float32)
    got = cb.moe_prefill_grouped(bf16_tensor(x), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), bank).cpu().numpy()
    want = np.zeros((tokens, hidden), np.float32)
    for t in range(tokens):
        for j in range(k):
            if ids[t, j] == 4:
                continue
            want[t] += affine.affine_expert_forward(x[t], experts[ids[t, j]], bits=2, group_size=128, weight=w[t, j], swiglu_limit=10.0,
                                                    acc=np.float64)
    err = np.abs(got - want) / np.max(np.abs(want))
    assert err.max() < 2 ** -7 and np.count_nonzero(err >= TOL) <= max(2, err.size // 64)


def test_prefill_bf16_activations_on_tensor_cores_at_full_dims():
    """The reference's per-expert prefill numerics (bf16 activations; g, u, h, y rounded to bf16) on the block-scaled
    tensor cores at hidden 4096 / inter 2880: whole tokens against the oracle (activations as four residual MXFP4
    terms, so a value on a bf16 rounding boundary may move one step), and against the one-warp-per-output kernels,
    which take the activations as they are."""
    import cachalot_b200 as cb
    tokens, hidden, inter, n_exp, k = 96, 4096, 2880, 12, 6
    rng = np.random.default_rng(17)
    bank = cb.SlabBank(cb.FP4_FORMAT, hidden, inter, n_exp)
    bank.fill_random(torch.Generator(device="cuda").manual_seed(5))
    x = round_bf16(rng.standard_normal((tokens, hidden)).astype(np.float32))
    ids = np.stack([rng.permutation(n_exp)[:k] for _ in range(tokens)]).astype(np.int32)
    w = rng.uniform(0.05, 0.3, (tokens, k)).astype(np.float32)
    xt, it, wt = bf16_tensor(x), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = cb.moe_prefill_grouped(xt, it, wt, bank, mxfp4_act=0, status=status)
    assert int(status.item()) == 0
    plain = cb.moe_forward(xt, it, wt, bank, numerics="bf16", simple=True)
    assert within_bf16_flips(got.cpu().numpy(), plain.cpu().numpy(), TOL)
    sample = [0, 41, 95]
    want = prefill.moe_prefill_fp4(x[sample], ids[sample], w[sample], lambda e: expert_from_bank(bank, e), n_experts=n_exp,
                                   swiglu_limit=10.0, act="bf16", acc=np.float64)
    assert within_bf16_flips(got[sample].cpu().numpy(), want, TOL)
    assert max_rel(plain[sample].cpu().numpy(), want) < TOL


def test_batched_expert_entry_runs_on_tensor_cores_and_meets_the_oracle():
    """`routed_expert_forward_batched` (one FP4 expert over a batch of rows, model/moe_prefill_batched.py:31-61) at
    64 rows: from eight rows up it goes through the grouped block-scaled kernels."""
    import cachalot_b200 as cb
    rng = np.random.default_rng(23)
    hidden, inter, m = 512, 384, 64
    e = configs.fp4_expert(rng, hidden, inter)
    x = round_bf16(rng.standard_normal((m, hidden)).astype(np.float32))
    w = rng.uniform(0.1, 1.0, m).astype(np.float32)
    got = cb.routed_expert_forward_batched(bf16_tensor(x), w1_packed=torch.from_numpy(e["w1.weight"]).cuda(), w1_scales=torch.from_numpy(e["w1.scale"]).cuda(),
                                           w2_packed=torch.from_numpy(e["w2.weight"]).cuda(), w2_scales=torch.from_numpy(e["w2.scale"]).cuda(),
                                           w3_packed=torch.from_numpy(e["w3.weight"]).cuda(), w3_scales=torch.from_numpy(e["w3.scale"]).cuda(),
                                           weights=torch.from_numpy(w).cuda(), swiglu_limit=10.0).cpu().numpy()
    want = prefill.fp4_expert_rows(x, e["w1.weight"], e["w1.scale"], e["w2.weight"], e["w2.scale"], e["w3.weight"], e["w3.scale"], w,
                                   swiglu_limit=10.0, act="bf16", acc=np.float64)
    assert within_bf16_flips(got, want, TOL)
