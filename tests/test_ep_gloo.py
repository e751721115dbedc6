"""Expert-parallel host logic on CPU: two gloo ranks, each with its shard's slot table; the summed
partial outputs (the oracle stands in for the per-rank compute) equal the unsharded result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cachalot_b200 import ep


def test_slot_table_partition_covers_every_expert_once():
    for world in (1, 2, 4, 8):
        tables = [ep.local_slot_table(3, 384, r, world) for r in range(world)]
        owned = torch.stack([(t >= 0) for t in tables]).sum(0)
        assert bool((owned == 1).all())
        for r, t in enumerate(tables):
            lo, hi = ep.local_range(384, r, world)
            assert hi - lo == 384 // world
            assert sorted(t[t >= 0].tolist()) == list(range(3 * (hi - lo)))
            assert all(ep.owner_of(e, 384, world) == r for e in range(lo, hi))
    # ragged split
    t = [ep.local_slot_table(1, 10, r, 4) for r in range(4)]
    assert [int((x >= 0).sum()) for x in t] == [3, 3, 3, 1]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import configs, fp4, router

        hidden, inter, n_exp, k = 64, 96, 8, 3
        rng = np.random.default_rng(0)           # same stream on every rank: replicated inputs
        experts = [configs.fp4_expert(rng, hidden, inter) for _ in range(n_exp)]
        x = configs.round_bf16(rng.standard_normal(hidden).astype(np.float32))
        logits = rng.standard_normal(n_exp).astype(np.float32)
        table = ep.local_slot_table(1, n_exp, rank, world).numpy()
        inds, w, slots = router.route_tail(logits, np.zeros(n_exp, np.float32), table, 0, k, 1.0, weights_bf16=False)
        lo, _ = ep.local_range(n_exp, rank, world)
        partial = np.zeros(hidden, np.float32)
        for e, wi, s in zip(inds, w, slots):
            if s < 0:
                continue                           # not owned: zero contribution
            assert int(e) - lo == int(s)
            m = experts[int(e)]
            partial += fp4.expert_forward(x, m["w1.weight"], m["w1.scale"], m["w2.weight"], m["w2.scale"],
                                          m["w3.weight"], m["w3.scale"], weight=wi)
        total = ep.reduce_partials(torch.from_numpy(partial)).numpy()
        want = fp4.routed_topk_forward(x, [experts[int(e)] for e in inds], w)
        q.put((rank, float(np.max(np.abs(total - want)) / np.max(np.abs(want)))))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_rank_partial_sum_equals_unsharded():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=100) for _ in procs]
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert sorted(r for r, _ in res) == [0, 1]
    assert all(err < 1e-5 for _, err in res)


class _OracleBackend:
    """CPU stand-ins for the four operators `ep_moe_prefill` calls, built on the numpy oracle."""

    def __init__(self, experts, hidden):
        self.experts, self.hidden = experts, hidden

    def group_rows(self, ids, n_experts, status=None):
        from oracle import prefill
        flat = ids.numpy().reshape(-1)
        keep = np.flatnonzero((flat >= 0) & (flat < n_experts))          # ids out of range are dropped, like the CUDA op
        perm, offsets = prefill.group_rows(flat[keep].reshape(-1, 1), n_experts)
        full = np.full(flat.size, 0, np.int32)
        full[:keep.size] = keep[perm]
        return torch.from_numpy(full), torch.from_numpy(offsets)

    def quantize_mxfp4(self, x, src_rows):
        from oracle import mxfp4
        from oracle.fp4 import pack_codes
        codes, scales = mxfp4.quantize_mxfp4(x.float().numpy()[src_rows.numpy()])
        return torch.from_numpy(pack_codes(codes)), torch.from_numpy(scales)

    def moe_prefill_rows(self, codes, scales, row_w, seg_offsets, seg_slots, bank, *, swiglu_limit, status=None):
        from oracle import mxfp4, prefill
        c = codes.numpy()
        nib = np.stack([c & 15, c >> 4], axis=-1).reshape(c.shape[0], -1)
        x = mxfp4.dequantize_mxfp4(nib, scales.numpy())
        y = np.zeros((c.shape[0], self.hidden), np.float32)
        off = seg_offsets.numpy()
        for g, slot in enumerate(seg_slots.numpy()):
            a, b = int(off[g]), int(off[g + 1])
            if b == a or slot < 0:
                continue
            m = bank[int(slot)]
            y[a:b] = prefill.fp4_expert_rows(x[a:b], m["w1.weight"], m["w1.scale"], m["w2.weight"], m["w2.scale"], m["w3.weight"],
                                             m["w3.scale"], row_w.numpy()[a:b], swiglu_limit=swiglu_limit, act="mxfp4", acc=np.float64)
        return torch.from_numpy(y).to(torch.bfloat16)

    def combine_rows(self, y, inv, tokens, k):
        yy, iv = y.float().numpy(), inv.numpy().reshape(tokens, k)
        out = np.zeros((tokens, yy.shape[1]), np.float32)
        for j in range(k):
            ok = iv[:, j] >= 0
            out[ok] += yy[iv[ok, j]]
        return torch.from_numpy(out)


class _Shard:
    """Just enough of a bank for ep_moe_prefill: a slot table and the shard's experts by local slot."""

    def __init__(self, experts, rank, world):
        n = len(experts)
        self.slot_table = ep.local_slot_table(1, n, rank, world)
        lo, hi = ep.local_range(n, rank, world)
        self._local = experts[lo:hi]

    def __getitem__(self, slot):
        return self._local[slot]


def _prefill_worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import configs, prefill

        hidden, inter, n_exp, k, tokens = 64, 64, 5, 3, 24      # 5 experts over 2 ranks: ragged split (3 + 2)
        x, ids, w, experts = configs.config3(seed=4, tokens=tokens, hidden=hidden, inter=inter, n_experts=n_exp, k=k,
                                             materialise=range(n_exp))
        experts = [experts[e] for e in range(n_exp)]
        ids = ids.copy()
        ids[1, 0] = n_exp + 3                                    # an id out of range is dropped, not an error
        mine = slice(rank * tokens // world, (rank + 1) * tokens // world)
        got = ep.ep_moe_prefill(torch.from_numpy(x[mine]).to(torch.bfloat16), torch.from_numpy(ids[mine]), torch.from_numpy(w[mine]),
                                _Shard(experts, rank, world), n_experts=n_exp, backend=_OracleBackend(experts, hidden)).numpy()
        ids_ok = np.where(ids < n_exp, ids, 0)
        w_ok = np.where(ids < n_exp, w, 0.0).astype(np.float32)   # a dropped row contributes nothing
        want = prefill.moe_prefill_fp4(x, ids_ok, w_ok, lambda e: experts[e], n_experts=n_exp, swiglu_limit=10.0, act="mxfp4",
                                       acc=np.float64)[mine]
        q.put((rank, float(np.max(np.abs(got - want)) / np.max(np.abs(want)))))
    except Exception as exc:  # report instead of leaving the parent to time out
        q.put((rank, f"{type(exc).__name__}: {exc}"))
        raise
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_two_rank_prefill_exchange_equals_unsharded():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_prefill_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=150) for _ in procs]
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0
    assert sorted(r for r, _ in res) == [0, 1]
    assert all(isinstance(err, float) and err < 2e-3 for _, err in res), res


def _report_and_exit(q, item):
    q.put(item)
    q.close()
    q.join_thread()      # the message is on its way before the process goes
    os._exit(0)


def _leaver_worker(rank, world, port, q):
    """Both ranks do one exchange; then rank 1 leaves between the steps and rank 0 tries the next one."""
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from oracle import configs

    hidden, inter, n_exp, k, tokens = 64, 64, 4, 2, 8
    x, ids, w, experts = configs.config3(seed=6, tokens=tokens, hidden=hidden, inter=inter, n_experts=n_exp, k=k, materialise=range(n_exp))
    experts = [experts[e] for e in range(n_exp)]
    mine = slice(rank * tokens // world, (rank + 1) * tokens // world)
    args = (torch.from_numpy(x[mine]).to(torch.bfloat16), torch.from_numpy(ids[mine]), torch.from_numpy(w[mine]), _Shard(experts, rank, world))
    kw = dict(n_experts=n_exp, backend=_OracleBackend(experts, hidden))
    first = ep.ep_moe_prefill(*args, **kw)
    dist.barrier()                      # the step is over on both ranks: nothing is in flight
    if rank == 1:
        _report_and_exit(q, (1, "left"))  # a rank that is gone: no goodbye, no destroy_process_group
    try:
        ep.ep_moe_prefill(*args, **kw)
        msg = "no error"
    except ep.ExchangeError as exc:
        msg = f"ExchangeError {tuple(first.shape)} {str(exc)[:60]}"
    except Exception as exc:          # anything else is a finding too
        msg = f"other {type(exc).__name__}"
    _report_and_exit(q, (0, msg))


@pytest.mark.timeout(120)
def test_a_rank_that_leaves_between_steps_gives_the_survivor_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leaver_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=90) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert res[1] == "left"
    assert res[0].startswith("ExchangeError"), res
