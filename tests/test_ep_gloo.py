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
