"""Peer-memory sum of the ranks' partial outputs: the stand-alone kernel (cachalot_peer_sum) and the exchange in the
decode kernel's tail (cachalot_moe_layer_decode_peer)."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

WAIT_EXPIRED = 8


def _call(world, rank, inbox_ptrs, flag_ptrs, partial, out, epoch, status):
    from cachalot_b200._lib import check, lib
    arr = ctypes.c_void_p * world
    check(lib.cachalot_peer_sum(arr(*inbox_ptrs), arr(*flag_ptrs), world, rank, partial.data_ptr(), out.data_ptr(),
                                partial.numel(), epoch.data_ptr(), status.data_ptr(), torch.cuda.current_stream().cuda_stream))


def _buffers(world, n):
    from cachalot_b200._lib import lib
    inbox = torch.zeros(lib.cachalot_peer_sum_inbox_bytes(world, n), dtype=torch.uint8, device="cuda")
    flags = torch.zeros(lib.cachalot_peer_sum_flag_bytes(world), dtype=torch.uint8, device="cuda")
    return inbox, flags


def test_one_rank_is_a_copy_and_replays():
    n = 4096
    inbox, flags = _buffers(1, n)
    epoch = torch.zeros(2, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for i in range(5):   # both slots, several exchanges
        partial = torch.randn(n, device="cuda")
        out = torch.empty_like(partial)
        _call(1, 0, [inbox.data_ptr()], [flags.data_ptr()], partial, out, epoch, status)
        assert torch.equal(out, partial)
    assert int(status.item()) == 0 and epoch.tolist() == [5, 0]


def test_missing_peer_makes_the_wait_expire_not_hang():
    """World of two, but nobody plays rank 1: its flags are never raised, the bounded wait gives up, the status
    word says so and the context stays usable."""
    n = 1024
    inbox0, flags0 = _buffers(2, n)
    inbox1, flags1 = _buffers(2, n)   # stands for rank 1's memory; nothing reads or signals from there
    epoch = torch.zeros(2, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    partial = torch.ones(n, device="cuda")
    out = torch.empty_like(partial)
    _call(2, 0, [inbox0.data_ptr(), inbox1.data_ptr()], [flags0.data_ptr(), flags1.data_ptr()], partial, out, epoch, status)
    torch.cuda.synchronize()
    assert int(status.item()) & WAIT_EXPIRED
    # rank 0's own row arrived; rank 1's row is still the zeros the inbox started with
    assert torch.equal(out, partial)
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0


def _two_rank_worker(rank, world, port, n, results):
    import os

    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from cachalot_b200 import ep
    ps = ep.PeerSum(n, dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    ok = True
    for i in range(6):
        part = torch.randn(n, generator=torch.Generator().manual_seed(10 * i + rank)).to(dev)
        want = part.clone()
        dist.all_reduce(want)
        got = ps(part.clone(), status=status)
        ok = ok and torch.allclose(got, want, rtol=1e-6, atol=1e-6)
    torch.cuda.synchronize(dev)
    results[rank] = bool(ok) and int(status.item()) == 0
    ok_layer = _sharded_layer_equals_whole(rank, world, dev)
    results[rank] = results[rank] and ok_layer
    ps.close()            # all ranks drop their mappings together, nothing in flight
    dist.barrier()
    torch.cuda.synchronize(dev)
    os._exit(0 if results[rank] else 1)


def _sharded_layer_equals_whole(rank, world, dev):
    """Expert-parallel decode layer with the exchange in the kernel's tail against the same layer on one whole bank."""
    import cachalot_b200 as cb
    from cachalot_b200 import ep
    hidden, inter, n_exp, k = 2048, 2816, 16, 6
    ok = True
    for kind in ("affine", "fp4"):
        fmt = cb.FP4_FORMAT if kind == "fp4" else cb.affine_format(hidden, inter)
        whole = cb.SlabBank(fmt, hidden, inter, n_exp, layers=1, n_experts=n_exp, device=dev)
        whole.fill_random(torch.Generator(device=dev).manual_seed(11))
        lo, hi = ep.local_range(n_exp, rank, world)
        shard = cb.SlabBank(fmt, hidden, inter, hi - lo, layers=1, n_experts=n_exp, device=dev)
        shard.slab.copy_(whole.slab[lo:hi])
        table = ep.local_slot_table(1, n_exp, rank, world).to(dev)
        peer = ep.PeerLayer(hidden, dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        g = torch.Generator().manual_seed(5)
        for i in range(5):
            x = torch.randn(hidden, generator=g).to(torch.bfloat16).to(dev)
            logits = torch.randn(n_exp, generator=g).to(dev)
            got = cb.moe_layer_decode(x, logits, shard, table=table, router="sigmoid", peer=peer, status=status)
            want = cb.moe_layer_decode(x, logits, whole, router="sigmoid")
            # the sharded sum adds the ranks' partial sums in rank order, the whole bank adds experts in routing order
            ok = ok and float((got - want).abs().max()) <= 2e-3 * float(want.abs().max())
        torch.cuda.synchronize(dev)
        ok = ok and int(status.item()) == 0
        peer.close()
    return ok


def _small_layer(kind="affine"):
    import cachalot_b200 as cb
    hidden, inter, n_exp = 2048, 2816, 16
    fmt = cb.FP4_FORMAT if kind == "fp4" else cb.affine_format(hidden, inter)
    bank = cb.SlabBank(fmt, hidden, inter, n_exp, layers=1, n_experts=n_exp)
    bank.fill_random(torch.Generator(device="cuda").manual_seed(2))
    return bank, hidden, n_exp


@pytest.mark.parametrize("kind", ["affine", "fp4"])
def test_layer_exchange_with_one_rank_equals_the_plain_layer(kind):
    """The exchange in the decode kernel's tail with a world of one (rows go through the inbox in local memory):
    bit-identical to the plain layer call, over both inbox slots, also inside a replayed CUDA graph."""
    import cachalot_b200 as cb
    from cachalot_b200 import ep
    bank, hidden, n_exp = _small_layer(kind)
    peer = ep.PeerLayer(hidden, torch.device("cuda"))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    g = torch.Generator().manual_seed(9)
    for i in range(5):
        x = torch.randn(hidden, generator=g).to(torch.bfloat16).cuda()
        logits = torch.randn(n_exp, generator=g).cuda()
        got = cb.moe_layer_decode(x, logits, bank, router="sigmoid", peer=peer, status=status)
        want = cb.moe_layer_decode(x, logits, bank, router="sigmoid")
        assert torch.equal(got, want)
    assert int(status.item()) == 0 and peer.epoch.tolist() == [5, 0]
    out = torch.empty(hidden, device="cuda")
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        cb.moe_layer_decode(x, logits, bank, router="sigmoid", peer=peer, status=status, out=out)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(3):
                cb.moe_layer_decode(x, logits, bank, router="sigmoid", peer=peer, status=status, out=out)
        graph.replay()
        graph.replay()
        stream.synchronize()
    assert torch.equal(out, want) and peer.epoch.tolist() == [12, 0] and int(status.item()) == 0


def test_layer_exchange_missing_peer_expires_not_hangs():
    """World of two, nobody plays rank 1: the bounded wait in the kernel's tail gives up, the status word says so,
    this rank's own partial sum is what comes out and the context stays usable."""
    import cachalot_b200 as cb
    from cachalot_b200 import ep
    from cachalot_b200._lib import lib
    bank, hidden, n_exp = _small_layer()
    peer = ep.PeerLayer(hidden, torch.device("cuda"))
    other = torch.zeros(int(lib.cachalot_peer_layer_inbox_bytes(2, hidden)) + 256,
                        dtype=torch.uint8, device="cuda")   # stands for rank 1's memory; nobody writes from there
    mine = torch.zeros_like(other)
    for r, buf in enumerate((mine, other)):
        peer.ctx.inbox[r] = buf.data_ptr()
    peer.ctx.world, peer.ctx.rank = 2, 0
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    g = torch.Generator().manual_seed(9)
    x = torch.randn(hidden, generator=g).to(torch.bfloat16).cuda()
    logits = torch.randn(n_exp, generator=g).cuda()
    got = cb.moe_layer_decode(x, logits, bank, router="sigmoid", peer=peer, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) & WAIT_EXPIRED
    assert torch.equal(got, cb.moe_layer_decode(x, logits, bank, router="sigmoid"))
    assert float(torch.ones(4, device="cuda").sum().item()) == 4.0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_match_nccl():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    procs = [ctx.Process(target=_two_rank_worker, args=(r, 2, 29611, 4096, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    assert all(p.exitcode == 0 for p in procs) and all(results.get(r) for r in range(2))
