"""Peer-memory sum of the ranks' partial outputs (cachalot_peer_sum)."""
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
    os._exit(0 if results[rank] else 1)


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
