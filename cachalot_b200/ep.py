"""Expert parallelism over the GPUs of one box: experts of every layer are split into contiguous
blocks, one block per rank; the decode input is replicated, every rank runs the routed experts it
owns (absent ones contribute zeros through slot -1) and the partial outputs are summed.

The reference is single-device (it has no collective); this module is the build's own
multi-GPU layer.  One process per GPU, `torch.distributed` for the plumbing.
"""
from __future__ import annotations

import torch


def owner_of(expert: int, n_experts: int, world: int) -> int:
    """Rank that holds `expert`: contiguous blocks of ceil(E / world)."""
    per = -(-n_experts // world)
    return expert // per


def local_range(n_experts: int, rank: int, world: int) -> tuple[int, int]:
    per = -(-n_experts // world)
    lo = min(rank * per, n_experts)
    return lo, min(lo + per, n_experts)


def local_slot_table(layers: int, n_experts: int, rank: int, world: int) -> torch.Tensor:
    """int32 [layers, E] table for this rank's shard: owned experts map to consecutive local slots
    (layer-major), every other expert to -1, so the routing kernel hands non-owned experts to the
    decode kernel as "absent"."""
    lo, hi = local_range(n_experts, rank, world)
    n_local = hi - lo
    table = torch.full((layers, n_experts), -1, dtype=torch.int32)
    if n_local > 0:
        table[:, lo:hi] = (torch.arange(layers, dtype=torch.int32)[:, None] * n_local
                           + torch.arange(n_local, dtype=torch.int32)[None, :])
    return table


def reduce_partials(partial: torch.Tensor, group=None) -> torch.Tensor:
    """Sum of the ranks' partial outputs, delivered to every rank (the next layer needs it
    everywhere).  In place."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial


class PeerSum:
    """Sum of the ranks' partial outputs through peer memory over NVLink (`cachalot_peer_sum`): one small
    launch per rank instead of a library all-reduce.  The inboxes live in a symmetric allocation
    (`torch.distributed._symmetric_memory`), mapped into every rank of the box.  `n` = floats per partial."""

    def __init__(self, n: int, device: torch.device, group=None):
        import ctypes

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from ._lib import lib

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank, self.n = dist.get_world_size(self.group), dist.get_rank(self.group), n
        inbox = int(lib.cachalot_peer_sum_inbox_bytes(self.world, n))
        flags = int(lib.cachalot_peer_sum_flag_bytes(self.world))
        self._inbox_bytes = (inbox + 255) // 256 * 256
        self.buf = symm.empty(self._inbox_bytes + flags, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm.rendezvous(self.buf, self.group)
        torch.cuda.synchronize(device)
        dist.barrier(self.group)   # every inbox is zeroed before anyone writes into it
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        arr = ctypes.c_void_p * self.world
        self._inbox = arr(*ptrs)
        self._flags = arr(*[p + self._inbox_bytes for p in ptrs])
        self.epoch = torch.zeros(2, dtype=torch.int32, device=device)

    def __call__(self, partial: torch.Tensor, out: torch.Tensor | None = None, status: torch.Tensor | None = None) -> torch.Tensor:
        from ._lib import check, lib

        if partial.dtype != torch.float32 or partial.numel() != self.n or not partial.is_contiguous():
            raise ValueError(f"partial must be contiguous float32 with {self.n} elements")
        out = partial if out is None else out
        stream = torch.cuda.current_stream(partial.device).cuda_stream
        check(lib.cachalot_peer_sum(self._inbox, self._flags, self.world, self.rank, partial.data_ptr(), out.data_ptr(), self.n,
                                    self.epoch.data_ptr(), status.data_ptr() if status is not None else None, stream))
        return out


def ep_moe_forward(x, slot_ids, gate_weights, bank, *, group=None, **kw) -> torch.Tensor:
    """moe_forward on this rank's shard followed by the cross-rank sum."""
    from .ops import moe_forward

    return reduce_partials(moe_forward(x, slot_ids, gate_weights, bank, **kw), group)
