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


def ep_moe_forward(x, slot_ids, gate_weights, bank, *, group=None, **kw) -> torch.Tensor:
    """moe_forward on this rank's shard followed by the cross-rank sum."""
    from .ops import moe_forward

    return reduce_partials(moe_forward(x, slot_ids, gate_weights, bank, **kw), group)
