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
        from ._lib import lib

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank, self.n = dist.get_world_size(self.group), dist.get_rank(self.group), n
        inbox = int(lib.cachalot_peer_sum_inbox_bytes(self.world, n))
        flags = int(lib.cachalot_peer_sum_flag_bytes(self.world))
        self._inbox_bytes = (inbox + 255) // 256 * 256
        self.buf, self.handle, ptrs = _symmetric_buffer(self._inbox_bytes + flags, device, self.group)
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

    def close(self):
        """Drop the mapping together with the peers: call on every rank, with no exchange in flight."""
        import torch.distributed as dist

        torch.cuda.synchronize(self.buf.device)
        dist.barrier(self.group)
        self.handle = None
        self.buf = None


def _symmetric_buffer(nbytes: int, device, group):
    """A zeroed uint8 buffer every rank of the group can write, and every rank's pointer to it in this process.
    No multicast object is wanted for it (the kernels use plain peer stores), so the switch that makes
    torch bind one is turned off before the rendezvous."""
    import os

    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm

    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
    buf.zero_()
    handle = symm.rendezvous(buf, group)
    torch.cuda.synchronize(device)
    dist.barrier(group)   # every buffer is zeroed before anyone writes into it
    return buf, handle, [int(p) for p in handle.buffer_ptrs]


class PeerLayer:
    """Peer memory for `moe_layer_decode(..., peer=...)`: the cross-rank sum of an expert-parallel decode layer done
    in the tail of the expert kernel (`cachalot_moe_layer_decode_peer`).  With `group=None` and no process group it
    is a one-rank exchange in local memory (the same code path, for single-GPU checks)."""

    def __init__(self, hidden: int, device: torch.device, group=None):
        import torch.distributed as dist

        from ._lib import PeerCtx, lib

        if dist.is_available() and dist.is_initialized():
            self.group = group if group is not None else dist.group.WORLD
            self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        else:
            self.group, self.world, self.rank = None, 1, 0
        inbox = (int(lib.cachalot_peer_layer_inbox_bytes(self.world, hidden)) + 255) // 256 * 256
        if self.world > 1:
            self.buf, self.handle, ptrs = _symmetric_buffer(inbox, device, self.group)
        else:
            self.buf = torch.zeros(inbox, dtype=torch.uint8, device=device)
            ptrs = [self.buf.data_ptr()]
        self.epoch = torch.zeros(2, dtype=torch.int32, device=device)
        ctx = PeerCtx()
        for r, p in enumerate(ptrs):
            ctx.inbox[r] = p
        ctx.epoch, ctx.world, ctx.rank = self.epoch.data_ptr(), self.world, self.rank
        self.ctx, self.hidden = ctx, hidden

    def close(self):
        """Drop the mapping together with the peers: call on every rank, with no exchange in flight."""
        import torch.distributed as dist

        torch.cuda.synchronize(self.buf.device)
        if self.world > 1:
            dist.barrier(self.group)
        self.handle = None
        self.buf = None


def ep_moe_forward(x, slot_ids, gate_weights, bank, *, group=None, **kw) -> torch.Tensor:
    """moe_forward on this rank's shard followed by the cross-rank sum."""
    from .ops import moe_forward

    return reduce_partials(moe_forward(x, slot_ids, gate_weights, bank, **kw), group)


class ExchangeError(RuntimeError):
    """A collective of the expert-parallel exchange did not complete (a peer left, or the group's timeout ran out).
    The ranks that are still there get this instead of a result; nothing of the step's output is valid."""


def _all_to_all_rows(send: torch.Tensor, send_rows: list[int], recv_rows: list[int], group) -> torch.Tensor:
    """Variable all-to-all over the leading dimension: block d of `send` (send_rows[d] rows) goes to rank d."""
    import torch.distributed as dist

    recv = torch.empty((sum(recv_rows), *send.shape[1:]), dtype=send.dtype, device=send.device)
    try:
        dist.all_to_all_single(recv, send.contiguous(), output_split_sizes=recv_rows, input_split_sizes=send_rows, group=group)
    except Exception as exc:  # torch raises backend-specific types (DistBackendError, RuntimeError, ...)
        raise ExchangeError(f"expert-parallel exchange failed: {type(exc).__name__}: {exc}") from exc
    return recv


def ep_moe_prefill(x: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, bank, *, n_experts: int, layer: int = 0,
                   swiglu_limit: float = 10.0, group=None, status: torch.Tensor | None = None, backend=None) -> torch.Tensor:
    """Expert-parallel prefill of this rank's tokens: x bf16 [T_local,H], expert_ids int32 [T_local,k] (global
    ids), weights float32 [T_local,k]; `bank` is this rank's shard whose slot table maps a global expert id to
    a local slot (-1 for experts of other ranks).  Returns float32 [T_local,H].

    Rows are grouped by global expert, quantised to MXFP4 (codes + scale bytes: 0.53 bytes per element cross
    NVLink instead of 2), dispatched to the owners of their experts with one variable all-to-all of packed records
    (codes, scale bytes and the row's router weight), run through
    the grouped FP4 GEMMs there, sent back as bf16 rows and summed per token in route-slot order -- the same
    arithmetic and the same order as `moe_prefill_grouped(mxfp4_act=1)` on one GPU.

    `backend` supplies group_rows / quantize_mxfp4 / moe_prefill_rows / combine_rows (default: this
    package's CUDA operators; the CPU tests of the exchange pass stand-ins)."""
    import torch.distributed as dist

    if backend is None:
        from . import ops as backend
    group = group if group is not None else dist.group.WORLD
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    per = -(-n_experts // world)
    t, k = expert_ids.shape
    dev = x.device

    perm, offsets = backend.group_rows(expert_ids, n_experts, status)
    n_grouped = t * k
    src_token = torch.div(perm, k, rounding_mode="floor")
    codes, scales = backend.quantize_mxfp4(x, src_token)
    row_w = weights.to(torch.float32).reshape(-1)[perm.long()]

    counts = torch.zeros(world * per, dtype=torch.int64, device=dev)
    counts[:n_experts] = (offsets[1:] - offsets[:-1]).to(torch.int64)
    send_counts = counts.view(world, per)
    recv_counts = torch.empty_like(send_counts)
    try:
        dist.all_to_all_single(recv_counts, send_counts.contiguous(), group=group)
    except Exception as exc:
        raise ExchangeError(f"expert-parallel exchange failed: {type(exc).__name__}: {exc}") from exc
    send_rows = send_counts.sum(1).tolist()   # host sync: the collective needs the split sizes
    recv_rows = recv_counts.sum(1).tolist()
    kept = sum(send_rows)                      # rows with an expert id in range (the others were dropped by the grouping)

    # one record per row -- codes, scale bytes, router weight -- so that one collective carries the dispatch
    nc, ns = codes.shape[1], scales.shape[1]
    record = torch.empty((kept, nc + ns + 4), dtype=torch.uint8, device=dev)
    record[:, :nc] = codes[:kept]
    record[:, nc:nc + ns] = scales[:kept]
    record[:, nc + ns:] = row_w[:kept].contiguous().view(torch.uint8).reshape(kept, 4)
    arrived = _all_to_all_rows(record, send_rows, recv_rows, group)
    r_codes = arrived[:, :nc].contiguous()
    r_scales = arrived[:, nc:nc + ns].contiguous()
    r_w = arrived[:, nc + ns:].contiguous().view(torch.float32).reshape(-1)

    # what arrived is ordered by source rank, then by local expert: one segment per (source, expert)
    seg_offsets = torch.zeros(world * per + 1, dtype=torch.int32, device=dev)
    seg_offsets[1:] = torch.cumsum(recv_counts.reshape(-1), 0).to(torch.int32)
    lo = rank * per
    local = torch.full((per,), -1, dtype=torch.int32, device=dev)
    n_own = max(0, min(per, n_experts - lo))
    if n_own:
        local[:n_own] = bank.slot_table[layer, lo:lo + n_own].to(device=dev, dtype=torch.int32)
    seg_slots = local.repeat(world)
    y = backend.moe_prefill_rows(r_codes, r_scales, r_w, seg_offsets, seg_slots, bank, swiglu_limit=swiglu_limit, status=status)

    y_home = _all_to_all_rows(y, recv_rows, send_rows, group)
    inv = torch.full((n_grouped,), -1, dtype=torch.int32, device=dev)
    inv[perm[:kept].long()] = torch.arange(kept, dtype=torch.int32, device=dev)
    return backend.combine_rows(y_home, inv, t, k)
