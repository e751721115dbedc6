"""Shared helpers for the GPU parity tests."""
from __future__ import annotations

import numpy as np


def max_rel(got: np.ndarray, want: np.ndarray) -> float:
    """max|got - want| / max|want| -- the reference's own error metric (benchmarks/micro_gemv_kernels.py:38)."""
    return float(np.max(np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))) / max(np.max(np.abs(want)), 1e-30))


def within_bf16_flips(got: np.ndarray, want: np.ndarray, tol: float = 2e-3, share: float = 1 / 32) -> bool:
    """The criterion for outputs that pass through bf16 rounding points when the inputs of those roundings carry a
    small error (the tensor-core path takes a bf16 activation as four MXFP4 terms, good to 2.4e-4): a value that sat
    on a rounding boundary moves one bf16 step.  Every element within `tol` of the largest output, except a counted
    share that may be off by one bf16 step of the largest output (2**-7)."""
    scale = float(np.max(np.abs(want)))
    err = np.abs(np.asarray(got, dtype=np.float64) - np.asarray(want, dtype=np.float64)) / scale
    return bool(err.max() < 2.0 ** -7 and np.count_nonzero(err >= tol) <= max(2, int(err.size * share)))


def bf16_tensor(x_f32: np.ndarray, device="cuda"):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x_f32, dtype=np.float32)).to(device).to(torch.bfloat16)


def make_bank(experts: list[dict], fmt, hidden, inter, device="cuda"):
    """Bank whose slot i holds experts[i] (dicts of numpy arrays named like the format's tensors)."""
    from cachalot_b200 import SlabBank

    bank = SlabBank(fmt, hidden, inter, len(experts), device=device)
    for i, e in enumerate(experts):
        bank.write_expert(i, e)
    return bank


def expert_from_bank(bank, slot: int) -> dict:
    """The bytes of one slot as the dict of numpy arrays the oracle takes (typed and shaped like the format)."""
    out = {}
    for name in bank.fmt.tensor_names:
        t = bank.typed_view(slot, name).cpu()
        if t.dtype.is_floating_point and t.dtype != __import__("torch").float16:
            out[name] = t.view(__import__("torch").int16).numpy().view(np.uint16)   # bf16 bit patterns
        else:
            out[name] = t.numpy()
        if name.endswith("weight") and bank.fmt.kind == "affine":
            out[name] = out[name].view(np.uint32)
    return out


def check_prefill_rows(bank, expert_of_slot, xt, ids_t, w_t, *, n_experts, k, sample=None, tol=2e-3, max_exempt=0.25):
    """Runs the rows-level prefill (grouping, MXFP4 quantiser, the two grouped GEMMs) and checks routed rows against
    the oracle with element-wise admissible deviations (oracle.prefill.fp4_expert_rows_bounds): every checked row
    must pass unless one of its blocks sits on a scale boundary; the exempted share is bounded.  `expert_of_slot(e)`
    returns the oracle's dict of expert e.  `sample`: positions in the grouped order to check (default all).
    Returns (y, perm, offsets, inv) for further use by the caller."""
    import torch

    import cachalot_b200 as cb
    from oracle import prefill

    tokens = ids_t.shape[0]
    perm, offsets = cb.group_rows(ids_t, n_experts)
    codes, scales = cb.quantize_mxfp4(xt, perm // k)
    row_w = w_t.reshape(-1)[perm.long()]
    status = torch.zeros(1, dtype=torch.int32, device=xt.device)
    y = cb.moe_prefill_rows(codes, scales, row_w, offsets, bank.slot_table[0], bank, status=status)
    assert int(status.item()) == 0
    inv = torch.full((tokens * k,), -1, dtype=torch.int32, device=xt.device)
    inv[perm.long()] = torch.arange(tokens * k, dtype=torch.int32, device=xt.device)
    off = offsets.cpu().numpy()
    perm_h = perm.cpu().numpy()
    x_h = xt.float().cpu().numpy()
    w_h = w_t.reshape(-1).cpu().numpy()
    pos = np.arange(tokens * k) if sample is None else np.asarray(sorted(set(int(p) for p in sample)))
    table = bank.slot_table[0].cpu().numpy()
    n_checked = n_exempt = 0
    for e in range(n_experts):
        mine = pos[(pos >= off[e]) & (pos < off[e + 1])]
        if mine.size == 0:
            continue
        got = y[torch.from_numpy(mine).to(xt.device)].float().cpu().numpy()
        if table[e] < 0:
            assert float(np.abs(got).max()) == 0.0
            continue
        m = expert_of_slot(e)
        rows = perm_h[mine]
        b = prefill.fp4_expert_rows_bounds(x_h[rows // k], m["w1.weight"], m["w1.scale"], m["w2.weight"], m["w2.scale"],
                                           m["w3.weight"], m["w3.scale"], w_h[rows])
        ok, exempt, worst = prefill.check_rows_against_bounds(got, b, tol)
        bad = ~ok & ~exempt
        assert not bad.any(), f"expert {e}: grouped rows {mine[bad].tolist()} outside the bound (worst excess {worst:.3e} of max|y|)"
        n_checked += mine.size
        n_exempt += int((exempt & ~ok).sum())
    print(f"prefill rows checked {n_checked}, exempted on a scale boundary {n_exempt}")
    assert n_checked > 0 and n_exempt <= max_exempt * n_checked
    return y, perm, offsets, inv
