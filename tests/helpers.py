"""Shared helpers for the GPU parity tests."""
from __future__ import annotations

import numpy as np


def max_rel(got: np.ndarray, want: np.ndarray) -> float:
    """max|got - want| / max|want| -- the reference's own error metric (benchmarks/micro_gemv_kernels.py:38)."""
    return float(np.max(np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))) / max(np.max(np.abs(want)), 1e-30))


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
