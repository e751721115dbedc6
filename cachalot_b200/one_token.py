"""Decodes a few tokens through one MoE layer on a small synthetic bank.

    python -m cachalot_b200.one_token [affine2|fp4] [calls] [tokens]

A minimal use of the package (build a bank, route nothing, call `moe_forward`) that is also the
small case the profiler is pointed at: a 120-slot bank (1.2 GB / 2.3 GB), one token (or a batch of
`tokens`), top-6, hidden 4096, inter 2880, a different random set of experts per call.  It prints the number of
distinct experts of the last call (what a batch has to stream).
"""
from __future__ import annotations

import sys


def main(kind: str = "affine2", calls: int = 5, tokens: int = 1) -> None:
    import torch

    import cachalot_b200 as cb

    hidden, inter, k, n_slots = 4096, 2880, 6, 120
    g = torch.Generator(device="cuda").manual_seed(0)
    fmt = cb.FP4_FORMAT if kind == "fp4" else cb.affine_format(hidden, inter)
    bank = cb.SlabBank(fmt, hidden, inter, n_slots)
    bank.fill_random(g)
    x = (torch.randn((tokens, hidden), device="cuda", generator=g) * 2).to(torch.bfloat16)
    w = torch.rand((tokens, k), device="cuda", generator=g) * 0.3
    out = torch.zeros((tokens, hidden), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for _ in range(calls):
        slots = torch.stack([torch.randperm(n_slots, device="cuda", generator=g)[:k] for _ in range(tokens)]).to(torch.int32).contiguous()
        cb.moe_forward(x, slots, w, bank, out=out, status=status)
    torch.cuda.synchronize()
    print("status", int(status.item()), "max |out|", float(out.abs().max()), "distinct experts in the last call", int(torch.unique(slots).numel()))


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "affine2", int(sys.argv[2]) if len(sys.argv) > 2 else 5,
         int(sys.argv[3]) if len(sys.argv) > 3 else 1)
