"""Host-side failure handling that needs no GPU: the routing validator and the self-check's fall-back switch."""
import pytest
import torch


def test_validate_routing_rejects_malformed_routing():
    from cachalot_b200 import ops

    ids = torch.tensor([[3, 1, 0], [2, 5, 4]], dtype=torch.int32)
    w = torch.full((2, 3), 1 / 3)
    ops.validate_routing(ids, w, 6)
    with pytest.raises(ValueError, match="outside"):
        ops.validate_routing(ids, w, 5)                      # id 5 with five experts
    bad = ids.clone()
    bad[0, 1] = -1
    with pytest.raises(ValueError, match="outside"):
        ops.validate_routing(bad, w, 6)
    ops.validate_routing(bad, w, 6, allow_absent=True)       # -1 = not resident is legal on the slot path
    dup = ids.clone()
    dup[1, 2] = 2
    with pytest.raises(ValueError, match="twice"):
        ops.validate_routing(dup, w, 6)
    nan = w.clone()
    nan[1, 0] = float("nan")
    with pytest.raises(ValueError, match="weight"):
        ops.validate_routing(ids, nan, 6)
    inf = w.clone()
    inf[0, 2] = float("inf")
    with pytest.raises(ValueError, match="weight"):
        ops.validate_routing(ids, inf, 6)
    with pytest.raises(ValueError, match="tokens, k"):
        ops.validate_routing(ids, w[:, :2], 6)


def test_self_check_switches_to_the_simple_kernels_on_a_mismatch(monkeypatch):
    from cachalot_b200 import ops

    monkeypatch.setattr(ops, "_self_check_done", {})
    monkeypatch.setattr(ops, "FORCE_SIMPLE_KERNELS", False)
    good = torch.ones(8)
    assert ops.self_check("fake:0", _run=lambda kind: (good, good.clone())) is True
    assert ops.FORCE_SIMPLE_KERNELS is False
    assert ops.self_check("fake:0", _run=lambda kind: (good * 2, good)) is True      # once per device: cached
    off = good.clone()
    off[3] = 1.5
    assert ops.self_check("fake:1", _run=lambda kind: (off, good)) is False
    assert ops.FORCE_SIMPLE_KERNELS is True
    nan = good.clone()
    nan[0] = float("nan")
    monkeypatch.setattr(ops, "FORCE_SIMPLE_KERNELS", False)
    assert ops.self_check("fake:2", _run=lambda kind: (nan, good)) is False and ops.FORCE_SIMPLE_KERNELS is True


def test_fp4_bank_tracks_its_scale_window_on_the_host():
    """`write_expert` re-centres the descriptor on the E8M0 bytes written so far, ignores byte 0 (a zero block) and
    refuses a bank wider than the 28 binades the grouped kernels can hold."""
    import numpy as np
    import torch

    import cachalot_b200 as cb
    hidden, inter = 64, 32
    bank = cb.SlabBank(cb.FP4_FORMAT, hidden, inter, 2, device="cpu")

    def expert(lo, hi, zero=False):
        rng = np.random.default_rng(lo)
        t = {}
        for proj, (n, k) in (("w1", (inter, hidden)), ("w3", (inter, hidden)), ("w2", (hidden, inter))):
            t[f"{proj}.weight"] = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
            sc = rng.integers(lo, hi + 1, (n, k // 32), dtype=np.uint8)
            sc.flat[0], sc.flat[1] = lo, hi
            if zero:
                sc.flat[2] = 0
            t[f"{proj}.scale"] = sc
        return t

    bank.write_expert(0, expert(100, 110, zero=True))
    assert bank.desc.fp4_scale_centre == 105
    bank.write_expert(1, expert(112, 120))
    assert bank.desc.fp4_scale_centre == 110
    with pytest.raises(NotImplementedError):
        bank.write_expert(1, expert(90, 130))
