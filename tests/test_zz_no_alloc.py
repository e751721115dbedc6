"""GPU check of cachalot_moe_decode_static, the decode entry point that brings its own scratch.

Some hosts of this library cannot give the decode op a workspace: their memory pool has taken all
of HBM, so a cudaMalloc would fail or stall every stream of the device; or the call site they plug
into has no parameter for scratch.  For them the library carries a fixed 4 MiB scratch array.  The
test calls the entry point through the C ABI twice in a row (different tokens, different experts,
so anything left over from the first call would show) and compares each result with
cachalot_moe_decode run on a caller-owned workspace.  The file name sorts last on purpose: the
test runs after every other GPU test, and it must also pass alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import configs  # noqa: E402
from tests.helpers import bf16_tensor, make_bank, max_rel  # noqa: E402

TOL = 2e-3  # the decode tests' bound on max relative error; both paths run the same kernels


def _decode_both_ways(bank, x, slots, w, numerics):
    from cachalot_b200 import _lib

    lib = _lib.lib
    rows, k = slots.shape
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out_static = torch.full((rows, bank.hidden), float("nan"), dtype=torch.float32, device="cuda")
    rc = lib.cachalot_moe_decode_static(bank.slab.data_ptr(), bank.desc_ptr, x.data_ptr(), slots.data_ptr(), w.data_ptr(), rows, k,
                                        10.0, numerics, out_static.data_ptr(), _lib.F32, status.data_ptr(), stream)
    assert rc == _lib.OK, _lib.last_error()
    need = lib.cachalot_moe_decode_workspace_bytes(bank.desc_ptr, rows, k)
    ws = torch.empty(need + 256, dtype=torch.uint8, device="cuda")
    base = (ws.data_ptr() + 255) // 256 * 256
    out_ws = torch.full((rows, bank.hidden), float("nan"), dtype=torch.float32, device="cuda")
    rc = lib.cachalot_moe_decode(bank.slab.data_ptr(), bank.desc_ptr, x.data_ptr(), slots.data_ptr(), w.data_ptr(), rows, k,
                                 10.0, numerics, base, need, out_ws.data_ptr(), _lib.F32, status.data_ptr(), stream)
    assert rc == _lib.OK, _lib.last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    return out_static.cpu().numpy(), out_ws.cpu().numpy()


@pytest.mark.parametrize("kind", ["fp4", "affine"])
def test_static_scratch_decode_matches_workspace_decode_twice(kind):
    import cachalot_b200 as cb
    from cachalot_b200 import _lib

    rng = np.random.default_rng(77)
    hidden, inter, n_exp, k = 512, 384, 10, 6
    if kind == "fp4":
        fmt, make, numerics = cb.FP4_FORMAT, configs.fp4_expert, _lib.NUMERICS_F32
    else:
        fmt, make, numerics = cb.affine_format(hidden, inter), configs.affine_expert, _lib.NUMERICS_BF16
    bank = make_bank([make(rng, hidden, inter) for _ in range(n_exp)], fmt, hidden, inter)
    for rows in (1, 3):  # two calls in a row on the shared scratch, the second larger than the first
        x = bf16_tensor(rng.standard_normal((rows, hidden)).astype(np.float32))
        slots = torch.from_numpy(np.stack([rng.permutation(n_exp)[:k] for _ in range(rows)]).astype(np.int32)).cuda()
        w = torch.from_numpy(rng.uniform(0.05, 0.5, (rows, k)).astype(np.float32)).cuda()
        got, want = _decode_both_ways(bank, x, slots, w, numerics)
        assert np.isfinite(got).all()
        assert max_rel(got, want) < TOL


def test_static_scratch_rejects_what_does_not_fit():
    import cachalot_b200 as cb
    from cachalot_b200 import _lib

    lib = _lib.lib
    limit = lib.cachalot_moe_decode_static_scratch_bytes()
    assert limit == 4 << 20
    bank = cb.SlabBank(cb.FP4_FORMAT, 4096, 2880, 1)
    rows, k = 64, 6
    assert lib.cachalot_moe_decode_workspace_bytes(bank.desc_ptr, rows, k) > limit
    x = torch.zeros((rows, 4096), dtype=torch.bfloat16, device="cuda")
    slots = torch.zeros((rows, k), dtype=torch.int32, device="cuda")
    w = torch.zeros((rows, k), dtype=torch.float32, device="cuda")
    out = torch.zeros((rows, 4096), dtype=torch.float32, device="cuda")
    rc = lib.cachalot_moe_decode_static(bank.slab.data_ptr(), bank.desc_ptr, x.data_ptr(), slots.data_ptr(), w.data_ptr(), rows, k,
                                        10.0, _lib.NUMERICS_F32, out.data_ptr(), _lib.F32, None, torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.ESCRATCH
    assert "built-in scratch" in _lib.last_error()
