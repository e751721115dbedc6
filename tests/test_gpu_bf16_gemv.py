"""GPU parity: the bf16-weight fp32 GEMV (output head) against its oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import bf16_gemv  # noqa: E402


def _case(n, k, rows, seed):
    rng = np.random.default_rng(seed)
    w = torch.from_numpy(rng.standard_normal((n, k)).astype(np.float32) * 0.05).to(torch.bfloat16)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    bits = w.view(torch.int16).numpy().view(np.uint16)
    return w, x, bits


@pytest.mark.parametrize("n,k,rows", [(64, 64, 1), (1000, 320, 1), (777, 5120, 3), (4099, 1024, 8), (33, 192, 2)])
def test_bf16_gemv_matches_oracle(n, k, rows):
    import cachalot_b200 as cb
    w, x, bits = _case(n, k, rows, n + k)
    got = cb.bf16_gemv_f32(torch.from_numpy(x).cuda(), w.cuda()).cpu().numpy()
    want, bound = bf16_gemv.bf16_gemv_f32(x, bits), bf16_gemv.bf16_gemv_bound(x, bits)
    assert got.shape == (rows, n)
    assert np.all(np.abs(got - want) <= bound + 1e-30)


def test_head_sized_gemv_and_one_dimensional_x():
    """The reference's head: 129,280 x 5,120 bf16 (1.3 GB), x [K] -> [N]."""
    import cachalot_b200 as cb
    n, k = 129280, 5120
    g = torch.Generator(device="cuda").manual_seed(5)
    w = (torch.randn((n, k), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(k, device="cuda", generator=g)
    got = cb.bf16_gemv_f32(x, w)
    assert got.shape == (n,) and got.dtype == torch.float32
    want = (w[::997].double() @ x.double()).float()       # sampled rows against a float64 product
    assert float((got[::997] - want).abs().max()) <= 1e-5 * float(want.abs().max())
    assert cb.bf16_gemv_f32(x.to(torch.bfloat16), w).dtype == torch.float32               # any float x is widened to fp32


def test_bf16_gemv_argument_errors():
    import cachalot_b200 as cb
    w = torch.zeros((8, 64), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="2D bfloat16"):
        cb.bf16_gemv_f32(torch.zeros(64, device="cuda"), w.float())
    with pytest.raises(ValueError, match="multiple of 64"):
        cb.bf16_gemv_f32(torch.zeros(96, device="cuda"), torch.zeros((8, 96), dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(ValueError, match="features"):
        cb.bf16_gemv_f32(torch.zeros(128, device="cuda"), w)
