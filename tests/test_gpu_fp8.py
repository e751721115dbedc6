"""GPU parity: FP8 E4M3 act_quant (bit-exact) and the trunk GEMV (2e-3)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
from oracle import configs, fp8  # noqa: E402
from oracle.bf16 import round_bf16  # noqa: E402
from tests.helpers import bf16_tensor, max_rel  # noqa: E402

TOL = 2e-3


def _cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_act_quant_golden_block32(golden):
    import cachalot_b200 as cb
    x = round_bf16(golden["fp8_act_x"])
    q = cb.quantize_fp8_activation(bf16_tensor(x))
    codes, scales = fp8.quantize_activation_fp8(x, 32, "e8m0")
    assert np.array_equal(q.scales.cpu().numpy(), scales)
    assert np.array_equal(q.values.cpu().numpy(), codes)
    assert q.in_features == x.size


@pytest.mark.parametrize("block,rule", [(32, "e8m0"), (128, "e8m0"), (128, "f32"), (32, "f32")])
def test_act_quant_bit_exact_random_rows(block, rule):
    import cachalot_b200 as cb
    rng = np.random.default_rng(block)
    x = rng.standard_normal((32, 4096)).astype(np.float32)
    x[3] *= 1e-6          # below the amax floor
    x[4] *= 1e4
    x[5, :128] = 0.0
    x[6] = np.round(x[6] * 8) / 8 * 56.0   # many exact ties after scaling
    x = round_bf16(x)
    q = cb.quantize_fp8_activation(bf16_tensor(x), block, rule)
    codes, scales = fp8.quantize_activation_fp8(x, block, rule)
    assert np.array_equal(q.scales.cpu().numpy(), scales)
    assert np.array_equal(q.values.cpu().numpy(), codes)


def test_e4m3_decode_table_and_nan_codes_read_as_zero():
    """GEMV of the identity-like activation against every weight byte recovers the decode table."""
    import cachalot_b200 as cb
    k = 256
    w = np.zeros((256, k), np.uint8)
    w[:, 0] = np.arange(256, dtype=np.uint8)
    ws = np.full((8, 8), 127, np.uint8)
    x = np.zeros(k, np.float32)
    x[0] = 256.0          # scale 1, code for 256.0
    got = cb.fp8_linear(bf16_tensor(x), _cuda(w), _cuda(ws), out_dtype=torch.float32).cpu().numpy()
    assert np.array_equal(got, fp8.E4M3_DECODE * np.float32(256.0))
    assert got[0x7F] == 0.0 and got[0xFF] == 0.0


def test_gemv_golden_block32(golden):
    import cachalot_b200 as cb
    for tag in ("a", "b"):
        x = round_bf16(golden[f"fp8_{tag}_x"])
        got = cb.fp8_linear(bf16_tensor(x), _cuda(golden[f"fp8_{tag}_w"]), _cuda(golden[f"fp8_{tag}_ws"]),
                            out_dtype=torch.float32).cpu().numpy()
        want = fp8.fp8_linear(x, golden[f"fp8_{tag}_w"], golden[f"fp8_{tag}_ws"])
        assert max_rel(got, want) < 1e-5, tag
        got16 = cb.fp8_linear(bf16_tensor(x), _cuda(golden[f"fp8_{tag}_w"]), _cuda(golden[f"fp8_{tag}_ws"])).float().cpu().numpy()
        assert got16.dtype == np.float32 and max_rel(got16, want) < 2 ** -8


@pytest.mark.parametrize("batch", [1, 32])
def test_config4_trunk_matrices_full_size(batch):
    """[12288,4096] and [4096,8192], fp32 scales per 128x128, activations per 1x128 = amax/448."""
    import cachalot_b200 as cb
    for x, w, s in configs.config4(seed=0, batch=batch):
        got = cb.fp8_linear(bf16_tensor(x), _cuda(w), _cuda(s), out_dtype=torch.float32).cpu().numpy()
        want = fp8.fp8_linear(x, w, s, block_size=128, scale_rule="f32")
        assert max_rel(got, want) < TOL
        got16 = cb.fp8_linear(bf16_tensor(x), _cuda(w), _cuda(s)).float().cpu().numpy()
        assert max_rel(got16, want) < 2 ** -8 + TOL


def test_shared_activation_two_projections_equal_one_fused():
    """One act_quant shared by two GEMVs equals the GEMV over the row-concatenated weight
    (the reference's w1||w3 and wq_a||wkv fusions are bit-identical to the separate calls)."""
    import cachalot_b200 as cb
    rng = np.random.default_rng(7)
    w1, s1 = configs.fp8_matrix(rng, 256, 512, 32, "e8m0")
    w3, s3 = configs.fp8_matrix(rng, 256, 512, 32, "e8m0")
    x = bf16_tensor(rng.standard_normal(512).astype(np.float32))
    q = cb.quantize_fp8_activation(x)
    a = cb.fp8_linear_quantized(q, _cuda(w1), _cuda(s1))
    b = cb.fp8_linear_quantized(q, _cuda(w3), _cuda(s3))
    both = cb.fp8_linear_quantized(q, _cuda(np.concatenate([w1, w3])), _cuda(np.concatenate([s1, s3])))
    assert torch.equal(torch.cat([a, b]), both)


def test_fp8_errors():
    import cachalot_b200 as cb
    x = torch.zeros(96, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="divisible"):
        cb.quantize_fp8_activation(x[:48])
    q = cb.quantize_fp8_activation(x)
    with pytest.raises(ValueError, match="weight expects"):
        cb.fp8_linear_quantized(q, torch.zeros((32, 64), dtype=torch.uint8, device="cuda"), torch.zeros((1, 2), dtype=torch.uint8, device="cuda"))
    with pytest.raises(ValueError, match="scale shape"):
        cb.fp8_linear_quantized(q, torch.zeros((32, 96), dtype=torch.uint8, device="cuda"), torch.zeros((2, 3), dtype=torch.uint8, device="cuda"))
    with pytest.raises(ValueError, match="must be 2D"):
        cb.fp8_linear_quantized(q, torch.zeros(96, dtype=torch.uint8, device="cuda"), torch.zeros((1, 3), dtype=torch.uint8, device="cuda"))


@pytest.mark.parametrize("n,k,block,rule,rows", [(64, 4096, 128, "f32", 1), (200, 8192, 128, "f32", 3), (96, 2880, 32, "e8m0", 8),
                                                 (40, 5120, 32, "e8m0", 1)])
def test_streaming_gemv_shapes_and_nan_codes(n, k, block, rule, rows):
    """The ring-fed GEMV (up to eight tokens, rows of at least 1 KB): a partial last tile, K cut into several stages,
    a K that is not a multiple of 128 bytes, and NaN codes (0x7F / 0xFF) scattered over the weights, which read as
    zero -- against the oracle on the same bytes with those codes replaced by zero."""
    import cachalot_b200 as cb
    rng = np.random.default_rng(n + k)
    w, ws = configs.fp8_matrix(rng, n, k, block, rule)
    w = w.copy()
    hit = rng.integers(0, n * k, 50)
    w.reshape(-1)[hit] = np.where(rng.integers(0, 2, 50) == 0, 0x7F, 0xFF).astype(np.uint8)
    clean = np.where((w & 0x7F) == 0x7F, 0, w).astype(np.uint8)
    x = round_bf16(rng.standard_normal((rows, k)).astype(np.float32))
    got = cb.fp8_linear(bf16_tensor(x), _cuda(w), _cuda(ws), out_dtype=torch.float32).cpu().numpy()
    want = fp8.fp8_linear(x, clean, ws, block_size=block, scale_rule=rule)
    assert np.isfinite(got).all() and max_rel(got, want) < TOL
    q = cb.quantize_fp8_activation(bf16_tensor(x), block, rule)
    two = cb.fp8_linear_quantized(q, _cuda(w), _cuda(ws), out_dtype=torch.float32).cpu().numpy()
    assert np.array_equal(two, got)
