"""The CPU oracle against outputs of the reference's own numpy modules (tests/golden)."""
import numpy as np

from oracle import fp4, fp8


def test_fp4_table_and_e8m0(golden):
    assert np.array_equal(fp4.E2M1_VALUES, golden["fp4_table"])
    # -0.0 vs 0.0 for code 8: both compare equal; check the sign explicitly
    assert not np.signbit(fp4.E2M1_VALUES[8])
    got = fp4.e8m0_to_f32(golden["e8m0_raw"])
    # byte 254 (2**127): numpy's float32 exp2 returns a value one ulp above the power of two on
    # this platform; the oracle keeps the exact power of two, as the reference's kernels do
    assert np.array_equal(got[:254], golden["e8m0_f32"][:254])
    assert got[254] == np.float32(2.0 ** 127)


def test_fp4_dequant_bit_exact(golden):
    got = fp4.dequantize_fp4_weight(golden["fp4_packed"], golden["fp4_scales"])
    want = golden["fp4_dequant"]
    assert got.dtype == np.float32 and got.shape == want.shape
    assert np.array_equal(got.view(np.uint32) & 0x7FFFFFFF, want.view(np.uint32) & 0x7FFFFFFF)
    assert np.array_equal(got, want)


def test_fp4_gemv_matches_reference_recipe(golden):
    w = fp4.dequantize_fp4_weight(golden["fp4_packed"][:24], golden["fp4_scales"][:24])
    got = (w @ golden["fp4_x"]).astype(np.float32)
    assert np.max(np.abs(got - golden["fp4_gemv"])) <= 1e-6 * np.max(np.abs(golden["fp4_gemv"]))


def test_fp4_shape_errors():
    import pytest
    with pytest.raises(ValueError):
        fp4.dequantize_fp4_weight(np.zeros((2, 16), np.uint8), np.zeros((2, 2), np.uint8))
    with pytest.raises(ValueError):
        fp4.dequantize_fp4_weight(np.zeros((2, 8), np.uint8), np.zeros((2, 1), np.uint8), block_size=32)


def test_fp8_act_quant_bit_exact(golden):
    codes, scales = fp8.quantize_activation_fp8(golden["fp8_act_x"], 32, "e8m0")
    assert np.array_equal(scales, golden["fp8_act_scales"])
    assert np.array_equal(codes, golden["fp8_act_codes"])


def test_fp8_gemv_matches_reference(golden):
    for tag in ("a", "b"):
        y = fp8.fp8_linear(golden[f"fp8_{tag}_x"], golden[f"fp8_{tag}_w"], golden[f"fp8_{tag}_ws"])
        want = golden[f"fp8_{tag}_y"]
        assert np.max(np.abs(y - want)) <= 2e-6 * np.max(np.abs(want)), tag


def test_e4m3_roundtrip_all_codes():
    codes = np.array([b for b in range(256) if (b & 0x7F) != 0x7F], dtype=np.uint8)
    vals = fp8.E4M3_DECODE[codes]
    back = fp8.e4m3_encode(vals)
    # -0 keeps its sign bit
    assert np.array_equal(back, codes)
    assert fp8.E4M3_DECODE[0x7F] == 0.0 and fp8.E4M3_DECODE[0xFF] == 0.0
    assert fp8.E4M3_DECODE[0x7E] == 448.0 and fp8.E4M3_DECODE[0x01] == 2.0 ** -9


def test_e4m3_encode_against_ml_dtypes():
    import ml_dtypes
    rng = np.random.default_rng(3)
    x = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * 100,
        rng.standard_normal(4000).astype(np.float32) * 0.01,
        (np.arange(0, 1024, dtype=np.float32) * 2.0 ** -10),      # subnormal grid, midpoints
        np.array([448.0, -448.0, 447.9, 464.0 - 1e-3, 0.0, -0.0], dtype=np.float32),
    ])
    x = np.clip(x, -448, 448)
    want = x.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    assert np.array_equal(fp8.e4m3_encode(x), want)
