"""Generates tests/golden/reference_numpy.npz from the reference's own numpy modules.

Run in a checkout where the reference tree is available:
    python tests/golden/make_golden.py /path/to/reference
It loads src/cachalot/model/fp4.py and src/cachalot/model/fp8_ref.py BY FILE PATH (the package's
__init__ needs MLX) and stores small seeded inputs together with the reference's outputs.  The
fixture file is what the test-suite reads; this script is never run by the tests.
"""
from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

import numpy as np


def _load(path: Path, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main(ref_root: str) -> None:
    model = Path(ref_root) / "src" / "cachalot" / "model"
    fp4 = _load(model / "fp4.py", "ref_fp4")
    fp8 = _load(model / "fp8_ref.py", "ref_fp8")
    rng = np.random.default_rng(20250101)
    out: dict[str, np.ndarray] = {}

    # the 16-entry table and the E8M0 decode over every byte that is finite in float32
    out["fp4_table"] = fp4.FP4_E2M1_TABLE.copy()
    out["e8m0_raw"] = np.arange(0, 255, dtype=np.uint8)
    out["e8m0_f32"] = fp4.decode_e8m0(out["e8m0_raw"])

    # dequant: every nibble code against a spread of scales, then a random matrix
    packed = rng.integers(0, 256, (48, 64), dtype=np.uint8)
    scales = rng.integers(1, 251, (48, 4), dtype=np.uint8)  # up to 6 * 2**123, finite in float32
    scales[:24] = rng.integers(118, 124, (24, 4), dtype=np.uint8)  # configured range 2^-9..2^-4
    out["fp4_packed"], out["fp4_scales"] = packed, scales
    out["fp4_dequant"] = fp4.dequantize_fp4_weight(packed, scales)
    x = rng.standard_normal(128).astype(np.float32)
    out["fp4_x"] = x
    out["fp4_gemv"] = (fp4.dequantize_fp4_weight(packed[:24], scales[:24]) @ x).astype(np.float32)

    # act_quant on plain, tiny, huge, tie-heavy and zero blocks
    k = 256
    a = rng.standard_normal(k).astype(np.float32)
    a[32:64] *= 1e-6          # below the 1e-4 amax floor
    a[64:96] *= 3e4           # large
    a[96:128] = np.linspace(-448, 448, 32, dtype=np.float32)  # lands on exact grid points / ties after scaling
    a[128:160] = 0.0
    a[160:192] = np.float32(2.0 ** -9) * np.arange(32, dtype=np.float32) * 0.5  # subnormal grid and its midpoints
    q, s = fp8.quantize_activation_fp8(a)
    out["fp8_act_x"], out["fp8_act_codes"], out["fp8_act_scales"] = a, q.view(np.uint8).copy(), s

    # GEMV: synthetic recipe of the reference's micro benchmark (codes < 0x38 with random sign,
    # E8M0 scales 125..129) plus one matrix over all finite codes
    for tag, n, kk in (("a", 64, 128), ("b", 96, 256)):
        if tag == "a":
            w = rng.integers(0, 0x38, (n, kk), dtype=np.uint8) | (rng.integers(0, 2, (n, kk), dtype=np.uint8) << 7)
            ws = rng.integers(125, 130, (-(-n // 32), kk // 32), dtype=np.uint8)
        else:
            finite = np.array([b for b in range(256) if (b & 0x7F) != 0x7F], dtype=np.uint8)
            w = finite[rng.integers(0, finite.size, (n, kk))]
            ws = rng.integers(120, 134, (-(-n // 32), kk // 32), dtype=np.uint8)
        xv = rng.standard_normal(kk).astype(np.float32)
        out[f"fp8_{tag}_w"], out[f"fp8_{tag}_ws"], out[f"fp8_{tag}_x"] = w, ws, xv
        out[f"fp8_{tag}_y"] = fp8.fp8_gemv_reference(xv, w, ws)

    dst = Path(__file__).resolve().parent / "reference_numpy.npz"
    np.savez_compressed(dst, **out)
    print(f"wrote {dst} ({dst.stat().st_size} bytes)")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path of a checkout of the reference>")
    main(sys.argv[1])
