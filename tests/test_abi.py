"""The C-ABI library loads and exports every symbol include/cachalot_b200.h declares (no GPU needed)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def declared_symbols() -> list[str]:
    text = (ROOT / "include" / "cachalot_b200.h").read_text()
    return sorted(set(re.findall(r"CACHALOT_API[^;(]*?\b(cachalot_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("cachalot_moe_decode", "cachalot_fp4_dequant", "cachalot_fp8_gemv", "cachalot_route_topk",
                 "cachalot_group_rows", "cachalot_moe_prefill", "cachalot_mxfp4_act_quant"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from cachalot_b200 import build

    lib_path = build.build()
    lib = ctypes.CDLL(str(lib_path))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_binding_table_matches_header():
    from cachalot_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_bank_desc_layout_matches_header():
    from cachalot_b200 import _lib

    # int64 + 9*int64 + 8*int32
    assert ctypes.sizeof(_lib.BankDesc) == 8 + 72 + 32


def test_host_side_argument_errors_need_no_gpu():
    """Argument validation happens before any CUDA call, with the reference's error wording."""
    from cachalot_b200 import _lib

    lib = _lib.lib
    rc = lib.cachalot_fp4_dequant(None, None, 4, 64, None, None)
    assert rc == _lib.EINVAL and "null" in _lib.last_error()
    buf = (ctypes.c_uint8 * 64)()
    out = (ctypes.c_float * 64)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    rc = lib.cachalot_fp4_dequant(p, p, 1, 48, ctypes.cast(out, ctypes.c_void_p), None)
    assert rc == _lib.EINVAL and "multiple of 32" in _lib.last_error()
    rc = lib.cachalot_route_topk(p, None, None, 0, 1, 8, 9, 0, 1.0, 1.0, 1, 0, p, p, None, None, None)
    assert rc == _lib.EINVAL and "Invalid topk=9 for 8 experts" in _lib.last_error()
    rc = lib.cachalot_fp8_act_quant(p, 1, 48, 32, 0, p, p, None)
    assert rc == _lib.EINVAL and "divisible" in _lib.last_error()
    rc = lib.cachalot_fp8_act_quant(p, 1, 64, 64, 0, p, p, None)
    assert rc == _lib.EUNSUPPORTED
    with pytest.raises(NotImplementedError):
        _lib.check(rc)
    d = _lib.BankDesc()
    d.format, d.hidden, d.inter, d.n_slots, d.bits = _lib.BANK_AFFINE, 128, 128, 1, 3
    rc = lib.cachalot_moe_decode(p, ctypes.byref(d), p, p, p, 1, 1, 0.0, 0, p, 64, p, _lib.F32, None, None)
    assert rc == _lib.EUNSUPPORTED and "bits=3" in _lib.last_error()
    assert lib.cachalot_moe_decode_workspace_bytes(ctypes.byref(d), 2, 6) >= 2 * 6 * 128 * 4


def test_bank_layout_and_sizes():
    """Slot record sizes of the configured shapes (bytes per expert quoted for the roofline)."""
    from cachalot_b200.bank import FP4_FORMAT, affine_format, tensor_sizes

    fp4 = tensor_sizes(FP4_FORMAT, 4096, 2880)
    assert fp4["w1.weight"] == 5_898_240 and fp4["w1.scale"] == 368_640
    assert sum(fp4.values()) == 18_800_640
    aff = tensor_sizes(affine_format(4096, 2880), 4096, 2880)
    assert sum(aff.values()) == 9_953_280
    assert sum(tensor_sizes(FP4_FORMAT, 5120, 2304).values()) == 18_800_640
