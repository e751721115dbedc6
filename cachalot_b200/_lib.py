"""ctypes binding of libcachalot_b200.so (the C ABI declared in include/cachalot_b200.h).

There is no fallback: if the library has not been built, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
import os

LIB_PATH = Path(os.environ.get("CACHALOT_B200_LIB", _PKG / "libcachalot_b200.so"))  # override: development builds

OK, EINVAL, EALIGN, EUNSUPPORTED, ECUDA, ESCRATCH = 0, -1, -2, -3, -4, -5
BANK_FP4, BANK_AFFINE = 0, 1
F16, BF16, F32 = 0, 1, 2
NUMERICS_F32, NUMERICS_BF16, NUMERICS_BF16_H32 = 0, 1, 2
DECODE_ONLY_GATE_UP, DECODE_ONLY_DOWN, DECODE_SIMPLE, DECODE_UNFUSED = 0x100, 0x200, 0x400, 0x800
ROUTER_SQRT_SOFTPLUS, ROUTER_SIGMOID = 0, 1
SCALE_E8M0, SCALE_F32 = 0, 1
STATUS_SLOT_RANGE, STATUS_ID_RANGE, STATUS_SCALE_RANGE, STATUS_WAIT_EXPIRED, STATUS_BAD_WEIGHT = 1, 2, 4, 8, 16


class BankDesc(C.Structure):
    """Mirror of `cachalot_bank_desc`."""

    _fields_ = [
        ("record_bytes", C.c_int64),
        ("off", C.c_int64 * 9),
        ("n_slots", C.c_int32),
        ("hidden", C.c_int32),
        ("inter", C.c_int32),
        ("format", C.c_int32),
        ("bits", C.c_int32),
        ("group", C.c_int32),
        ("scale_dtype", C.c_int32),
        ("fp4_scale_centre", C.c_int32),
    ]


class PeerCtx(C.Structure):
    """Mirror of `cachalot_peer_ctx`."""

    _fields_ = [("inbox", C.c_void_p * 8), ("epoch", C.c_void_p), ("world", C.c_int32), ("rank", C.c_int32)]


_vp, _i, _f, _sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
_desc = C.POINTER(BankDesc)

# name -> (restype, argtypes); the list is also what the symbol-export test walks
SIGNATURES = {
    "cachalot_last_error": (C.c_char_p, []),
    "cachalot_version": (_i, []),
    "cachalot_fp4_dequant": (_i, [_vp, _vp, _i, _i, _vp, _vp]),
    "cachalot_affine_dequant": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _vp]),
    "cachalot_requant_fp4_to_affine": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp]),
    "cachalot_router_logits": (_i, [_vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "cachalot_route_topk": (_i, [_vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _f, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "cachalot_moe_decode_workspace_bytes": (_sz, [_desc, _i, _i]),
    "cachalot_moe_decode": (_i, [_vp, _desc, _vp, _vp, _vp, _i, _i, _f, _i, _vp, _sz, _vp, _i, _vp, _vp]),
    "cachalot_moe_layer_decode_workspace_bytes": (_sz, [_desc, _i]),
    "cachalot_moe_layer_decode": (_i, [_vp, _desc, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _i, _i, _f, _i, _vp, _sz, _vp, _i,
                                       _vp, _vp, _vp, _vp]),
    "cachalot_moe_decode_static_scratch_bytes": (_sz, []),
    "cachalot_moe_decode_static": (_i, [_vp, _desc, _vp, _vp, _vp, _i, _i, _f, _i, _vp, _i, _vp, _vp]),
    "cachalot_fp8_act_quant": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp]),
    "cachalot_fp8_gemv": (_i, [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp, _i, _vp]),
    "cachalot_bf16_gemv_f32": (_i, [_vp, _i, _vp, _i, _i, _vp, _vp]),
    "cachalot_fp8_linear": (_i, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp]),
    "cachalot_shared_expert_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "cachalot_shared_expert": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp, _vp, _sz, _vp, _vp]),
    "cachalot_group_rows_scratch_ints": (_sz, [_i, _i, _i]),
    "cachalot_group_rows": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "cachalot_mxfp4_act_quant": (_i, [_vp, _vp, _i, _i, _vp, _vp, _vp]),
    "cachalot_moe_prefill_workspace_bytes": (_sz, [_desc, _i, _i, _i]),
    "cachalot_moe_prefill_rows_workspace_bytes": (_sz, [_desc, C.c_longlong, _i]),
    "cachalot_moe_prefill_rows": (_i, [_vp, _desc, _vp, _vp, _vp, _vp, _vp, _i, C.c_longlong, _f, _vp, _sz, _vp, _vp, _vp]),
    "cachalot_moe_combine_rows": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp]),
    "cachalot_peer_sum_inbox_bytes": (_sz, [_i, _i]),
    "cachalot_peer_sum_flag_bytes": (_sz, [_i]),
    "cachalot_peer_sum": (_i, [_vp, _vp, _i, _i, _vp, _vp, _i, _vp, _vp, _vp]),
    "cachalot_peer_layer_inbox_bytes": (_sz, [_i, _i]),
    "cachalot_moe_layer_decode_peer": (_i, [_vp, _desc, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _f, _i, _i, _f, _i, _vp, _sz, _vp, _i,
                                            _vp, _vp, _vp, _vp, _vp]),
    "cachalot_moe_prefill": (_i, [_vp, _desc, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _f, _i, _vp, _sz, _vp, _vp, _vp]),
}


def _load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m cachalot_b200.build` "
            "(needs nvcc; there is no CPU or PyTorch fallback for these kernels)"
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype, fn.argtypes = res, args
    return lib


lib = _load()


def last_error() -> str:
    return lib.cachalot_last_error().decode("utf-8", "replace")


def check(rc: int) -> None:
    """Map a C return code onto the exception the reference raises for the same condition."""
    if rc == OK:
        return
    msg = last_error()
    if rc == EUNSUPPORTED:
        raise NotImplementedError(msg)
    if rc == ECUDA:
        raise RuntimeError(msg)
    raise ValueError(msg)
