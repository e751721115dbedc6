"""Shared FP8 expert and the closing sum of the decode MoE layer.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  Composition of the pinned FP8 pieces (oracle/fp8.py, bit-compared
with the reference's model/fp8_ref.py) in the order of
  src/cachalot/model/shared_expert_metal.py:94-134, 160-188   one act_quant for w1 and w3; the two linears come back as
       bf16 and are read as f32; up = clip(up, +-L), gate = min(gate, L); hidden = silu(gate) * up -> the activation
       dtype (bf16) -> act_quant -> w2 -> bf16
  src/cachalot/model/moe_prefill_batched.py:100-125           the same per row of a prompt chunk
  src/cachalot/model/moe_layer_metal.py:394-403               output = (routed + shared.astype(f32)).astype(x.dtype)
"""
from __future__ import annotations

import numpy as np

from . import fp8
from .bf16 import round_bf16
from .fp4 import swiglu


def shared_expert_forward(x, w1, w1_scales, w2, w2_scales, w3, w3_scales, *, swiglu_limit=10.0, block_size=32, scale_rule="e8m0"):
    """x [H] or [M,H] (bf16 values) -> the shared expert's output rounded to bf16, as float32."""
    xb = round_bf16(np.asarray(x, dtype=np.float32))
    codes, scales = fp8.quantize_activation_fp8(xb, block_size, scale_rule)
    gate = round_bf16(fp8.fp8_gemv_quantized(codes, scales, w1, w1_scales, block_size=block_size, scale_rule=scale_rule))
    up = round_bf16(fp8.fp8_gemv_quantized(codes, scales, w3, w3_scales, block_size=block_size, scale_rule=scale_rule))
    hidden = round_bf16(swiglu(gate, up, swiglu_limit).astype(np.float32))
    hc, hs = fp8.quantize_activation_fp8(hidden, block_size, scale_rule)
    return round_bf16(fp8.fp8_gemv_quantized(hc, hs, w2, w2_scales, block_size=block_size, scale_rule=scale_rule))


def close_layer(routed_f32, shared_bf16):
    """(routed + shared.f32) -> bf16, as float32."""
    return round_bf16((np.asarray(routed_f32, np.float32) + np.asarray(shared_bf16, np.float32)).astype(np.float32))
