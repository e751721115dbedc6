"""cachalot_b200: B200 (sm_100a) kernels for the routed-expert MoE hot path and the FP8 trunk
GEMV, behind the reference's operator names.

The operators load libcachalot_b200.so on first use and raise ImportError if it has not been
built (`python -m cachalot_b200.build`); there is no CPU or PyTorch fallback.  Only
`cachalot_b200.build` can be imported without the library.
"""
NUMERICS_VERSION = "cachalot_b200-1"

_BANK = ("FP4_FORMAT", "ExpertFormat", "ResidentExpert", "SlabBank", "affine_format", "tensor_sizes")
_OPS = (
    "QuantizedActivation", "RouterResult", "affine_routed_experts", "dequantize_affine", "dequantize_fp4_weight",
    "fp8_linear", "fp8_linear_quantized", "fused_routed_experts", "group_rows", "moe_forward", "moe_layer_decode",
    "combine_rows", "moe_prefill_grouped", "moe_prefill_rows",
    "quantize_fp8_activation", "quantize_mxfp4", "route_tail", "route_topk", "route_topk_fused", "route_topk_rows",
    "routed_expert_forward", "router_logits", "routed_expert_forward_batched", "routed_expert_forward_sgmm",
    "affine_expert_forward_batched", "SlabExperts", "shared_expert_forward", "shared_expert_forward_fused",
    "shared_expert_forward_batched", "fp8_linear_rows", "bf16_gemv_f32", "fused_qr_kv_linear", "moe_layer_forward", "validate_routing", "self_check", "requantize_fp4_to_affine", "requantize_bank",
)
_LOADER = ("load_bank", "detect_expert_bank", "build_expert_index", "build_stacked_expert_index")
__all__ = [*_BANK, *_OPS, *_LOADER, "NUMERICS_VERSION"]


def __getattr__(name):
    import importlib

    if name in _BANK:
        return getattr(importlib.import_module(".bank", __name__), name)
    if name in _OPS:
        return getattr(importlib.import_module(".ops", __name__), name)
    if name in _LOADER:
        return getattr(importlib.import_module(".loader", __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
