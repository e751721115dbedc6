"""Host-side operators with the reference's names and argument meaning, on CUDA tensors.

Every function here calls the C ABI (libcachalot_b200.so); none has a PyTorch or CPU fallback.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from ._lib import check, lib
from .bank import FP4_FORMAT, ExpertFormat, ResidentExpert, SlabBank


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("cachalot_b200 operators take CUDA tensors (there is no CPU path)")


# ---- dequantisation ---------------------------------------------------------------------------

def dequantize_fp4_weight(packed: torch.Tensor, scales: torch.Tensor, block_size: int = 32) -> torch.Tensor:
    """packed uint8 [N, K/2], scales uint8 [N, K/32] -> float32 [N, K] (model/fp4.py:67-109)."""
    _need_cuda(packed, scales)
    if block_size != 32:
        raise NotImplementedError("FP4 banks use per-32 scales")
    if packed.dim() != 2 or packed.dtype != torch.uint8 or scales.dtype != torch.uint8:
        raise ValueError(f"packed/scales must be 2-D uint8, got {packed.dtype} {tuple(packed.shape)}")
    n, k = packed.shape[0], packed.shape[1] * 2
    if k % block_size:
        raise ValueError(f"K={k} must be divisible by block_size={block_size}")
    if tuple(scales.shape) != (n, k // block_size):
        raise ValueError(f"Scale shape {tuple(scales.shape)} does not match expected {(n, k // block_size)}")
    packed, scales = packed.contiguous(), scales.contiguous()
    out = torch.empty((n, k), dtype=torch.float32, device=packed.device)
    if n == 0:
        return out
    check(lib.cachalot_fp4_dequant(_ptr(packed), _ptr(scales), n, k, _ptr(out), _stream()))
    return out


def dequantize_affine(words: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, *, bits: int, group_size: int) -> torch.Tensor:
    """words int32/uint32 [N, K*bits/32]; scales/biases f16 or bf16 -> float32 [N, K] = scale*q + bias."""
    _need_cuda(words, scales, biases)
    n = words.shape[0]
    k = words.shape[1] * 32 // bits
    if scales.dtype not in (torch.float16, torch.bfloat16) or biases.dtype != scales.dtype:
        raise ValueError("scales and biases must both be float16 or both bfloat16")
    if scales.numel() != n * k // group_size:
        raise ValueError(f"{scales.numel()} scales for {n}x{k} at group {group_size}")
    out = torch.empty((n, k), dtype=torch.float32, device=words.device)
    sdt = _lib.BF16 if scales.dtype == torch.bfloat16 else _lib.F16
    check(lib.cachalot_affine_dequant(_ptr(words.contiguous()), _ptr(scales.contiguous()), _ptr(biases.contiguous()),
                                      n, k, bits, group_size, sdt, _ptr(out), _stream()))
    return out


def requantize_fp4_to_affine(packed: torch.Tensor, scales: torch.Tensor, *, bits: int = 2, group_size: int = 128,
                             scale_dtype=torch.float16, lsq_iters: int = 4):
    """FP4 matrix (packed uint8 [N,K/2], E8M0 uint8 [N,K/32]) -> (words int32 [N, K*bits/32], scales, biases
    [N*K/group_size] in `scale_dtype`): the searched affine fit with least-squares refinement that builds a 2-bit
    bank from the FP4 checkpoint (benchmarks/quant_affine.py:138-329, fit_search_lsq + quantize_affine)."""
    _need_cuda(packed, scales)
    n, k = packed.shape[0], packed.shape[1] * 2
    if tuple(scales.shape) != (n, k // 32):
        raise ValueError(f"Scale shape {tuple(scales.shape)} does not match expected {(n, k // 32)}")
    if scale_dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("scales and biases are stored as float16 or bfloat16")
    words = torch.empty((n, k * bits // 32), dtype=torch.int32, device=packed.device)
    s = torch.empty(n * k // group_size, dtype=scale_dtype, device=packed.device)
    b = torch.empty_like(s)
    sdt = _lib.BF16 if scale_dtype == torch.bfloat16 else _lib.F16
    check(lib.cachalot_requant_fp4_to_affine(_ptr(packed.contiguous()), _ptr(scales.contiguous()), n, k, bits, group_size, sdt,
                                             int(lsq_iters), _ptr(words), _ptr(s), _ptr(b), _stream()))
    return words, s, b


def requantize_bank(bank: SlabBank, *, bits: int = 2, group_size: int = 128, scale_dtype=torch.float16, lsq_iters: int = 4) -> SlabBank:
    """An affine bank with the same slots and slot table as the FP4 `bank`, every expert re-quantised on the GPU
    (what benchmarks/build_affine_bank.py does offline for the 2-bit bank)."""
    from .bank import affine_format

    if bank.fmt.kind != "fp4":
        raise ValueError("requantize_bank takes an FP4 bank")
    name = "bfloat16" if scale_dtype == torch.bfloat16 else "float16"
    out = SlabBank(affine_format(bank.hidden, bank.inter, bits, group_size, name), bank.hidden, bank.inter, bank.n_slots,
                   layers=bank.layers, n_experts=bank.n_experts, device=bank.slab.device)
    out.slot_table_host, out.slot_table = bank.slot_table_host.clone(), bank.slot_table.clone()
    for slot in range(bank.n_slots):
        t = {}
        for proj in ("w1", "w2", "w3"):
            w, s, b = requantize_fp4_to_affine(bank.typed_view(slot, f"{proj}.weight"), bank.typed_view(slot, f"{proj}.scale"), bits=bits,
                                               group_size=group_size, scale_dtype=scale_dtype, lsq_iters=lsq_iters)
            t[f"{proj}.weight"], t[f"{proj}.scales"], t[f"{proj}.biases"] = w, s, b
        out.write_expert(slot, t)
    return out


# ---- routing ----------------------------------------------------------------------------------

@dataclass(frozen=True)
class RouterResult:
    """Same fields as the reference's RouterResult (model/router_mlx.py:9-13)."""

    indices: torch.Tensor
    weights: torch.Tensor
    scores: torch.Tensor


def router_logits(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """fp32 gate logits [rows, E] of bf16 rows x [rows, H] against weight [E, H] (bf16 or f32)."""
    _need_cuda(x, weight)
    x2 = x.reshape(-1, x.shape[-1]).to(torch.bfloat16).contiguous()
    e, h = weight.shape
    if x2.shape[1] != h:
        raise ValueError(f"x has {x2.shape[1]} elements, gate expects {h}")
    if weight.dtype == torch.bfloat16:
        wdt = _lib.BF16
    elif weight.dtype == torch.float32:
        wdt = _lib.F32
    else:
        raise ValueError(f"gate weight must be bfloat16 or float32, got {weight.dtype}")
    out = torch.empty((x2.shape[0], e), dtype=torch.float32, device=x.device)
    check(lib.cachalot_router_logits(_ptr(x2), _ptr(weight.contiguous()), wdt, x2.shape[0], e, h, _ptr(out), _stream()))
    return out


def _route(logits, bias, table, layer, k, mode, gate_temp, route_scale, norm, weights_bf16, want_scores):
    rows, e = logits.shape
    dev = logits.device
    idx = torch.empty((rows, k), dtype=torch.int32, device=dev)
    w = torch.empty((rows, k), dtype=torch.float32, device=dev)
    slots = torch.empty((rows, k), dtype=torch.int32, device=dev)
    scores = torch.empty((rows, e), dtype=torch.float32, device=dev) if want_scores else None
    b = None if bias is None else bias.to(torch.float32).contiguous()
    check(lib.cachalot_route_topk(_ptr(logits), _ptr(b), _ptr(table), layer, rows, e, k, mode, float(gate_temp),
                                  float(route_scale), int(norm), int(weights_bf16), _ptr(idx), _ptr(w), _ptr(slots),
                                  _ptr(scores), _stream()))
    return idx, w, slots, scores


def route_topk_fused(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, *, topk: int = 6, gate_temp: float = 1.0,
                     route_scale: float = 1.5, norm_topk_prob: bool = True) -> RouterResult:
    """DeepSeek router for one decode token (model/router_fused_metal.py:111-148): indices int32 [k]
    ascending by selection score, weights float32 [k], scores float32 [E]."""
    if x.dim() != 1:
        raise ValueError(f"x must be 1D, got {tuple(x.shape)}")
    if weight.dim() != 2:
        raise ValueError(f"weight must be 2D, got {tuple(weight.shape)}")
    if tuple(bias.shape) != (weight.shape[0],):
        raise ValueError(f"bias shape {tuple(bias.shape)} != ({weight.shape[0]},)")
    if not 1 <= topk <= weight.shape[0]:
        raise ValueError(f"Invalid topk={topk} for {weight.shape[0]} experts")
    logits = router_logits(x, weight)
    idx, w, _, scores = _route(logits, bias, None, 0, topk, _lib.ROUTER_SQRT_SOFTPLUS, gate_temp, route_scale,
                               norm_topk_prob, False, True)
    return RouterResult(indices=idx[0], weights=w[0], scores=scores[0])


route_topk = route_topk_fused


def route_topk_rows(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, *, topk: int = 6, gate_temp: float = 1.0,
                    route_scale: float = 1.5, norm_topk_prob: bool = True) -> RouterResult:
    """Row-wise router for a prompt chunk (model/moe_prefill_batched.py:128-178): [T,k] outputs."""
    if x.dim() != 2:
        raise ValueError(f"x must be 2D, got {tuple(x.shape)}")
    logits = router_logits(x, weight)
    idx, w, _, scores = _route(logits, bias, None, 0, topk, _lib.ROUTER_SQRT_SOFTPLUS, gate_temp, route_scale,
                               norm_topk_prob, False, True)
    return RouterResult(indices=idx, weights=w, scores=scores)


def route_tail(raw: torch.Tensor, bias: torch.Tensor | None, table: torch.Tensor | None, layer: int, k: int, scale: float,
               *, weights_bf16: bool = True):
    """Sigmoid routing tail with slot lookup (minimax/gpu_select.py:119-132).  raw float32 [..., E]
    (rows = leading dims); returns (inds int32 [rows,k], weights float32 [rows,k] rounded to bf16
    precision by default, slots int32 [rows,k]); no host round trip."""
    _need_cuda(raw)
    logits = raw.reshape(-1, raw.shape[-1]).to(torch.float32).contiguous()
    idx, w, slots, _ = _route(logits, bias, table, layer, k, _lib.ROUTER_SIGMOID, 1.0, scale, True, weights_bf16, False)
    return idx, w, slots


# ---- decode: routed experts -------------------------------------------------------------------

_workspaces: dict = {}


def _workspace(device, nbytes: int) -> torch.Tensor:
    key = (device, torch.cuda.current_stream().cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def moe_forward(x: torch.Tensor, slot_ids: torch.Tensor, gate_weights: torch.Tensor, bank: SlabBank, *,
                swiglu_limit: float = 10.0, numerics: str | None = None, out_dtype=torch.float32,
                out: torch.Tensor | None = None, status: torch.Tensor | None = None,
                workspace: torch.Tensor | None = None, phase: str | None = None, simple: bool = False,
                unfused: bool = False) -> torch.Tensor:
    """Routed experts for `rows` tokens: x bf16 [rows,H], slot_ids int32 [rows,k] (bank slots, -1 =
    absent -> zero contribution), gate_weights float32 [rows,k] -> [rows,H].

    x of another float dtype is ROUNDED TO BF16 first: the kernels take bf16 activations only.  The reference's
    runtime passes bf16 hidden states, for which this is the identity; its op would read a float32 x unrounded
    (model/moe_fused_metal.py:200,208), so a float32 caller sees up to 2**-9 relative input rounding here.

    numerics "f32" keeps fp32 between the projections (the FP4 decode op,
    model/moe_fused_metal.py:189-233); "bf16" rounds g, u, h and each expert's output to bf16 (the
    affine op, model/expert_affine.py:65-81).  Default: by bank format.  `phase` ("gate_up" or
    "down") runs only one of the two launches; it exists for per-kernel timing.  `simple` selects
    the one-warp-per-output kernels instead of the tensor-core ones (a cross-check, any shape);
    `unfused` selects the two-launch tensor-core kernels where the single-launch kernel (one token)
    would run."""
    _need_cuda(x, slot_ids, gate_weights)
    if x.dim() != 2 or x.shape[1] != bank.hidden:
        raise ValueError(f"x must be [rows, {bank.hidden}], got {tuple(x.shape)}")
    rows = x.shape[0]
    if slot_ids.dim() != 2 or slot_ids.shape[0] != rows or tuple(gate_weights.shape) != tuple(slot_ids.shape):
        raise ValueError(f"slot_ids {tuple(slot_ids.shape)} / gate_weights {tuple(gate_weights.shape)} do not match rows={rows}")
    k = slot_ids.shape[1]
    if numerics is None:
        numerics = "f32" if bank.fmt.kind == "fp4" else "bf16"
    num = {"f32": _lib.NUMERICS_F32, "bf16": _lib.NUMERICS_BF16, "bf16_h32": _lib.NUMERICS_BF16_H32}[numerics]
    num |= {None: 0, "gate_up": _lib.DECODE_ONLY_GATE_UP, "down": _lib.DECODE_ONLY_DOWN}[phase]
    if simple or FORCE_SIMPLE_KERNELS:
        num |= _lib.DECODE_SIMPLE
    if unfused:
        num |= _lib.DECODE_UNFUSED
    xb = x.to(torch.bfloat16).contiguous()
    slot_ids = slot_ids.to(torch.int32).contiguous()
    gate_weights = gate_weights.to(torch.float32).contiguous()
    odt = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}[out_dtype]
    if out is None:
        out = torch.empty((rows, bank.hidden), dtype=out_dtype, device=x.device)
    need = lib.cachalot_moe_decode_workspace_bytes(bank.desc_ptr, rows, k)
    ws = workspace if workspace is not None else _workspace(x.device, need + 256)
    base = (ws.data_ptr() + 255) // 256 * 256
    check(lib.cachalot_moe_decode(_ptr(bank.slab), bank.desc_ptr, _ptr(xb), _ptr(slot_ids), _ptr(gate_weights), rows, k,
                                  float(swiglu_limit), num, base, ws.numel() - (base - ws.data_ptr()), _ptr(out), odt,
                                  _ptr(status), _stream()))
    return out


def moe_layer_decode(x: torch.Tensor, logits: torch.Tensor, bank: SlabBank, *, layer: int = 0, topk: int = 6,
                     bias: torch.Tensor | None = None, table: torch.Tensor | None = None, router: str = "sigmoid",
                     gate_temp: float = 1.0, route_scale: float = 1.0, norm_topk_prob: bool = True, weights_bf16: bool = False,
                     swiglu_limit: float = 10.0, numerics: str | None = None, out_dtype=torch.float32,
                     out: torch.Tensor | None = None, status: torch.Tensor | None = None,
                     workspace: torch.Tensor | None = None, want_routing: bool = False, peer=None):
    """Routing tail + routed experts of one decode token as ONE launch: the GPU-side form of the routed half
    of `moe_layer_forward` (model/moe_layer_metal.py:133-405) with slot selection on the device as in
    minimax/gpu_select.py:330-551.  x bf16 [H]; logits float32 [E] (gate output); `table` int32 [layers,E]
    (default: the bank's slot table); router "sigmoid" (route_tail rules) or "sqrt_softplus" (route_topk rules).
    Returns out [H], or (out, indices int32 [k], weights float32 [k]) with want_routing.
    `peer` (an `ep.PeerLayer`): the bank is this rank's shard of an expert-parallel layer and `out` receives the sum
    over all ranks, exchanged through peer memory in the tail of the same launch."""
    _need_cuda(x, logits)
    if x.dim() != 1 or x.numel() != bank.hidden:
        raise ValueError(f"x must be 1-D with {bank.hidden} elements, got {tuple(x.shape)}")
    if logits.dim() != 1:
        raise ValueError(f"logits must be 1-D [E], got {tuple(logits.shape)}")
    e = logits.numel()
    if not 1 <= topk <= e:
        raise ValueError(f"Invalid topk={topk} for {e} experts")
    if bias is not None and tuple(bias.shape) != (e,):
        raise ValueError(f"bias shape {tuple(bias.shape)} != ({e},)")
    mode = {"sigmoid": _lib.ROUTER_SIGMOID, "sqrt_softplus": _lib.ROUTER_SQRT_SOFTPLUS}[router]
    if numerics is None:
        numerics = "f32" if bank.fmt.kind == "fp4" else "bf16"
    num = {"f32": _lib.NUMERICS_F32, "bf16": _lib.NUMERICS_BF16, "bf16_h32": _lib.NUMERICS_BF16_H32}[numerics]
    if table is None:
        table = bank.slot_table
    xb = x.to(torch.bfloat16).contiguous()
    lg = logits.to(torch.float32).contiguous()
    b = None if bias is None else bias.to(torch.float32).contiguous()
    odt = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}[out_dtype]
    if out is None:
        out = torch.empty(bank.hidden, dtype=out_dtype, device=x.device)
    idx = torch.empty(topk, dtype=torch.int32, device=x.device) if want_routing else None
    w = torch.empty(topk, dtype=torch.float32, device=x.device) if want_routing else None
    need = lib.cachalot_moe_layer_decode_workspace_bytes(bank.desc_ptr, topk)
    ws = workspace if workspace is not None else _workspace(x.device, need + 256)
    base = (ws.data_ptr() + 255) // 256 * 256
    if peer is not None:
        import ctypes as C

        check(lib.cachalot_moe_layer_decode_peer(_ptr(bank.slab), bank.desc_ptr, _ptr(xb), _ptr(lg), _ptr(b), _ptr(table.contiguous()),
                                                 int(layer), e, int(topk), mode, float(gate_temp), float(route_scale),
                                                 int(norm_topk_prob), int(weights_bf16), float(swiglu_limit), num, base,
                                                 ws.numel() - (base - ws.data_ptr()), _ptr(out), odt, _ptr(idx), _ptr(w),
                                                 C.cast(C.byref(peer.ctx), C.c_void_p), _ptr(status), _stream()))
        return (out, idx, w) if want_routing else out
    check(lib.cachalot_moe_layer_decode(_ptr(bank.slab), bank.desc_ptr, _ptr(xb), _ptr(lg), _ptr(b), _ptr(table.contiguous()), int(layer),
                                        e, int(topk), mode, float(gate_temp), float(route_scale), int(norm_topk_prob),
                                        int(weights_bf16), float(swiglu_limit), num, base, ws.numel() - (base - ws.data_ptr()),
                                        _ptr(out), odt, _ptr(idx), _ptr(w), _ptr(status), _stream()))
    return (out, idx, w) if want_routing else out


def _slots_of(experts) -> tuple[SlabBank, torch.Tensor]:
    if len(experts) == 0:
        raise ValueError("no experts given")
    bank = experts[0].bank
    for e in experts:
        if not isinstance(e, ResidentExpert) or e.bank is not bank:
            raise ValueError("experts must be ResidentExpert objects of one bank")
    return bank, torch.tensor([[e.slot for e in experts]], dtype=torch.int32, device=bank.slab.device)


def fused_routed_experts(x: torch.Tensor, experts, router_weights: torch.Tensor, *, hidden_size: int = 5120,
                         intermediate: int = 2304, swiglu_limit: float = 10.0) -> torch.Tensor:
    """Top-k routed experts of one decode token over an FP4 bank (model/moe_fused_metal.py:189-233):
    x [hidden_size] bf16 (another float dtype is rounded to bf16, see `moe_forward`), experts = ResidentExpert
    objects, router_weights float32 [k] -> float32 [hidden_size]."""
    bank, slots = _slots_of(experts)
    if bank.fmt.kind != "fp4":
        raise ValueError("fused_routed_experts needs an FP4 bank; use affine_routed_experts")
    if (bank.hidden, bank.inter) != (hidden_size, intermediate):
        raise ValueError(f"bank is {bank.hidden}x{bank.inter}, call says {hidden_size}x{intermediate}")
    if x.dim() != 1 or x.numel() != hidden_size:
        raise ValueError(f"x must be 1-D with {hidden_size} elements, got {tuple(x.shape)}")
    if router_weights.numel() != len(experts):
        raise ValueError(f"{len(experts)=} does not match {router_weights.numel()=}")
    return moe_forward(x[None], slots, router_weights.reshape(1, -1), bank, swiglu_limit=swiglu_limit, numerics="f32")[0]


def affine_routed_experts(x: torch.Tensor, experts, fmt: ExpertFormat, weights: torch.Tensor,
                          swiglu_limit: float = 10.0) -> torch.Tensor:
    """Sum of the routed experts of one decode token over an affine bank
    (model/expert_affine.py:186-206) -> float32 [hidden]."""
    bank, slots = _slots_of(experts)
    if bank.fmt.kind != "affine" or (fmt.bits, fmt.group_size) != (bank.fmt.bits, bank.fmt.group_size):
        raise ValueError("format does not match the experts' bank")
    if x.dim() != 1:
        raise ValueError(f"x must be 1-D, got {tuple(x.shape)}")
    return moe_forward(x[None], slots, weights.reshape(1, -1), bank, swiglu_limit=swiglu_limit, numerics="bf16")[0]


def routed_expert_forward(x: torch.Tensor, *, w1_packed, w1_scales, w2_packed, w2_scales, w3_packed, w3_scales,
                          weight=None, swiglu_limit: float = 10.0) -> torch.Tensor:
    """One FP4 expert on loose tensors (model/expert_metal.py:9-64).  The tensors are copied into a
    one-slot bank first; the slot path (fused_routed_experts / moe_forward) is the fast one."""
    inter, hidden = w1_packed.reshape(w1_scales.shape[0], -1).shape[0], w1_packed.numel() * 2 // w1_scales.shape[0]
    bank = SlabBank(FP4_FORMAT, hidden, inter, 1, device=x.device)
    bank.write_expert(0, {"w1.weight": w1_packed, "w1.scale": w1_scales, "w2.weight": w2_packed, "w2.scale": w2_scales,
                          "w3.weight": w3_packed, "w3.scale": w3_scales})
    w = torch.ones(1, 1, dtype=torch.float32, device=x.device) if weight is None else \
        torch.as_tensor(weight, dtype=torch.float32, device=x.device).reshape(1, 1)
    slots = torch.zeros((1, 1), dtype=torch.int32, device=x.device)
    return moe_forward(x.reshape(1, -1), slots, w, bank, swiglu_limit=swiglu_limit, numerics="f32")[0]


# ---- FP8 trunk GEMV ---------------------------------------------------------------------------

@dataclass(frozen=True)
class QuantizedActivation:
    """Same fields as the reference's (model/fp8_linear_metal.py:22-27); `decoded` is unused here
    because the GEMV decodes E4M3 in registers."""

    values: torch.Tensor
    scales: torch.Tensor
    in_features: int
    decoded: torch.Tensor | None = None
    block_size: int = 32
    scale_rule: str = "e8m0"


_RULE = {"e8m0": _lib.SCALE_E8M0, "f32": _lib.SCALE_F32}


def quantize_fp8_activation(x: torch.Tensor, block_size: int = 32, scale_rule: str = "e8m0") -> QuantizedActivation:
    """act_quant (model/fp8_ref.py:27-92).  The reference takes one token (1-D); [rows, K] is the
    same per row."""
    _need_cuda(x)
    if x.dim() not in (1, 2):
        raise ValueError(f"Decode FP8 activation must be 1D, got {tuple(x.shape)}")
    k = x.shape[-1]
    if k % block_size:
        raise ValueError(f"K={k} must be divisible by block_size={block_size}")
    x2 = x.reshape(-1, k).to(torch.bfloat16).contiguous()
    codes = torch.empty(x2.shape, dtype=torch.uint8, device=x.device)
    scales = torch.empty((x2.shape[0], k // block_size), dtype=torch.float32, device=x.device)
    check(lib.cachalot_fp8_act_quant(_ptr(x2), x2.shape[0], k, block_size, _RULE[scale_rule], _ptr(codes), _ptr(scales), _stream()))
    if x.dim() == 1:
        codes, scales = codes[0], scales[0]
    return QuantizedActivation(codes, scales, k, None, block_size, scale_rule)


def fp8_linear_quantized(x: QuantizedActivation, weight: torch.Tensor, weight_scales: torch.Tensor, *,
                         out_dtype=torch.bfloat16) -> torch.Tensor:
    """FP8 GEMV on a quantised activation (model/fp8_linear_metal.py:56-89) -> bf16 [N] / [rows,N]."""
    if weight.dim() != 2:
        raise ValueError(f"weight must be 2D, got {tuple(weight.shape)}")
    n, k = weight.shape
    if k != x.in_features:
        raise ValueError(f"weight expects {k} inputs, quantized activation has {x.in_features}")
    rule = "e8m0" if weight_scales.dtype == torch.uint8 else "f32"
    if rule != x.scale_rule:
        raise ValueError(f"activation was quantised with {x.scale_rule!r} scales, weight scales are {rule!r}")
    expected = (-(-n // x.block_size), k // x.block_size)
    if tuple(weight_scales.shape) != expected:
        raise ValueError(f"scale shape {tuple(weight_scales.shape)} != {expected}")
    codes = x.values.reshape(-1, k)
    out = torch.empty((codes.shape[0], n), dtype=out_dtype, device=weight.device)
    odt = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}[out_dtype]
    check(lib.cachalot_fp8_gemv(_ptr(codes.contiguous()), _ptr(x.scales.contiguous()), _ptr(weight.contiguous()),
                                _ptr(weight_scales.contiguous()), _RULE[rule], x.block_size, codes.shape[0], n, k,
                                _ptr(out), odt, _stream()))
    return out[0] if x.values.dim() == 1 else out


def fp8_linear(x: torch.Tensor, weight: torch.Tensor, weight_scales: torch.Tensor, *, out_dtype=torch.bfloat16) -> torch.Tensor:
    """act_quant + GEMV (model/fp8_linear_metal.py:92-107).  uint8 weight scales select the
    reference's E8M0 / block-32 form, float32 scales the fp32 / block-(K / scale columns) form."""
    if weight_scales.dtype == torch.uint8:
        block, rule = 32, "e8m0"
    else:
        block, rule = weight.shape[1] // weight_scales.shape[1], "f32"
    _need_cuda(x, weight, weight_scales)
    if x.dim() not in (1, 2):
        raise ValueError(f"Decode FP8 activation must be 1D, got {tuple(x.shape)}")
    if weight.dim() != 2:
        raise ValueError(f"weight must be 2D, got {tuple(weight.shape)}")
    n, k = weight.shape
    if x.shape[-1] != k:
        raise ValueError(f"weight expects {k} inputs, activation has {x.shape[-1]}")
    if k % block:
        raise ValueError(f"K={k} must be divisible by block_size={block}")
    expected = (-(-n // block), k // block)
    if tuple(weight_scales.shape) != expected:
        raise ValueError(f"scale shape {tuple(weight_scales.shape)} != {expected}")
    x2 = x.reshape(-1, k).to(torch.bfloat16).contiguous()
    rows = x2.shape[0]
    codes = torch.empty((rows, k), dtype=torch.uint8, device=x.device)
    scales = torch.empty((rows, k // block), dtype=torch.float32, device=x.device)
    out = torch.empty((rows, n), dtype=out_dtype, device=x.device)
    odt = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}[out_dtype]
    if rows:
        check(lib.cachalot_fp8_linear(_ptr(x2), rows, k, block, _RULE[rule], _ptr(codes), _ptr(scales), _ptr(weight.contiguous()),
                                      _ptr(weight_scales.contiguous()), n, _ptr(out), odt, _stream()))
    return out[0] if x.dim() == 1 else out


# ---- prefill ----------------------------------------------------------------------------------

def group_rows(expert_ids: torch.Tensor, n_experts: int, status: torch.Tensor | None = None):
    """Expert-major grouping of routed rows (model/moe_prefill_grouped.py:201-225): expert_ids int32
    [T,k] -> (perm int32 [T*k], offsets int32 [E+1])."""
    _need_cuda(expert_ids)
    t, k = expert_ids.shape
    ids = expert_ids.to(torch.int32).contiguous()
    perm = torch.empty(t * k, dtype=torch.int32, device=ids.device)
    offsets = torch.empty(n_experts + 1, dtype=torch.int32, device=ids.device)
    scratch = torch.empty(max(int(lib.cachalot_group_rows_scratch_ints(t, k, n_experts)), 1), dtype=torch.int32, device=ids.device)
    if t * k == 0:
        return perm, offsets.zero_()
    check(lib.cachalot_group_rows(_ptr(ids), t, k, n_experts, _ptr(perm), _ptr(offsets), _ptr(scratch), _ptr(status), _stream()))
    return perm, offsets


def quantize_mxfp4(x: torch.Tensor, src_rows: torch.Tensor | None = None):
    """MXFP4 activation quantisation (model/fp4_act_mlx.py:101-250, block 32 / E8M0): x bf16 [rows,K]
    -> (codes uint8 [rows,K/2] low nibble first, scale bytes uint8 [rows,K/32])."""
    _need_cuda(x)
    k = x.shape[-1]
    if k % 32:
        raise ValueError(f"last dimension {k} must be divisible by block_size=32")
    x2 = x.reshape(-1, k).to(torch.bfloat16).contiguous()
    rows = x2.shape[0] if src_rows is None else src_rows.numel()
    codes = torch.empty((rows, k // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty((rows, k // 32), dtype=torch.uint8, device=x.device)
    src = None if src_rows is None else src_rows.to(torch.int32).contiguous()
    check(lib.cachalot_mxfp4_act_quant(_ptr(x2), _ptr(src), rows, k, _ptr(codes), _ptr(scales), _stream()))
    return codes, scales


def moe_prefill_grouped(x: torch.Tensor, expert_ids: torch.Tensor, weights: torch.Tensor, bank: SlabBank, *,
                        layer: int = 0, swiglu_limit: float = 10.0, mxfp4_act: bool = False,
                        status: torch.Tensor | None = None) -> torch.Tensor:
    """Expert-major routed experts for a prompt chunk (model/moe_prefill_grouped.py:74-635, routed
    part): x bf16 [T,H], expert_ids int32 [T,k], weights float32 [T,k] -> float32 [T,H] = per-slot
    results summed in slot order.  mxfp4_act quantises x and the hidden activation per 32 first."""
    _need_cuda(x, expert_ids, weights)
    t, k = expert_ids.shape
    e = bank.n_experts
    perm, offsets = group_rows(expert_ids, e, status)
    slot_of_expert = bank.slot_table[layer].contiguous()
    xb = x.to(torch.bfloat16).contiguous()
    out = torch.empty((t, bank.hidden), dtype=torch.float32, device=x.device)
    if t == 0:
        return out
    need = lib.cachalot_moe_prefill_workspace_bytes(bank.desc_ptr, t, k, int(mxfp4_act))
    ws = _workspace(x.device, need + 256)
    base = (ws.data_ptr() + 255) // 256 * 256
    check(lib.cachalot_moe_prefill(_ptr(bank.slab), bank.desc_ptr, _ptr(xb), _ptr(perm), _ptr(offsets), _ptr(slot_of_expert),
                                   _ptr(weights.to(torch.float32).contiguous()), t, k, e, float(swiglu_limit), int(mxfp4_act),
                                   base, ws.numel() - (base - ws.data_ptr()), _ptr(out), _ptr(status), _stream()))
    return out


def moe_prefill_rows(x_codes: torch.Tensor, x_scales: torch.Tensor, row_weights: torch.Tensor, seg_offsets: torch.Tensor,
                     seg_slots: torch.Tensor | None, bank: SlabBank, *, swiglu_limit: float = 10.0,
                     status: torch.Tensor | None = None) -> torch.Tensor:
    """Expert outputs of rows that are already MXFP4-quantised and laid out in segments (one expert per segment):
    codes uint8 [R,H/2], scale bytes uint8 [R,H/32], row_weights float32 [R], seg_offsets int32 [S+1],
    seg_slots int32 [S] bank slots (-1 = absent -> zero rows) -> bfloat16 [R,H].  The middle of
    `moe_prefill_grouped`, which an expert-parallel rank runs between its dispatch and combine exchanges."""
    _need_cuda(x_codes, x_scales, row_weights, seg_offsets)
    rows = x_codes.shape[0]
    n_seg = seg_offsets.numel() - 1
    y = torch.empty((rows, bank.hidden), dtype=torch.bfloat16, device=x_codes.device)
    if rows == 0 or n_seg <= 0:
        return y
    need = lib.cachalot_moe_prefill_rows_workspace_bytes(bank.desc_ptr, rows, n_seg)
    ws = _workspace(x_codes.device, need + 256)
    base = (ws.data_ptr() + 255) // 256 * 256
    slots = None if seg_slots is None else seg_slots.to(torch.int32).contiguous()
    check(lib.cachalot_moe_prefill_rows(_ptr(bank.slab), bank.desc_ptr, _ptr(x_codes.contiguous()), _ptr(x_scales.contiguous()),
                                        _ptr(row_weights.to(torch.float32).contiguous()), _ptr(seg_offsets.to(torch.int32).contiguous()),
                                        _ptr(slots), n_seg, rows, float(swiglu_limit), base, ws.numel() - (base - ws.data_ptr()),
                                        _ptr(y), _ptr(status), _stream()))
    return y


def combine_rows(y: torch.Tensor, inv: torch.Tensor, tokens: int, k: int) -> torch.Tensor:
    """out[t] = sum over route slots j = 0..k-1, in that order, of y[inv[t*k+j]] (inv < 0 skipped)
    (model/moe_prefill_grouped.py:526-530): y bfloat16 [R,H], inv int32 [T*k] -> float32 [T,H]."""
    _need_cuda(y, inv)
    out = torch.empty((tokens, y.shape[1]), dtype=torch.float32, device=y.device)
    if tokens:
        check(lib.cachalot_moe_combine_rows(_ptr(y.contiguous()), _ptr(inv.to(torch.int32).contiguous()), tokens, k, y.shape[1],
                                            _ptr(out), _stream()))
    return out


# ---- the reference's per-expert prefill entries ---------------------------------------------------

def _one_expert_rows(x, tensors, fmt, weights, swiglu_limit, numerics):
    """[M,H] rows through ONE expert given as loose tensors: the tensors are copied into a one-slot bank and every
    row is routed to it with its own weight (k = 1)."""
    if x.dim() != 2:
        raise ValueError(f"x must be [M, H], got {tuple(x.shape)}")
    m = x.shape[0]
    if weights.numel() != m:
        raise ValueError(f"{weights.numel()} router weights for {m} rows")
    if fmt.kind == "fp4":
        inter = tensors["w1.scale"].shape[0]
        hidden = tensors["w1.weight"].numel() * 2 // inter
    else:
        inter, hidden = fmt.shapes["w1.weight"][0], fmt.shapes["w2.weight"][0]
    bank = SlabBank(fmt, hidden, inter, 1, device=x.device)
    bank.write_expert(0, tensors)
    slots = torch.zeros((m, 1), dtype=torch.int32, device=x.device)
    return moe_forward(x, slots, weights.reshape(m, 1), bank, swiglu_limit=swiglu_limit, numerics=numerics)


def routed_expert_forward_batched(x: torch.Tensor, *, w1_packed, w1_scales, w2_packed, w2_scales, w3_packed, w3_scales,
                                  weights: torch.Tensor, swiglu_limit: float = 10.0) -> torch.Tensor:
    """One FP4 expert over a batch of rows with the reference's prefill rounding points (g, u -> bf16; h -> bf16;
    output -> bf16 -> f32): model/moe_prefill_batched.py:31-61.  x [M,H], weights [M] -> float32 [M,H]."""
    t = {"w1.weight": w1_packed, "w1.scale": w1_scales, "w2.weight": w2_packed, "w2.scale": w2_scales,
         "w3.weight": w3_packed, "w3.scale": w3_scales}
    return _one_expert_rows(x, t, FP4_FORMAT, weights, swiglu_limit, "bf16")


routed_expert_forward_sgmm = routed_expert_forward_batched   # same contract (model/fp4_sgmm_metal.py:318-333)


def affine_expert_forward_batched(x: torch.Tensor, arrays: dict, fmt: ExpertFormat, weights: torch.Tensor,
                                  swiglu_limit: float = 10.0) -> torch.Tensor:
    """One affine-quantised expert over a batch of rows (model/expert_affine.py:84-99): x [M,H], `arrays` = the
    expert's nine tensors by the format's names, weights [M] -> float32 [M,H]."""
    if fmt.kind != "affine":
        raise ValueError("affine_expert_forward_batched needs an affine format")
    return _one_expert_rows(x, arrays, fmt, weights, swiglu_limit, "bf16")


class SlabExperts:
    """The routed experts of any layer from a slot index array on the device, each expert's output kept apart
    (minimax/gpu_select.py:279-327): `SlabExperts(bank)(x[1,D], slots int32 [k]) -> [k, D]`.  The reference passes
    the activation as a callable between its two kernels; here the two projections are one launch, so only the
    SwiGLU of the routed experts is offered (`activation` None, or a float = its clamp limit)."""

    def __init__(self, pool: SlabBank, fmt: ExpertFormat | None = None) -> None:
        if fmt is not None and fmt.kind != pool.fmt.kind:
            raise ValueError("format does not match the pool")
        self.pool = pool

    def __call__(self, x: torch.Tensor, slots: torch.Tensor, activation=None) -> torch.Tensor:
        if callable(activation):
            raise NotImplementedError("a custom activation between the projections is not built; pass None or the clamp limit")
        limit = 0.0 if activation is None else float(activation)
        k = slots.numel()
        xs = x.reshape(1, -1).expand(k, -1)
        ones = torch.ones((k, 1), dtype=torch.float32, device=x.device)
        return moe_forward(xs, slots.reshape(k, 1), ones, self.pool, swiglu_limit=limit).to(x.dtype)


# ---- shared FP8 expert and the whole MoE layer -------------------------------------------------------

def _fp8_rule(scales: torch.Tensor, n: int, k: int):
    if scales.dtype == torch.uint8:
        return "e8m0", 32
    if scales.dtype != torch.float32:
        raise ValueError(f"weight scales must be uint8 (E8M0) or float32, got {scales.dtype}")
    return "f32", k // scales.shape[1]


def _shared(x2, w1, w1s, w3, w3s, w2, w2s, swiglu_limit, addend):
    rows, hidden = x2.shape
    inter = w2.shape[1]
    rule, block = _fp8_rule(w2s, hidden, inter)
    if tuple(w2.shape) != (hidden, inter) or w1.shape[1] != hidden or w1.shape[0] != (inter if w3 is not None else 2 * inter):
        raise ValueError(f"shared expert shapes do not fit: x {tuple(x2.shape)}, w1 {tuple(w1.shape)}, w2 {tuple(w2.shape)}")
    xb = x2.to(torch.bfloat16).contiguous()
    out = torch.empty((rows, hidden), dtype=torch.bfloat16, device=x2.device)
    if rows == 0:
        return out
    need = lib.cachalot_shared_expert_workspace_bytes(rows, hidden, inter, block)
    ws = _workspace(x2.device, need + 256)
    base = (ws.data_ptr() + 255) // 256 * 256
    ad = None if addend is None else addend.to(torch.float32).contiguous()
    check(lib.cachalot_shared_expert(_ptr(xb), rows, hidden, inter, _ptr(w1.contiguous()), _ptr(w1s.contiguous()),
                                     _ptr(None if w3 is None else w3.contiguous()), _ptr(None if w3s is None else w3s.contiguous()),
                                     _ptr(w2.contiguous()), _ptr(w2s.contiguous()), _RULE[rule], block, float(swiglu_limit),
                                     _ptr(ad), base, ws.numel() - (base - ws.data_ptr()), _ptr(out), _stream()))
    return out


def shared_expert_forward(x: torch.Tensor, *, w1, w1_scales, w2, w2_scales, w3, w3_scales, swiglu_limit: float = 10.0) -> torch.Tensor:
    """The resident FP8 expert for one decode token (model/shared_expert_metal.py:45-134): bf16 [H]."""
    if x.dim() != 1:
        raise ValueError(f"x must be 1D for decode, got {tuple(x.shape)}")
    return _shared(x[None], w1, w1_scales, w3, w3_scales, w2, w2_scales, swiglu_limit, None)[0]


def shared_expert_forward_fused(x: torch.Tensor, *, w13, w13_scales, w2, w2_scales, swiglu_limit: float = 10.0) -> torch.Tensor:
    """The same with w1 and w3 concatenated along the rows, one GEMV (model/shared_expert_metal.py:137-188)."""
    if x.dim() != 1:
        raise ValueError(f"x must be 1D for decode, got {tuple(x.shape)}")
    return _shared(x[None], w13, w13_scales, None, None, w2, w2_scales, swiglu_limit, None)[0]


def shared_expert_forward_batched(x: torch.Tensor, *, w1, w1_scales, w2, w2_scales, w3, w3_scales, swiglu_limit: float = 10.0) -> torch.Tensor:
    """The shared expert over a prompt chunk (model/moe_prefill_batched.py:100-125): x [M,H] -> bf16 [M,H]."""
    if x.dim() != 2:
        raise ValueError(f"x must be [M, H], got {tuple(x.shape)}")
    return _shared(x, w1, w1_scales, w3, w3_scales, w2, w2_scales, swiglu_limit, None)


def bf16_gemv_f32(x: torch.Tensor, weight_bf16: torch.Tensor) -> torch.Tensor:
    """bf16-weight, fp32-activation GEMV with fp32 accumulation (model/bf16_gemv_metal.py:50-63; the output head):
    x [K] any float dtype (or [rows<=8, K]: the rows share one pass over the weights), weight_bf16 [N, K] bfloat16
    -> float32 [N] (or [rows, N])."""
    if weight_bf16.dtype != torch.bfloat16 or weight_bf16.dim() != 2:
        raise ValueError("weight must be 2D bfloat16")
    _need_cuda(x, weight_bf16)
    n, k = weight_bf16.shape
    if k % 64:
        raise ValueError("in_features must be a multiple of 64")
    x2 = x.reshape(-1, x.shape[-1]) if x.dim() > 1 else x.reshape(1, -1)
    if x2.shape[1] != k:
        raise ValueError(f"x has {x2.shape[1]} features, weight has {k}")
    xf = x2.to(torch.float32).contiguous()
    w = weight_bf16.contiguous()
    out = torch.empty((xf.shape[0], n), dtype=torch.float32, device=x.device)
    for r0 in range(0, xf.shape[0], 8):
        r1 = min(r0 + 8, xf.shape[0])
        check(lib.cachalot_bf16_gemv_f32(_ptr(xf[r0:r1]), r1 - r0, _ptr(w), n, k, _ptr(out[r0:r1]), _stream()))
    return out[0] if x.dim() == 1 else out.reshape(*x.shape[:-1], n)


def fp8_linear_rows(x: torch.Tensor, weight: torch.Tensor, weight_scales: torch.Tensor) -> torch.Tensor:
    """x [T,K] -> bf16 [T,N] (model/moe_prefill_batched.py:93-97): act_quant per row, then the GEMV's arithmetic."""
    return fp8_linear(x, weight, weight_scales)


_fused_rows_cache: dict = {}


def fused_qr_kv_linear(x: torch.Tensor, wq_a, wq_a_scales, wkv, wkv_scales):
    """qr = fp8_linear(x, wq_a), window_kv = fp8_linear(x, wkv) as ONE act_quant and ONE GEMV over the rows of both
    matrices (model/attention_qkv_fusion.py:46-68); the concatenation is built once per pair of weights."""
    key = (wq_a.data_ptr(), wkv.data_ptr())
    hit = _fused_rows_cache.get(key)
    if hit is None or hit[0] is not wq_a or hit[1] is not wkv:
        hit = (wq_a, wkv, torch.cat([wq_a, wkv], 0).contiguous(), torch.cat([wq_a_scales, wkv_scales], 0).contiguous())
        _fused_rows_cache[key] = hit
    block = 32 if wq_a_scales.dtype == torch.uint8 else wq_a.shape[1] // wq_a_scales.shape[1]
    if wq_a.shape[0] % block:
        raise ValueError(f"{wq_a.shape[0]} rows of the first matrix are not whole scale blocks of {block}")
    out = fp8_linear(x, hit[2], hit[3])
    rows = wq_a.shape[0]
    return out[..., :rows], out[..., rows:]


def moe_layer_forward(x: torch.Tensor, *, layer_id: int, gate_weight: torch.Tensor, gate_bias: torch.Tensor,
                      expert_store: SlabBank, shared_w1, shared_w1_scales, shared_w2, shared_w2_scales, shared_w3,
                      shared_w3_scales, expert_index=None, topk: int = 6, gate_temp: float = 1.0, route_scale: float = 1.5,
                      norm_topk_prob: bool = True, swiglu_limit: float = 10.0, fused: bool | None = None,
                      scores: bool = True, status: torch.Tensor | None = None):
    """The whole MoE block of one decode token, keyword for keyword the reference's entry
    (model/moe_layer_metal.py:133-405): bf16 x [H] -> fp32 router (gate GEMV, sqrt-softplus scores, top-k) ->
    routed experts over the resident bank -> shared FP8 expert -> (routed + shared.f32) -> bf16 [H].  Returns
    (output, RouterResult).  Nothing here waits for the device: the selected ids go from the routing tail to the
    expert kernel on the GPU (an expert whose slot is -1 contributes zeros), so `expert_index` -- the reference's
    host-side (layer, expert) -> entry map -- is only checked for the layer's presence when given.
    `expert_store` is the SlabBank; `shared_w3 = None` means `shared_w1` holds the w1 || w3 concatenation.
    `fused` is accepted for signature parity (there is one path).  `scores=False` skips the [E] score vector."""
    if x.dim() != 1:
        raise ValueError(f"x must be 1D for decode, got {tuple(x.shape)}")
    bank = expert_store
    e = gate_weight.shape[0]
    if tuple(gate_bias.shape) != (e,):
        raise ValueError(f"bias shape {tuple(gate_bias.shape)} != ({e},)")
    if expert_index is not None and not any(k[0] == layer_id for k in expert_index):
        raise KeyError(f"Missing routed expert layer={layer_id}")
    logits = router_logits(x, gate_weight)[0]
    routed, idx, w = moe_layer_decode(x, logits, bank, layer=layer_id, topk=topk, bias=gate_bias, router="sqrt_softplus",
                                      gate_temp=gate_temp, route_scale=route_scale, norm_topk_prob=norm_topk_prob,
                                      swiglu_limit=swiglu_limit, status=status, want_routing=True)
    sc = None
    if scores:
        _, _, _, s2 = _route(logits[None], gate_bias, None, 0, topk, _lib.ROUTER_SQRT_SOFTPLUS, gate_temp, route_scale,
                             norm_topk_prob, False, True)
        sc = s2[0]
    out = _shared(x[None], shared_w1, shared_w1_scales, shared_w3, shared_w3_scales, shared_w2, shared_w2_scales, swiglu_limit,
                  routed[None])[0]
    return out, RouterResult(indices=idx, weights=w, scores=sc)


# ---- checks --------------------------------------------------------------------------------------

def validate_routing(expert_ids: torch.Tensor, weights: torch.Tensor, n_experts: int, *, allow_absent: bool = False) -> None:
    """Host-side check of a routing result before it is handed to the expert operators (it reads the tensors, so on
    CUDA tensors it waits for the device: a debugging aid, not part of the hot path).  Raises ValueError for an expert
    id outside [0, n_experts) (-1 passes with `allow_absent`), for an expert chosen twice by one token, for a weight
    that is NaN or infinite, and for shapes that do not match.  The kernels themselves never trap on such input: an id
    out of range is dropped (CACHALOT_STATUS_ID_RANGE / SLOT_RANGE), a bad weight is used as it is
    (CACHALOT_STATUS_BAD_WEIGHT)."""
    if expert_ids.dim() != 2 or tuple(weights.shape) != tuple(expert_ids.shape):
        raise ValueError(f"expert_ids {tuple(expert_ids.shape)} and weights {tuple(weights.shape)} must both be [tokens, k]")
    ids = expert_ids.detach().to("cpu", torch.int64)
    w = weights.detach().to("cpu", torch.float32)
    low = -1 if allow_absent else 0
    bad = (ids < low) | (ids >= n_experts)
    if bool(bad.any()):
        t, j = (int(v) for v in bad.nonzero()[0])
        raise ValueError(f"expert id {int(ids[t, j])} of token {t}, slot {j} is outside [0, {n_experts})")
    srt, _ = torch.sort(ids, dim=1)
    dup = (srt[:, 1:] == srt[:, :-1]) & (srt[:, 1:] >= 0)
    if bool(dup.any()):
        t = int(dup.nonzero()[0][0])
        raise ValueError(f"token {t} routes to one expert twice: {ids[t].tolist()}")
    if not bool(torch.isfinite(w).all()):
        t, j = (int(v) for v in (~torch.isfinite(w)).nonzero()[0])
        raise ValueError(f"router weight of token {t}, slot {j} is {float(w[t, j])}")


_self_check_done: dict = {}
FORCE_SIMPLE_KERNELS = False   # set by a failed self_check: moe_forward then takes the one-warp-per-output kernels


def self_check(device=None, *, tol: float = 2e-3, _run=None) -> bool:
    """Load-time check in the manner of the reference's kernel self-check (minimax/codes_qmv.py:8-15, 475-477: a
    custom kernel that stops matching the library path is switched off): one tiny decode through the single-launch
    kernel against the one-warp-per-output kernels for both bank formats.  Returns True when they agree; on a
    mismatch it sets FORCE_SIMPLE_KERNELS, so `moe_forward` keeps to the simple kernels, and returns False.  Once per
    device.  `_run(kind) -> (fast, slow)` replaces the device work (tests)."""
    global FORCE_SIMPLE_KERNELS
    key = str(device)
    if key in _self_check_done:
        return _self_check_done[key]

    def run(kind):
        from .bank import affine_format
        dev = torch.device("cuda") if device is None else torch.device(device)
        hidden, inter, k = 256, 192, 3
        fmt = FP4_FORMAT if kind == "fp4" else affine_format(hidden, inter)
        bank = SlabBank(fmt, hidden, inter, 4, device=dev)
        gen = torch.Generator(device=dev).manual_seed(0)
        bank.fill_random(gen)
        x = torch.randn((1, hidden), device=dev, generator=gen).to(torch.bfloat16)
        slots = torch.tensor([[2, 0, 3]], dtype=torch.int32, device=dev)
        w = torch.tensor([[0.5, 0.3, 0.2]], dtype=torch.float32, device=dev)
        return moe_forward(x, slots, w, bank, numerics="f32"), moe_forward(x, slots, w, bank, numerics="f32", simple=True)

    ok = True
    for kind in ("fp4", "affine"):
        fast, slow = (_run or run)(kind)
        ok = ok and bool(torch.isfinite(fast).all()) and float((fast - slow).abs().max()) <= tol * max(float(slow.abs().max()), 1e-30)
    if not ok:
        FORCE_SIMPLE_KERNELS = True
    _self_check_done[key] = ok
    return ok
