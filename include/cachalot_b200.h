/*
 * cachalot_b200 -- C ABI of the B200 (sm_100a) routed-expert MoE / FP8 trunk GEMV kernels.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, launches on the stream
 * the caller passes (never synchronises, never allocates) and returns 0 on success or a
 * negative CACHALOT_E* code; cachalot_last_error() gives the message for the calling thread.
 * Pointers are DEVICE pointers unless the comment says "host".  Conditions only the device
 * can see (a slot id outside the bank) set bits in the caller's `status` word and the kernel
 * still returns normally: no trap, no hang.
 *
 * Each declaration names the interface of the reference (prooshani/cachalot, paths relative
 * to its repository root) that it replaces.
 */
#ifndef CACHALOT_B200_H
#define CACHALOT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define CACHALOT_API __attribute__((visibility("default")))
#else
#define CACHALOT_API
#endif

typedef struct CUstream_st* cachalot_stream_t; /* a cudaStream_t */

enum {
  CACHALOT_OK = 0,
  CACHALOT_EINVAL = -1,       /* bad shape / null pointer / size not supported */
  CACHALOT_EALIGN = -2,       /* pointer or offset not aligned as required */
  CACHALOT_EUNSUPPORTED = -3, /* legal in the reference but not built here */
  CACHALOT_ECUDA = -4,        /* a CUDA call failed; see cachalot_last_error() */
  CACHALOT_ESCRATCH = -5      /* workspace too small */
};

/* bits of the device-side status word */
enum {
  CACHALOT_STATUS_SLOT_RANGE = 1, /* a slot id >= n_slots was seen and treated as absent */
  CACHALOT_STATUS_ID_RANGE = 2,   /* an expert id outside [0, E) was seen and dropped */
  CACHALOT_STATUS_SCALE_RANGE = 4, /* an FP4 block scale outside the window around fp4_scale_centre was clamped */
  CACHALOT_STATUS_WAIT_EXPIRED = 8, /* a bounded device-side wait ran out (the result of that call is not valid) */
  CACHALOT_STATUS_BAD_WEIGHT = 16 /* a router weight was NaN or infinite (it was used as it is) */
};

enum { CACHALOT_BANK_FP4 = 0, CACHALOT_BANK_AFFINE = 1 };
enum { CACHALOT_F16 = 0, CACHALOT_BF16 = 1, CACHALOT_F32 = 2 };
/* rounding points of the expert FFN */
enum {
  CACHALOT_NUMERICS_F32 = 0, /* decode FP4 op: fp32 everywhere (model/moe_fused_metal.py:101-179) */
  CACHALOT_NUMERICS_BF16 = 1, /* affine and prefill ops: g,u -> bf16; h -> bf16; each expert's W2 h -> bf16
                                 (model/expert_affine.py:74-81, model/fp4_sgmm_metal.py:203-233) */
  CACHALOT_NUMERICS_BF16_H32 = 2 /* as BF16 but h stays fp32 (it is quantised to MXFP4 next) */
};
/* Kernel selection, OR-ed into `numerics`.  These exist for cross-checks and per-kernel timing; a caller that
 * wants the result leaves them clear.
 *   SIMPLE  : the one-warp-per-output kernels (any shape; the cross-check of the tensor-core kernels, as the
 *             reference checks its fused kernels against the unfused loop)
 *   UNFUSED : the two-launch kernels (rows grouped by expert) even where the single-launch kernel applies
 *   ONLY_*  : development only, not part of the ABI contract: run one of the two launches of the two-launch path
 *             (the output of such a call is not the layer's result) */
enum { CACHALOT_DECODE_SIMPLE = 0x400, CACHALOT_DECODE_UNFUSED = 0x800 };
enum { CACHALOT_DECODE_ONLY_GATE_UP = 0x100, CACHALOT_DECODE_ONLY_DOWN = 0x200 };
enum { CACHALOT_ROUTER_SQRT_SOFTPLUS = 0, CACHALOT_ROUTER_SIGMOID = 1 };
enum { CACHALOT_SCALE_E8M0 = 0, CACHALOT_SCALE_F32 = 1 };

/*
 * An expert bank: n_slots records of record_bytes each in one device allocation; tensor i of a
 * record starts at byte off[i] (multiple of 16).  This is the device-side form of the
 * reference's slab slot pool (cache/slots.py:185-251: rows of a [slots, record_bytes] uint8
 * array with fixed per-tensor offsets) and of its per-expert accessors (cache/resident.py:11-52).
 *   FP4 bank    off[0..5] = w1.weight, w1.scale, w2.weight, w2.scale, w3.weight, w3.scale
 *               (names and order of cache/slots.py:30-37); weight = E2M1 nibbles [N, K/2], low
 *               nibble first; scale = E8M0 bytes [N, K/32] (model/fp4.py:44-109).
 *   affine bank off[0..8] = w1.weight, w1.scales, w1.biases, w2.*, w3.*; weight = u32 words
 *               [N, K*bits/32] (little-endian bit stream, benchmarks/quant_affine.py:69-105),
 *               scales / biases [N, K/group] in scale_dtype (model/expert_affine.py:26-51).
 * w1 (gate) and w3 (up) are [inter, hidden]; w2 (down) is [hidden, inter].
 */
typedef struct {
  int64_t record_bytes;
  int64_t off[9];
  int32_t n_slots;
  int32_t hidden;
  int32_t inter;
  int32_t format;      /* CACHALOT_BANK_* */
  int32_t bits;        /* affine: 2 (built); FP4: 4 */
  int32_t group;       /* affine: 128 or 64; FP4: 32 */
  int32_t scale_dtype; /* affine: CACHALOT_F16 or CACHALOT_BF16 */
  int32_t fp4_scale_centre; /* FP4: an E8M0 byte near the middle of the bank's scale range (0 = 121);
                               scales must lie within [centre-14, centre+13], else CACHALOT_STATUS_SCALE_RANGE */
} cachalot_bank_desc;

CACHALOT_API const char* cachalot_last_error(void);
CACHALOT_API int cachalot_version(void); /* ABI revision, 2 for this header */

/* ---- dequantisation (bit-exact against the reference's numpy path) ------------------------ */

/* Replaces model/fp4.py:67-109 dequantize_fp4_weight and the Metal twins
 * model/fp4_dequant_metal.py:11-65: packed u8 [N,K/2] + scales u8 [N,K/32] -> f32 [N,K]. */
CACHALOT_API int cachalot_fp4_dequant(const uint8_t* packed, const uint8_t* scales, int n, int k, float* out,
                         cachalot_stream_t stream);

/* Replaces mx.dequantize as the reference uses it for affine banks (benchmarks/quant_affine.py:
 * 119-123, 366-367): out = f32(scale)*q + f32(bias), one rounding.  bits in {2,4,8}. */
CACHALOT_API int cachalot_affine_dequant(const uint32_t* words, const void* scales, const void* biases, int n, int k,
                            int bits, int group, int scale_dtype, float* out, cachalot_stream_t stream);

/* Replaces benchmarks/quant_affine.py:138-329 (fit_search + refine_lsq + quantize_affine), the step that builds a
 * 2-bit affine bank from FP4 weights (benchmarks/build_affine_bank.py:72-187): per group of `group` (64 or 128)
 * consecutive elements of the flattened [N*K] matrix a min/max fit, the 5 x 5 grid search over shrunk ranges, then
 * `lsq_iters` rounds of least-squares refinement with scale and bias rounded to the storage dtype every round;
 * levels are taken against the rounded scale and bias.  packed u8 [N,K/2], scales u8 [N,K/32] (FP4 as above) ->
 * out_words u32 [N*K*bits/32] (little-endian bit stream), out_scales / out_biases [N*K/group] in scale_dtype.
 * bits 2 or 4. */
CACHALOT_API int cachalot_requant_fp4_to_affine(const uint8_t* packed, const uint8_t* scales, int n, int k, int bits, int group,
                                   int scale_dtype, int lsq_iters, uint32_t* out_words, void* out_scales,
                                   void* out_biases, cachalot_stream_t stream);

/* ---- routing ------------------------------------------------------------------------------ */

/* Replaces the score half of model/router_fused_metal.py:33-58 (router_scores): for each of
 * `rows` tokens, logits[e] = dot(x, gate_w[e]) in fp32; x is bf16 [rows,H]; gate_w is
 * [E,H] in w_dtype (CACHALOT_BF16 or CACHALOT_F32).  The non-linearity is applied by
 * cachalot_route_topk so that both routers share this kernel. */
CACHALOT_API int cachalot_router_logits(const void* x_bf16, const void* gate_w, int w_dtype, int rows, int n_experts,
                           int hidden, float* logits, cachalot_stream_t stream);

/* Replaces model/router_fused_metal.py:62-108 + router_mlx.py:16-118 (mode SQRT_SOFTPLUS:
 * score = sqrt(softplus(logit/gate_temp)); top-k of score+bias, written ascending, ties to the
 * larger index; weights = score/(sum+1e-20)*route_scale), model/moe_prefill_batched.py:128-178
 * (the same per row) and minimax/gpu_select.py:80-132 route_tail (mode SIGMOID: strongest first,
 * ties to the lower index, slot table lookup).  logits f32 [rows,E]; bias f32 [E] or NULL;
 * slot_table i32 [layers,E] or NULL (then slots = expert ids); outputs indices i32 [rows,k],
 * weights f32 [rows,k] (rounded to bf16 precision when weights_bf16 != 0, as route_tail does),
 * slots i32 [rows,k] (may be NULL), scores f32 [rows,E] (may be NULL). E <= 1024, k <= 32. */
CACHALOT_API int cachalot_route_topk(const float* logits, const float* bias, const int32_t* slot_table, int layer, int rows,
                        int n_experts, int k, int mode, float gate_temp, float route_scale, int norm_topk_prob,
                        int weights_bf16, int32_t* indices, float* weights, int32_t* slots, float* scores,
                        cachalot_stream_t stream);

/* ---- decode: routed experts over bank slots ----------------------------------------------- */

/* Bytes of workspace cachalot_moe_decode needs for `rows` tokens and top-k `k`. */
CACHALOT_API size_t cachalot_moe_decode_workspace_bytes(const cachalot_bank_desc* desc /* host */, int rows, int k);

/* Replaces model/moe_fused_metal.py:189-233 fused_routed_experts (FP4 bank),
 * model/expert_affine.py:186-206 affine_routed_experts (affine bank) and the slot-indexed slab
 * op minimax/gpu_select.py:279-327 SlabExperts: for each of `rows` tokens,
 *   out[t] = sum_{j<k} W2_s( silu(min(W1_s x, L)) * clip(W3_s x, +-L) * gate_w[t,j] ),  s = slots[t,j]
 * with the router weight applied before the down projection (model/expert_metal.py:54-56), the
 * clamp skipped when swiglu_limit <= 0, and a slot < 0 contributing zeros
 * (minimax/gpu_select.py:265-273).  x bf16 [rows,H]; slots i32 [rows,k]; gate_w f32 [rows,k];
 * out f32 [rows,H] (or bf16 when out_dtype == CACHALOT_BF16).  The reference runs one token at a
 * time (model/moe_layer_metal.py:168-171); rows > 1 is the same math per row. */
CACHALOT_API int cachalot_moe_decode(const void* bank, const cachalot_bank_desc* desc /* host */, const void* x_bf16,
                        const int32_t* slots, const float* gate_w, int rows, int k, float swiglu_limit,
                        int numerics, void* workspace, size_t workspace_bytes, void* out, int out_dtype,
                        int* status, cachalot_stream_t stream);

/* Replaces the routed half of model/moe_layer_metal.py:133-405 moe_layer_forward for one decode token
 * without its host round trip (router -> mx.eval -> store.get_many -> experts, :279-355), in the way
 * minimax/gpu_select.py:330-551 keeps slot selection on the GPU: the routing tail of
 * cachalot_route_topk (same modes, tie rules and weight formulas) runs inside the expert kernel's
 * prologue, so a layer is one launch.  logits f32 [E]; bias f32 [E] or NULL; slot_table i32
 * [layers,E] or NULL; x bf16 [H]; out [H].  indices_out i32 [k] / weights_out f32 [k] (either may
 * be NULL) receive the routing result.  k <= 8 runs as one launch; otherwise (and for bank shapes
 * the single-launch kernel does not cover) the call issues the routing kernel and
 * cachalot_moe_decode. */
CACHALOT_API size_t cachalot_moe_layer_decode_workspace_bytes(const cachalot_bank_desc* desc /* host */, int k);
CACHALOT_API int cachalot_moe_layer_decode(const void* bank, const cachalot_bank_desc* desc /* host */, const void* x_bf16,
                              const float* logits, const float* bias, const int32_t* slot_table, int layer,
                              int n_experts, int k, int mode, float gate_temp, float route_scale, int norm_topk_prob,
                              int weights_bf16, float swiglu_limit, int numerics, void* workspace,
                              size_t workspace_bytes, void* out, int out_dtype, int32_t* indices_out,
                              float* weights_out, int* status, cachalot_stream_t stream);

/* No counterpart in the reference.  The same computation as cachalot_moe_decode for callers that
 * must not allocate device memory and have no workspace to hand over: an embedding whose memory
 * pool already owns all of HBM (a cudaMalloc there fails, or forces a device-wide
 * synchronisation in the middle of a token), a plugin slot whose signature has no room for a
 * scratch pointer, or a real-time decode loop that may not call into the allocator.  The scratch is
 * a 4 MiB array that is part of the library image: every GPU that loads the library holds it until
 * the process exits.  A call whose cachalot_moe_decode_workspace_bytes(desc, rows, k) exceeds
 * cachalot_moe_decode_static_scratch_bytes() is refused with CACHALOT_ESCRATCH and nothing is
 * launched (decode batches of a few tokens fit; larger ones need the caller's own workspace).  The
 * entry point calls no cudaMalloc, cudaFree or other allocating routine.
 *   - The first call on each device looks the array's device address up (with that device
 *     current); make that first call outside any stream capture.
 *   - All calls on one device share the one array: two calls that can overlap on the GPU
 *     (different streams without an ordering between them) race.  Calls on one stream are safe.
 *   - The array keeps the previous call's intermediates; no call depends on them. */
CACHALOT_API size_t cachalot_moe_decode_static_scratch_bytes(void);
CACHALOT_API int cachalot_moe_decode_static(const void* bank, const cachalot_bank_desc* desc /* host */, const void* x_bf16,
                               const int32_t* slots, const float* gate_w, int rows, int k, float swiglu_limit,
                               int numerics, void* out, int out_dtype, int* status, cachalot_stream_t stream);

/* ---- FP8 E4M3 trunk GEMV with act_quant ---------------------------------------------------- */

/* Replaces model/fp8_ref.py:27-92 quantize_activation_fp8 and model/fp8_fused_metal.py:175-233:
 * per block of `block` (32 or 128) along K: amax = max(|x|, 1e-4); scale = 2^ceil(log2(amax/448))
 * (CACHALOT_SCALE_E8M0) or amax/448 (CACHALOT_SCALE_F32); codes = E4M3FN(clip(x/scale, +-448)).
 * x bf16 [rows,K] -> codes u8 [rows,K], scales f32 [rows,K/block]. */
CACHALOT_API int cachalot_fp8_act_quant(const void* x_bf16, int rows, int k, int block, int scale_rule, uint8_t* codes,
                           float* scales, cachalot_stream_t stream);

/* Replaces model/fp8_ref.py:95-231 fp8_gemv_reference, model/fp8_gemv_metal.py:163-277 and
 * model/fp8_fused_metal.py:265-342 (fp8_linear_quantized of model/fp8_linear_metal.py:56-89):
 *   y[r,n] = sum_kb (sum_{j in kb} a[r,j] w[n,j]) * act_scale[r,kb] * wscale[n/block, kb]
 * weight u8 [N,K] raw E4M3 (codes 0x7F/0xFF read as 0); w_scales [ceil(N/block), K/block] as E8M0
 * bytes or f32 by scale_rule; out bf16 [rows,N] (f32 when out_dtype == CACHALOT_F32). */
CACHALOT_API int cachalot_fp8_gemv(const uint8_t* codes, const float* act_scales, const uint8_t* weight, const void* w_scales,
                      int scale_rule, int block, int rows, int n, int k, void* out, int out_dtype,
                      cachalot_stream_t stream);

/* Replaces model/bf16_gemv_metal.py:50-63 bf16_gemv_f32 (the output head, model/model_boundary_mlx.py:183, and any
 * other bf16 trunk matrix): out[r,n] = sum_k f32(weight[n,k]) * x[r,k], fp32 accumulation.  x f32 [rows,K] (rows <=
 * 8 share one pass over the weights), weight bf16 [N,K] row-major, K a multiple of 64 (the reference's condition),
 * out f32 [rows,N].  x and weight 16-byte aligned. */
CACHALOT_API int cachalot_bf16_gemv_f32(const float* x_f32, int rows, const void* weight_bf16, int n, int k, float* out,
                           cachalot_stream_t stream);

/* Replaces model/fp8_linear_metal.py:92-107 fp8_linear: the two calls above as one (act_quant, then the GEMV, which
 * starts to stream its weights while the quantiser still runs).  codes u8 [rows,K] and scales f32 [rows,K/block]
 * are the caller's buffers and hold the quantised activation afterwards (another projection of the same
 * activation can go on with cachalot_fp8_gemv).  The weights must not be written by the kernel that directly
 * precedes this call in the stream. */
CACHALOT_API int cachalot_fp8_linear(const void* x_bf16, int rows, int k, int block, int scale_rule, uint8_t* codes, float* scales,
                        const uint8_t* weight, const void* w_scales, int n, void* out, int out_dtype,
                        cachalot_stream_t stream);

/* Replaces model/shared_expert_metal.py:45-188 shared_expert_forward / shared_expert_forward_fused (decode, rows = 1)
 * and model/moe_prefill_batched.py:100-125 shared_expert_forward_batched (rows = M): the resident FP8 expert
 *   qx = act_quant(x);  gate = bf16(w1 qx), up = bf16(w3 qx)  (one act_quant for both);
 *   up = clip(up, +-L), gate = min(gate, L) when L > 0;  h = bf16(silu(gate) * up);  y = bf16(w2 act_quant(h))
 * and, when `addend` (f32 [rows, hidden], the routed experts' sum) is given, the layer's closing line
 * out = bf16(addend + f32(y)) of model/moe_layer_metal.py:394-403.  x bf16 [rows, hidden]; w1, w3 u8 [inter, hidden],
 * w2 u8 [hidden, inter] raw E4M3; scales as in cachalot_fp8_gemv.  w3 == NULL: w1 holds the [2*inter, hidden]
 * concatenation w1 || w3 with its scales (the reference's fused form; one GEMV).  hidden and inter must be
 * multiples of `block`.  out bf16 [rows, hidden]. */
CACHALOT_API size_t cachalot_shared_expert_workspace_bytes(int rows, int hidden, int inter, int block);
CACHALOT_API int cachalot_shared_expert(const void* x_bf16, int rows, int hidden, int inter, const uint8_t* w1,
                           const void* w1_scales, const uint8_t* w3, const void* w3_scales, const uint8_t* w2,
                           const void* w2_scales, int scale_rule, int block, float swiglu_limit, const float* addend,
                           void* workspace, size_t workspace_bytes, void* out_bf16, cachalot_stream_t stream);

/* ---- prefill: expert-major grouping, MXFP4 activations, grouped FFN ------------------------ */

/* Replaces the host-side grouping of model/moe_prefill_grouped.py:201-225 (and
 * glm/experts.py:301-303): a stable sort of the flattened [tokens*k] expert ids.
 * perm i32 [tokens*k] = flattened (token*k + route slot) ids in expert-major order, offsets
 * i32 [E+1]; ids outside [0,E) are dropped from perm (offsets[E] < tokens*k) and flagged.
 * A stable counting sort: 1024 ids per CTA, per-CTA histograms, one scan, in-order placement.
 * counts_scratch: i32 [cachalot_group_rows_scratch_ints(tokens, k, E)] device scratch. */
CACHALOT_API size_t cachalot_group_rows_scratch_ints(int tokens, int k, int n_experts);
CACHALOT_API int cachalot_group_rows(const int32_t* expert_ids, int tokens, int k, int n_experts, int32_t* perm,
                        int32_t* offsets, int32_t* counts_scratch, int* status, cachalot_stream_t stream);

/* Replaces model/fp4_act_mlx.py:101-250 (block 32, E8M0 scales) as a quantiser that keeps the
 * codes: x bf16 [rows,K] (row r read from src_rows[r] when src_rows != NULL) ->
 * codes u8 [rows,K/2] (low nibble first) + scale bytes u8 [rows,K/32]. */
CACHALOT_API int cachalot_mxfp4_act_quant(const void* x_bf16, const int32_t* src_rows, int rows, int k, uint8_t* codes,
                             uint8_t* scales, cachalot_stream_t stream);

CACHALOT_API size_t cachalot_moe_prefill_workspace_bytes(const cachalot_bank_desc* desc /* host */, int tokens, int k,
                                            int mxfp4_act);

/* Replaces the expert loop and combine of model/moe_prefill_grouped.py:384-530 with
 * model/fp4_sgmm_metal.py:318-333 / model/moe_prefill_batched.py:31-61 /
 * model/expert_affine.py:84-99 as the per-expert op: rows grouped by (perm, offsets) run through
 * their expert once, results are kept per route slot and summed in slot order 0..k-1.
 * x bf16 [tokens,H]; slot_of_expert i32 [E] maps expert id -> bank slot (-1 = absent -> zeros);
 * gate_w f32 [tokens,k]; mxfp4_act != 0 quantises x and the hidden activation to MXFP4 per 32
 * first: 1 = on the block-scaled FP4 tensor cores when the bank is FP4 (grouped GEMM, weights as
 * the M side), 2 = always on the plain per-row kernels (the same arithmetic in a fixed summation
 * order, kept as the check for 1).  mxfp4_act = 0 keeps the bf16 activations and the reference's per-expert
 * rounding points (g, u, h and each expert's output rounded to bf16); on an FP4 bank this also runs on the tensor
 * cores, every activation row as four residual MXFP4 rows whose sum reproduces the bf16 values to 2.4e-4 (a result
 * that sat on a bf16 rounding boundary may come out one step away from the per-row kernels').  out f32 [tokens,H].
 * tokens * k <= 65535 only where the per-row kernels run (2-bit banks, mxfp4_act = 2). */
CACHALOT_API int cachalot_moe_prefill(const void* bank, const cachalot_bank_desc* desc /* host */, const void* x_bf16,
                         const int32_t* perm, const int32_t* offsets, const int32_t* slot_of_expert,
                         const float* gate_w, int tokens, int k, int n_experts, float swiglu_limit, int mxfp4_act,
                         void* workspace, size_t workspace_bytes, float* out, int* status,
                         cachalot_stream_t stream);

/* The two halves of cachalot_moe_prefill that an expert-parallel rank runs on either side of its
 * exchanges (no counterpart in the single-device reference; the arithmetic is that of
 * cachalot_moe_prefill with mxfp4_act = 1).
 * cachalot_moe_prefill_rows: rows already quantised to MXFP4 (cachalot_mxfp4_act_quant) and laid
 * out in segments -- seg_offsets i32 [n_segments+1] (device), segment g holds rows of the expert
 * in bank slot seg_slot[g] (NULL: slot g; negative or out of range: absent, its rows come back as
 * zeros); row_weights f32 [rows] = the router weight of every row -> y bf16 [rows, H], the
 * expert output of every row (gate/up, SwiGLU, weight, MXFP4 of the hidden activation, down).
 * FP4 bank only.  cachalot_moe_combine_rows: out[t,:] = sum over j = 0..k-1, in that order, of
 * y[inv[t*k+j],:], skipping inv < 0. */
CACHALOT_API size_t cachalot_moe_prefill_rows_workspace_bytes(const cachalot_bank_desc* desc /* host */, long long rows, int n_segments);
CACHALOT_API int cachalot_moe_prefill_rows(const void* bank, const cachalot_bank_desc* desc /* host */, const uint8_t* x_codes,
                              const uint8_t* x_scales, const float* row_weights, const int32_t* seg_offsets,
                              const int32_t* seg_slot, int n_segments, long long rows, float swiglu_limit, void* workspace,
                              size_t workspace_bytes, void* y_bf16, int* status, cachalot_stream_t stream);
CACHALOT_API int cachalot_moe_combine_rows(const void* y_bf16, const int32_t* inv, int tokens, int k, int hidden, float* out,
                              cachalot_stream_t stream);

/* ---- expert-parallel decode: sum of the ranks' partial outputs over peer memory ------------- */

/* No counterpart in the reference (it is single-device).  Every rank r owns, in memory that all
 * ranks of the box can write (CUDA IPC / a symmetric allocation made by the host), an inbox of
 * cachalot_peer_sum_inbox_bytes(world, n) bytes and a flag array of cachalot_peer_sum_flag_bytes
 * bytes, both zeroed once before the first call; inbox_ptrs[r] / flag_ptrs[r] (host arrays of
 * device pointers, as mapped in THIS process) are rank r's.  epoch: u32 [2] in local device
 * memory, zeroed once.  Every rank calls with its own partial f32 [n]; out f32 [n] receives the
 * sum in rank order on every rank.  All ranks must make the same sequence of calls; a peer that
 * does not show up makes the bounded wait expire (CACHALOT_STATUS_WAIT_EXPIRED in *status) and
 * the call returns with an incomplete sum instead of hanging.  world <= 8, n a multiple of 4. */
CACHALOT_API size_t cachalot_peer_sum_inbox_bytes(int world, int n);
CACHALOT_API size_t cachalot_peer_sum_flag_bytes(int world);
CACHALOT_API int cachalot_peer_sum(void* const* inbox_ptrs /* host */, void* const* flag_ptrs /* host */, int world, int rank,
                      const float* partial, float* out, int n, uint32_t* epoch, int* status, cachalot_stream_t stream);

/* No counterpart in the reference.  cachalot_moe_layer_decode for an expert-parallel rank with the sum over the ranks
 * done in the tail of the same launch: every thread that owns an output element stores it into row `rank` of every
 * rank's inbox as one 64-bit word (fp32 value | number of the exchange << 32; plain peer stores over NVLink, no
 * multicast, no flag, no fence), reads the same element of every rank's row in its own inbox until the word carries
 * this exchange's number, and adds the values in rank order, so `out` holds the full layer output on every rank and
 * all ranks hold the same bits.  The ranks must run on GPUs with the same number of SMs and make the same sequence
 * of calls; a peer that does not show up makes the bounded wait expire (CACHALOT_STATUS_WAIT_EXPIRED), its values
 * count as zero and the call returns instead of hanging.  inbox[r] (device pointer as mapped in THIS process): rank
 * r's inbox of cachalot_peer_layer_inbox_bytes(world, hidden) bytes in memory every rank can write, 16-byte aligned,
 * zeroed once; epoch: u32 [2] in local device memory, zeroed once.  Only bank shapes and top-k the single-launch
 * kernel covers (else CACHALOT_EUNSUPPORTED: use cachalot_peer_sum).  The launch takes every SM and waits for its
 * peers: do not let a kernel of another stream that itself waits for peers (an NCCL collective) run between two
 * queued calls, or the two can block each other across ranks until the bounded wait expires. */
typedef struct {
  void* inbox[8];
  uint32_t* epoch;
  int32_t world, rank;
} cachalot_peer_ctx;
CACHALOT_API size_t cachalot_peer_layer_inbox_bytes(int world, int hidden);
CACHALOT_API int cachalot_moe_layer_decode_peer(const void* bank, const cachalot_bank_desc* desc /* host */, const void* x_bf16,
                                   const float* logits, const float* bias, const int32_t* slot_table, int layer,
                                   int n_experts, int k, int mode, float gate_temp, float route_scale, int norm_topk_prob,
                                   int weights_bf16, float swiglu_limit, int numerics, void* workspace,
                                   size_t workspace_bytes, void* out, int out_dtype, int32_t* indices_out,
                                   float* weights_out, const cachalot_peer_ctx* peer /* host */, int* status,
                                   cachalot_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* CACHALOT_B200_H */
