// Internal launch helpers shared between translation units.
#pragma once
#include "common.cuh"

namespace cachalot {

// In-place MXFP4 round trip (quantise per 32 along K to E2M1 codes with an E8M0 scale, then
// decode) of a float32 [rows, k] array.
int launch_mxfp4_roundtrip_f32(float* data, long long rows, int k, cudaStream_t stream);
// bf16 [rows,k] -> bf16 [rows,k] round trip (every MXFP4 value is exact in bf16).
int launch_mxfp4_roundtrip_bf16(const __nv_bfloat16* in, __nv_bfloat16* out, long long rows, int k, cudaStream_t stream);

struct BankView {
  const uint8_t* base;
  long long record_bytes;
  long long off[9];
  int n_slots, hidden, inter, bits, group, scale_dtype;
  int format;        // CACHALOT_BANK_*
  int scale_centre;  // FP4: E8M0 byte the tensor-core path scales relative to
};

template <int FMT>
struct Fmt;
template <>
struct Fmt<CACHALOT_BANK_FP4> {
  static constexpr int CH = 32;  // elements per 16-byte chunk
};
template <>
struct Fmt<CACHALOT_BANK_AFFINE> {
  static constexpr int CH = 64;  // 2-bit codes per 16-byte chunk
};


// Grouping of the routed rows r = token*k + route slot by bank slot, so that a slot's bytes are
// streamed once for all rows that use it.  Null pointers mean "every row is its own group".
struct Plan {
  const int32_t* group_start;  // [n_groups + 1] offsets into order
  const int32_t* order;        // [rows] row ids sorted by slot (stable)
  const int32_t* group_slot;   // [n_groups]
  const int32_t* n_groups;     // device scalar
};

// Tensor-core decode path (moe_decode_mma.cu).  Returns CACHALOT_EUNSUPPORTED without launching
// when the shape is outside what it handles, so the caller can use the simple kernels.
int launch_decode_mma(const BankView& v, const void* x, const int32_t* slots, const float* gate_w, int rows, int k,
                      float limit, int numerics_flags, void* workspace, void* out, int out_dtype, int* status,
                      cudaStream_t stream);
size_t decode_mma_workspace_bytes(int hidden, int inter, int rows, int k);
bool decode_mma_supported(const BankView& v, int rows, int k);


// Expert-parallel exchange done in the tail of the single-launch decode kernel: every rank's inbox (u64
// [2 slots][world][hidden]: fp32 value | number of the exchange << 32) as mapped in this process, the device-resident
// exchange counter, and this rank.  world == 0: no exchange.
constexpr int PEER_LINK_MAX = 8;
struct PeerLink {
  unsigned long long* inbox[PEER_LINK_MAX];
  uint32_t* epoch;  // u32 [2]: exchanges done, arrival ticket
  int world, rank;
};

// Single-launch decode for one token (moe_decode_fused.cu).  Same contract as launch_decode_mma.
int launch_decode_fused(const BankView& v, const void* x, const int32_t* slots, const float* gate_w, int rows, int k,
                        float limit, int numerics_flags, void* workspace, void* out, int out_dtype, int* status,
                        cudaStream_t stream);
size_t decode_fused_workspace_bytes(int hidden, int inter, int rows, int k);
bool decode_fused_supported(const BankView& v, int rows, int k);
// ... with the routing tail (scores, top-k, weights, slot lookup) done inside the same launch
int launch_layer_fused(const BankView& v, const void* x, const float* logits, const float* bias, const int32_t* slot_table,
                       int layer, int n_experts, int k, int mode, float gate_temp, float route_scale, int norm,
                       int weights_bf16, float limit, int numerics_flags, void* workspace, void* out, int out_dtype,
                       int32_t* indices_out, float* weights_out, int* status, cudaStream_t stream,
                       const PeerLink* peer = nullptr);
bool layer_fused_supported(const BankView& v, int n_experts, int k);


// Prefill on the block-scaled FP4 tensor cores (prefill_tc.cu): FP4 bank, MXFP4 activations.
int launch_prefill_tc(const BankView& v, const void* x_bf16, const int32_t* perm, const int32_t* offsets,
                      const int32_t* slot_of_expert, const float* gate_w, int tokens, int k, int n_experts, float limit,
                      void* workspace, float* out, int* status, cudaStream_t stream);
size_t prefill_tc_workspace_bytes(int hidden, int inter, int tokens, int k, int n_experts);
// the same from already quantised rows laid out in segments, up to the per-row outputs (what an expert-parallel
// rank runs between the dispatch and the combine exchange), and the slot-ordered sum of a token's rows
int launch_prefill_rows(const BankView& v, const uint8_t* x_codes, const uint8_t* x_scales, const float* row_w,
                        const int32_t* seg_offsets, const int32_t* seg_slot, int n_seg, long long rows, float limit, bool zero_absent,
                        void* workspace, __nv_bfloat16* y, int* status, cudaStream_t stream);
size_t prefill_rows_workspace_bytes(int inter, long long rows, int n_seg);
int launch_combine_rows(const __nv_bfloat16* y, const int32_t* inv, int tokens, int k, int hidden, float* out, cudaStream_t stream);
bool prefill_tc_supported(const BankView& v);
// decode batches through the same grouped kernels (FP4 bank, fp32 numerics), every distinct expert streamed once
int launch_decode_tc(const BankView& v, const void* x_bf16, const int32_t* slots, const float* gate_w, int rows, int k, float limit,
                     void* workspace, void* out, int out_dtype, int* status, cudaStream_t stream, bool round_bf16 = false);
// Expert-major prefill with bf16 activations as they are and the reference's per-expert rounding points, on the same
// grouped kernels (prefill_tc.cu).
size_t prefill_exact_workspace_bytes(int hidden, int inter, int tokens, int k, int n_experts);
int launch_prefill_exact(const BankView& v, const void* x_bf16, const int32_t* perm, const int32_t* offsets, const int32_t* slot_of_expert,
                         const float* gate_w, int tokens, int k, int n_experts, float limit, void* workspace, float* out, int* status,
                         cudaStream_t stream);
size_t decode_tc_workspace_bytes(int hidden, int inter, int rows, int k);
bool decode_tc_supported(const BankView& v, int rows, int k);

}  // namespace cachalot
