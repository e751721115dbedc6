// Internal launch helpers shared between translation units.
#pragma once
#include "common.cuh"

namespace cachalot {

// In-place MXFP4 round trip (quantise per 32 along K to E2M1 codes with an E8M0 scale, then
// decode) of a float32 [rows, k] array.
int launch_mxfp4_roundtrip_f32(float* data, long long rows, int k, cudaStream_t stream);
// bf16 [rows,k] -> bf16 [rows,k] round trip (every MXFP4 value is exact in bf16).
int launch_mxfp4_roundtrip_bf16(const __nv_bfloat16* in, __nv_bfloat16* out, long long rows, int k, cudaStream_t stream);

}  // namespace cachalot
