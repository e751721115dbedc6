// FP8 E4M3 trunk GEMV with dynamic activation quantisation (act_quant).
#include <cuda_fp8.h>

#include "common.cuh"

namespace cachalot {

// ceil(log2(v)) for a positive normal float, exact (no libm rounding near powers of two)
__device__ __forceinline__ int ceil_log2(float v) {
  uint32_t b = __float_as_uint(v);
  return (int)((b >> 23) & 0xffu) - 127 + ((b & 0x7fffffu) ? 1 : 0);
}

// one warp per (row, block); block = 32 * PER
template <int PER>
__global__ void act_quant_kernel(const __nv_bfloat16* __restrict__ x, int rows, int k, int scale_rule,
                                 uint8_t* __restrict__ codes, float* __restrict__ scales) {
  constexpr int BLOCK = 32 * PER;
  const int nblk = k / BLOCK;
  long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)rows * nblk) return;
  const size_t base = (size_t)warp * BLOCK + (size_t)lane * PER;  // rows are contiguous, so warp*BLOCK is the flat offset
  float v[PER];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    v[i] = __bfloat162float(x[base + i]);
    amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = fmaxf(warp_max(amax), 1e-4f);
  float raw = __fdiv_rn(amax, 448.0f);
  float scale = raw;
  if (scale_rule == CACHALOT_SCALE_E8M0) scale = __uint_as_float((uint32_t)(ceil_log2(raw) + 127) << 23);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    float q = fminf(fmaxf(__fdiv_rn(v[i], scale), -448.0f), 448.0f);
    codes[base + i] = (uint8_t)__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3);
  }
  if (lane == 0) scales[warp] = scale;
}

// four E4M3 codes -> four floats; the two NaN encodings (0x7F, 0xFF) read as zero like the
// reference's decode table
__device__ __forceinline__ void e4m3x4_to_f32(uint32_t w, float* o) {
  uint32_t nan_mask = __vcmpeq4(w & 0x7F7F7F7Fu, 0x7F7F7F7Fu);
  w &= ~nan_mask;
  __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xffffu), __NV_E4M3);
  __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3);
  float2 a = __half22float2(*reinterpret_cast<__half2*>(&lo));
  float2 b = __half22float2(*reinterpret_cast<__half2*>(&hi));
  o[0] = a.x;
  o[1] = a.y;
  o[2] = b.x;
  o[3] = b.y;
}

constexpr int GEMV_WARPS = 8;

// grid = (ceil(N / 8), rows): one warp per (token, output row).  Activations are decoded once
// per CTA into shared memory (16-element chunks, chunk-transposed); each lane multiplies its
// 16-byte weight chunks and applies act_scale * weight_scale of the chunk's K-block to the
// chunk's partial sum before accumulating, which is the reference's per-block scale placement.
template <typename OutT>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
fp8_gemv_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ act_scales,
                const uint8_t* __restrict__ weight, const void* __restrict__ w_scales, int scale_rule, int block,
                int n_out, int k, OutT* __restrict__ out) {
  extern __shared__ float smem[];
  const int nch = k / 16, nkb = k / block;
  float* xs = smem;             // [16][nch]
  float* as = smem + k;         // [nkb]
  const int t = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t* crow = reinterpret_cast<const uint32_t*>(codes + (size_t)t * k);
  for (int w = threadIdx.x; w < k / 4; w += blockDim.x) {
    float f[4];
    e4m3x4_to_f32(crow[w], f);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int e = w * 4 + i;
      xs[(e & 15) * nch + (e >> 4)] = f[i];
    }
  }
  for (int b = threadIdx.x; b < nkb; b += blockDim.x) as[b] = act_scales[(size_t)t * nkb + b];
  __syncthreads();
  const int n = blockIdx.x * GEMV_WARPS + warp;
  if (n >= n_out) return;
  const uint8_t* wrow = weight + (size_t)n * k;
  const size_t srow = (size_t)(n / block) * nkb;
  float acc = 0.f;
  for (int c = lane; c < nch; c += 32) {
    uint4 v = ld_stream_u4(wrow + (size_t)c * 16);
    uint32_t words[4] = {v.x, v.y, v.z, v.w};
    float part = 0.f;
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
      float f[4];
      e4m3x4_to_f32(words[wi], f);
#pragma unroll
      for (int i = 0; i < 4; ++i) part = fmaf(f[i], xs[(wi * 4 + i) * nch + c], part);
    }
    const int kb = (c * 16) / block;
    float ws = scale_rule == CACHALOT_SCALE_E8M0 ? e8m0_to_f32(reinterpret_cast<const uint8_t*>(w_scales)[srow + kb])
                                                 : reinterpret_cast<const float*>(w_scales)[srow + kb];
    acc = fmaf(part, as[kb] * ws, acc);
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    if constexpr (sizeof(OutT) == 2)
      out[(size_t)t * n_out + n] = __float2bfloat16_rn(acc);
    else
      out[(size_t)t * n_out + n] = acc;
  }
}

}  // namespace cachalot

using namespace cachalot;

extern "C" int cachalot_fp8_act_quant(const void* x_bf16, int rows, int k, int block, int scale_rule, uint8_t* codes,
                                      float* scales, cachalot_stream_t stream) {
  if (!x_bf16 || !codes || !scales) return fail(CACHALOT_EINVAL, "fp8_act_quant: null pointer");
  if (block != 32 && block != 128) return fail(CACHALOT_EUNSUPPORTED, "fp8_act_quant: block=%d (32 or 128)", block);
  if (rows < 0 || k <= 0 || k % block) return fail(CACHALOT_EINVAL, "K=%d must be divisible by block_size=%d", k, block);
  if (scale_rule != CACHALOT_SCALE_E8M0 && scale_rule != CACHALOT_SCALE_F32) return fail(CACHALOT_EINVAL, "fp8_act_quant: unknown scale rule");
  if (rows == 0) return CACHALOT_OK;
  long long warps = (long long)rows * (k / block);
  int threads = 256;
  unsigned blocks = (unsigned)((warps * 32 + threads - 1) / threads);
  if (block == 32)
    act_quant_kernel<1><<<blocks, threads, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x_bf16, rows, k, scale_rule, codes, scales);
  else
    act_quant_kernel<4><<<blocks, threads, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x_bf16, rows, k, scale_rule, codes, scales);
  return check_launch("fp8_act_quant");
}

extern "C" int cachalot_fp8_gemv(const uint8_t* codes, const float* act_scales, const uint8_t* weight,
                                 const void* w_scales, int scale_rule, int block, int rows, int n, int k, void* out,
                                 int out_dtype, cachalot_stream_t stream) {
  if (!codes || !act_scales || !weight || !w_scales || !out) return fail(CACHALOT_EINVAL, "fp8_gemv: null pointer");
  if (block != 32 && block != 128) return fail(CACHALOT_EUNSUPPORTED, "fp8_gemv: block=%d (32 or 128)", block);
  if (rows < 0 || n <= 0 || k <= 0 || k % block) return fail(CACHALOT_EINVAL, "K=%d is not divisible by %d", k, block);
  if (rows > 65535) return fail(CACHALOT_EINVAL, "fp8_gemv: rows=%d exceeds 65535", rows);
  if (scale_rule != CACHALOT_SCALE_E8M0 && scale_rule != CACHALOT_SCALE_F32) return fail(CACHALOT_EINVAL, "fp8_gemv: unknown scale rule");
  if (out_dtype != CACHALOT_BF16 && out_dtype != CACHALOT_F32) return fail(CACHALOT_EINVAL, "fp8_gemv: out dtype must be bf16 or f32");
  if (!aligned(weight, 16) || !aligned(codes, 4)) return fail(CACHALOT_EALIGN, "fp8_gemv: weight needs 16-byte, codes 4-byte alignment");
  if (rows == 0) return CACHALOT_OK;
  size_t smem = (size_t)k * 4 + (size_t)(k / block) * 4;
  if (smem > 200 * 1024) return fail(CACHALOT_EINVAL, "fp8_gemv: K=%d too large", k);
  static bool attr_done = false;
  if (!attr_done) {
    cudaFuncSetAttribute(fp8_gemv_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    cudaFuncSetAttribute(fp8_gemv_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    attr_done = true;
  }
  dim3 grid((n + GEMV_WARPS - 1) / GEMV_WARPS, rows);
  if (out_dtype == CACHALOT_BF16)
    fp8_gemv_kernel<__nv_bfloat16><<<grid, GEMV_WARPS * 32, smem, (cudaStream_t)stream>>>(codes, act_scales, weight, w_scales, scale_rule, block, n, k, (__nv_bfloat16*)out);
  else
    fp8_gemv_kernel<float><<<grid, GEMV_WARPS * 32, smem, (cudaStream_t)stream>>>(codes, act_scales, weight, w_scales, scale_rule, block, n, k, (float*)out);
  return check_launch("fp8_gemv");
}
