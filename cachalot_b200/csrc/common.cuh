// Shared helpers for the sm_100a kernels: error plumbing, cache-hinted loads, small numeric
// conversions.  Everything here is header-only and internal to the library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <mutex>
#include <set>
#include <utility>

#include "../../include/cachalot_b200.h"

namespace cachalot {

void set_error(const char* fmt, ...);

inline int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  set_error("%s", buf);
  return code;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(CACHALOT_ECUDA, "%s: %s", what, cudaGetErrorString(e));
  return CACHALOT_OK;
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ---- device helpers ---------------------------------------------------------------------

// 128-bit streaming load: weights are read exactly once, so keep them out of L1.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_stream_u2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_stream_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// 2**(raw-127) for an E8M0 byte, exact: normal floats for raw >= 1, the denormal 2**-127 for raw == 0.
__device__ __forceinline__ float e8m0_to_f32(uint32_t raw) {
  return raw ? __uint_as_float(raw << 23) : __uint_as_float(0x00400000u);
}

// E2M1 code (low 3 bits = magnitude index, bit 3 = sign) -> float.  Magnitudes 0,.5,1,1.5,2,3,4,6;
// code 8 gives +0.0 like the reference's table.
__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
  // magnitude m: e = m>>1, f = m&1.  e==0: f*0.5 ; else 2**(e-1) * (1 + f/2)
  uint32_t m = code & 7u;
  uint32_t e = m >> 1, f = m & 1u;
  uint32_t bits = e ? (((e + 126u) << 23) | (f << 22)) : (f ? 0x3F000000u : 0u);
  if ((code & 8u) && m) bits |= 0x80000000u;
  return __uint_as_float(bits);
}

// E2M1 nearest with ties to even, as a threshold chain (the reference's explicit table)
__device__ __forceinline__ uint32_t e2m1_round_code(float v) {
  float a = fabsf(v);
  uint32_t mag = a <= 0.25f ? 0u : a < 0.75f ? 1u : a <= 1.25f ? 2u : a < 1.75f ? 3u : a <= 2.5f ? 4u : a < 3.5f ? 5u : a <= 5.0f ? 6u : 7u;
  return mag | ((__float_as_uint(v) >> 28) & 8u);
}

// block scale of MXFP4: 2**ceil(log2(max(amax, 6*2**-126) / 6)); returns the exponent.  With
// amax = m * 2**E (1 <= m < 2) the fp32 quotient amax/6 is at most 2**(E-2) exactly when m <= 1.5, so the
// answer is E-2, plus one when the mantissa is above 1.5 (checked against the division form over all
// exponents and 2e8 random values).
__device__ __forceinline__ int mxfp4_exponent(float amax) {
  const uint32_t b = __float_as_uint(fmaxf(amax, 6.0f * 1.1754943508222875e-38f));
  return (int)(b >> 23) - 129 + ((b & 0x7fffffu) > 0x400000u ? 1 : 0);
}

// two floats -> one byte of E2M1 codes (lo in bits 0-3), round to nearest even, saturating at +-6
__device__ __forceinline__ uint32_t e2m1x2_byte(float lo, float hi) {
  uint32_t r;
  asm("{\n.reg .b8 t;\ncvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\nmov.b32 %0, {t, t, t, t};\n}" : "=r"(r) : "f"(hi), "f"(lo));
  return r & 0xffu;
}

__device__ __forceinline__ float pow2f(int e) {  // e in [-127, 127]
  return e >= -126 ? __uint_as_float((uint32_t)(e + 127) << 23) : __uint_as_float(0x00400000u);
}

// SwiGLU with the reference's clamp: up both sides, gate from above only, when limit > 0.
__device__ __forceinline__ float swiglu(float g, float u, float limit) {
  if (limit > 0.f) {
    u = fminf(fmaxf(u, -limit), limit);
    g = fminf(g, limit);
  }
  return g / (1.0f + expf(-g)) * u;
}


// Router score and selection key of one expert (both routers, one arithmetic):
//   SQRT_SOFTPLUS: score = sqrt(softplus(raw / temp)), key = score + bias (higher first, ties to the larger index)
//   SIGMOID:       score = sigmoid(raw) as y = 1/(1+exp(|x|)), x < 0 ? y : 1-y;  key = -(score + bias) (lower
//                  first, ties to the lower index)
__device__ __forceinline__ void router_score_key(int mode, float raw, float b, float gate_temp, float& score, float& key) {
  if (mode == CACHALOT_ROUTER_SQRT_SOFTPLUS) {
    const float s = raw / gate_temp;
    const float sp = fmaxf(s, 0.f) + logf(1.0f + expf(-fabsf(s)));
    score = sqrtf(sp);
    key = score + b;
  } else {
    const float y = 1.0f / (1.0f + expf(fabsf(raw)));
    score = raw < 0.f ? y : 1.0f - y;
    key = -(score + b);
  }
}
// true when expert (ka, ia) is selected before expert (kb, ib)
__device__ __forceinline__ bool router_before(int mode, float ka, int ia, float kb, int ib) {
  if (mode == CACHALOT_ROUTER_SQRT_SOFTPLUS) return ka > kb || (ka == kb && ia > ib);
  return ka < kb || (ka == kb && ia < ib);
}

// The dynamic shared-memory opt-in is an attribute of a kernel on a device: set it the first time a kernel is launched
// on a device, not on every launch (the pointer types of different instantiations coincide, so the record is keyed
// by the pointer's value).  `bytes` must be the same for every call with one kernel.
template <typename K>
inline cudaError_t smem_optin_once(K kern, int bytes) {
  static std::mutex mu;
  static std::set<std::pair<const void*, int>> done;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  if (done.count({(const void*)kern, dev})) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done.insert({(const void*)kern, dev});
  return e;
}

}  // namespace cachalot
