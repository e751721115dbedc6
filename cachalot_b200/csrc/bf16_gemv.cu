// bf16-weight GEMV with fp32 activations and fp32 accumulation: the output head (and any other bf16 trunk matrix).
// The reference reads the bf16 bits once and widens them in registers (model/bf16_gemv_metal.py:20-63): out[n] =
// sum_k f32(w[n, k]) * x[k], one SIMD group per row.  Here: persistent CTAs (a few per SM) stage the activation rows
// in shared memory once, then every warp walks rows n = warp, warp + W, ...; a lane reads 16 bytes (8 weights) per
// step with streaming loads, several in flight, and the lanes' partial sums meet in a shuffle tree.  Up to eight
// activation rows share one pass over the weights; from two rows up a warp takes four weight rows at a time so that
// an activation read from shared memory serves four of them.  HBM-bound: N * K * 2 bytes per call.
#include "common.cuh"

namespace cachalot {
namespace {

constexpr int BG_THREADS = 256;       // threads of a CTA; 512 where the staged activations leave room for one CTA per SM only

__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// 8 weights of WR weight rows against the same 8 activations of ROWS activation rows: an activation is read from shared
// memory once for WR weight rows (with one weight row per warp, two or more activation rows made the kernel
// shared-memory bound)
template <int ROWS, int WR>
__device__ __forceinline__ void fma8(float (&acc)[ROWS][WR], const uint4 (&w)[WR], const float* xs, int k, int col) {
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const float4 a = *reinterpret_cast<const float4*>(xs + (size_t)r * k + col);
    const float4 b = *reinterpret_cast<const float4*>(xs + (size_t)r * k + col + 4);
    const float xv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < WR; ++j) {
      const uint32_t ww[4] = {w[j].x, w[j].y, w[j].z, w[j].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[r][j] = fmaf(__uint_as_float(ww[i] << 16), xv[2 * i], acc[r][j]);
        acc[r][j] = fmaf(__uint_as_float(ww[i] & 0xffff0000u), xv[2 * i + 1], acc[r][j]);
      }
    }
  }
}

template <int ROWS, int WR, int UNROLL, int THREADS>
__global__ void __launch_bounds__(THREADS) bf16_gemv_kernel(const float* __restrict__ x, const __nv_bfloat16* __restrict__ w, int n, int k,
                                                               float* __restrict__ out) {
  extern __shared__ __align__(16) float xs[];  // [ROWS][k]
  for (int i = threadIdx.x * 4; i < ROWS * k; i += THREADS * 4)
    *reinterpret_cast<float4*>(xs + i) = *reinterpret_cast<const float4*>(x + i);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (THREADS / 32);
  const int steps = k / 256;  // a warp step covers 256 weights of a row
  const int groups = (n + WR - 1) / WR;  // a warp walks groups of WR consecutive weight rows
  for (int gq = blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5); gq < groups; gq += warps) {
    const __nv_bfloat16* wr[WR];
#pragma unroll
    for (int j = 0; j < WR; ++j) {
      const int row = gq * WR + j < n ? gq * WR + j : n - 1;  // past the end: the last row again, never stored
      wr[j] = w + (size_t)row * k + lane * 8;
    }
    float acc[ROWS][WR];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
      for (int j = 0; j < WR; ++j) acc[r][j] = 0.f;
    int s = 0;
    for (; s + UNROLL <= steps; s += UNROLL) {
      uint4 v[UNROLL][WR];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u)
#pragma unroll
        for (int j = 0; j < WR; ++j) v[u][j] = ld_stream_v4(wr[j] + (size_t)(s + u) * 256);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) fma8<ROWS, WR>(acc, v[u], xs, k, (s + u) * 256 + lane * 8);
    }
    for (; s < steps; ++s) {
      uint4 v[WR];
#pragma unroll
      for (int j = 0; j < WR; ++j) v[j] = ld_stream_v4(wr[j] + (size_t)s * 256);
      fma8<ROWS, WR>(acc, v, xs, k, s * 256 + lane * 8);
    }
    // the part of the rows past the last whole step (K is a multiple of 64: 8 weights for some of the lanes)
    const int col = steps * 256 + lane * 8;
    if (col < k) {
      uint4 v[WR];
#pragma unroll
      for (int j = 0; j < WR; ++j) v[j] = ld_stream_v4(wr[j] + (size_t)steps * 256);
      fma8<ROWS, WR>(acc, v, xs, k, col);
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
      for (int j = 0; j < WR; ++j) {
        const float t = warp_sum(acc[r][j]);
        if (lane == 0 && gq * WR + j < n) out[(size_t)r * n + gq * WR + j] = t;
      }
  }
}

}  // namespace
}  // namespace cachalot

using namespace cachalot;

extern "C" int cachalot_bf16_gemv_f32(const float* x_f32, int rows, const void* weight_bf16, int n, int k, float* out,
                                      cachalot_stream_t stream) {
  if (!x_f32 || !weight_bf16 || !out) return fail(CACHALOT_EINVAL, "bf16_gemv: null pointer");
  if (n <= 0 || k <= 0 || k % 64) return fail(CACHALOT_EINVAL, "in_features must be a multiple of 64");
  if (rows < 0 || rows > 8) return fail(CACHALOT_EUNSUPPORTED, "bf16_gemv: %d activation rows (at most 8 per call)", rows);
  if (!aligned(x_f32, 16) || !aligned(weight_bf16, 16)) return fail(CACHALOT_EALIGN, "bf16_gemv: x and weight need 16-byte alignment");
  if (rows == 0) return CACHALOT_OK;
  const size_t smem = (size_t)rows * k * sizeof(float);
  if (smem > 200 * 1024) return fail(CACHALOT_EUNSUPPORTED, "bf16_gemv: %d rows of %d activations do not fit shared memory", rows, k);
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return fail(CACHALOT_ECUDA, "bf16_gemv: cannot read the SM count");
  // CTAs per SM: as many as the staged activations leave room for, at most 6 (48 warps)
  int per_sm = (int)((220 * 1024) / (smem + 1024));
  per_sm = per_sm < 1 ? 1 : (per_sm > 6 ? 6 : per_sm);
  const int wrows = rows == 1 ? 1 : 4;  // weight rows a warp takes at a time
  const int threads = per_sm == 1 && rows >= 6 ? 2 * BG_THREADS : BG_THREADS;  // sixteen warps per SM either way
  const long long want = (((long long)n + wrows - 1) / wrows + threads / 32 - 1) / (threads / 32);
  const unsigned grid = (unsigned)(want < (long long)sms * per_sm ? want : (long long)sms * per_sm);
  cudaStream_t s = (cudaStream_t)stream;
  const __nv_bfloat16* w = static_cast<const __nv_bfloat16*>(weight_bf16);
  cudaError_t e = cudaSuccess;
  auto go = [&](auto kern) {
    if (smem > 48 * 1024) e = smem_optin_once(kern, 200 * 1024);
    if (e == cudaSuccess) kern<<<grid, threads, smem, s>>>(x_f32, w, n, k, out);
  };
  switch (rows) {
    case 1: go(bf16_gemv_kernel<1, 1, 4, BG_THREADS>); break;  // one weight row per warp, four 16-byte loads in flight per lane
    case 2: go(bf16_gemv_kernel<2, 4, 1, BG_THREADS>); break;  // four weight rows per warp share every activation read
    case 3: go(bf16_gemv_kernel<3, 4, 1, BG_THREADS>); break;
    case 4: go(bf16_gemv_kernel<4, 4, 1, BG_THREADS>); break;
    case 5: go(bf16_gemv_kernel<5, 4, 1, BG_THREADS>); break;
    case 6: threads > BG_THREADS ? go(bf16_gemv_kernel<6, 4, 1, 2 * BG_THREADS>) : go(bf16_gemv_kernel<6, 4, 1, BG_THREADS>); break;
    case 7: threads > BG_THREADS ? go(bf16_gemv_kernel<7, 4, 1, 2 * BG_THREADS>) : go(bf16_gemv_kernel<7, 4, 1, BG_THREADS>); break;
    default: threads > BG_THREADS ? go(bf16_gemv_kernel<8, 4, 1, 2 * BG_THREADS>) : go(bf16_gemv_kernel<8, 4, 1, BG_THREADS>); break;
  }
  if (e != cudaSuccess) return fail(CACHALOT_ECUDA, "bf16_gemv: %s", cudaGetErrorString(e));
  return check_launch("bf16_gemv");
}
