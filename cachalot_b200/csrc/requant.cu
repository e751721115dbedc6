// FP4 (E2M1 / E8M0) -> affine re-quantiser: builds the 2-bit (or 4-bit) group-quantised form of a weight matrix from
// its FP4 bytes on the GPU.  Per group of 64 or 128 consecutive elements of a row, one warp:
//   min/max fit -> 5 x 5 grid search over shrunk ranges (lowest squared error, earlier candidate on ties)
//   -> least-squares refinement (assign levels, refit the line in closed form, scale and bias rounded to the storage
//      dtype on every iteration, best iterate kept) -> levels against the rounded scale and bias -> packed words.
// The arithmetic follows benchmarks/quant_affine.py:113-123, 138-193, 213-251, 303-329 of the reference step by
// step in fp32; sums over a group are warp-shuffle trees, so a scale may differ from a sequential sum's in the last
// bit before it is rounded to f16 / bf16.
#include "common.cuh"

namespace cachalot {
namespace {

__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <int SDT>
__device__ __forceinline__ float store_round(float v) {
  if constexpr (SDT == CACHALOT_F16) return __half2float(__float2half_rn(v));
  return bf16_round(v);
}

template <int PER>
__device__ __forceinline__ float group_error(const float (&w)[PER], float scale, float bias, float levels) {
  float e = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const float q = fminf(fmaxf(rintf(__fdiv_rn(w[i] - bias, scale)), 0.f), levels);
    const float d = scale * q + bias - w[i];
    e += d * d;
  }
  return warp_sum(e);
}

template <int PER, int SDT>
__global__ void requant_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales, long long n_groups, int k, int bits,
                               int iters, uint32_t* __restrict__ out_words, void* __restrict__ out_scales, void* __restrict__ out_biases) {
  constexpr int GROUP = 32 * PER;
  const long long grp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (grp >= n_groups) return;
  const float levels = (float)((1 << bits) - 1);
  float w[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const long long flat = grp * GROUP + lane * PER + i;
    const long long row = flat / k;
    const int col = (int)(flat - row * k);
    const uint8_t byte = packed[row * (k / 2) + (col >> 1)];
    w[i] = e2m1_to_f32((col & 1) ? byte >> 4 : byte & 15u) * e8m0_to_f32(scales[row * (k / 32) + (col >> 5)]);
  }
  float lo = w[0], hi = w[0], sw = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) lo = fminf(lo, w[i]), hi = fmaxf(hi, w[i]), sw += w[i];
  lo = warp_min(lo), hi = warp_max(hi), sw = warp_sum(sw);
  const float mid = (lo + hi) / 2.f;
  float best_s = fmaxf(__fdiv_rn(hi - lo, levels), 1e-8f), best_b = lo;
  float best = group_error<PER>(w, best_s, best_b, levels);
  const float shr[5] = {1.0f, 0.925f, 0.85f, 0.775f, 0.7f};
#pragma unroll 1
  for (int a = 0; a < 5; ++a)
#pragma unroll 1
    for (int b = 0; b < 5; ++b) {
      if (a == 0 && b == 0) continue;
      const float new_lo = mid + (lo - mid) * shr[a], new_hi = mid + (hi - mid) * shr[b];
      const float s = fmaxf(__fdiv_rn(new_hi - new_lo, levels), 1e-8f);
      const float e = group_error<PER>(w, s, new_lo, levels);
      if (e < best) best = e, best_s = s, best_b = new_lo;
    }
  if (iters > 0) {
    float s = store_round<SDT>(best_s), bi = store_round<SDT>(best_b);
    best_s = s, best_b = bi;
    best = group_error<PER>(w, s, bi, levels);
    const float n = (float)GROUP;
#pragma unroll 1
    for (int it = 0; it < iters; ++it) {
      float sq = 0.f, sqq = 0.f, sqw = 0.f;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        const float q = fminf(fmaxf(rintf(__fdiv_rn(w[i] - bi, s)), 0.f), levels);
        sq += q, sqq += q * q, sqw += q * w[i];
      }
      sq = warp_sum(sq), sqq = warp_sum(sqq), sqw = warp_sum(sqw);
      const float den = n * sqq - sq * sq;
      const bool flat = fabsf(den) < 1e-12f;
      float ns = __fdiv_rn(n * sqw - sq * sw, flat ? 1.f : den);
      float nb = __fdiv_rn(sw - ns * sq, n);
      ns = store_round<SDT>(ns), nb = store_round<SDT>(nb);
      if (!(flat || ns <= 0.f)) s = ns, bi = nb;
      const float e = group_error<PER>(w, s, bi, levels);
      if (e < best) best = e, best_s = s, best_b = bi;
    }
  }
  const float s = store_round<SDT>(best_s), bi = store_round<SDT>(best_b);
  // levels of this lane's PER elements as one field of PER * bits bits; a word holds 32 / bits levels
  uint32_t field = 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const uint32_t q = (uint32_t)fminf(fmaxf(rintf(__fdiv_rn(w[i] - bi, s)), 0.f), levels);
    field |= q << (i * bits);
  }
  const int fbits = PER * bits;            // 4, 8 or 16 bits per lane
  const int lanes_per_word = 32 / fbits;   // 8, 4 or 2
  uint32_t word = 0;
  for (int j = 0; j < lanes_per_word; ++j)
    word |= __shfl_sync(0xffffffffu, field, (lane / lanes_per_word) * lanes_per_word + j) << (j * fbits);
  if (lane % lanes_per_word == 0) out_words[grp * (GROUP * bits / 32) + lane / lanes_per_word] = word;
  if (lane == 0) {
    if constexpr (SDT == CACHALOT_F16) {
      reinterpret_cast<__half*>(out_scales)[grp] = __float2half_rn(s);
      reinterpret_cast<__half*>(out_biases)[grp] = __float2half_rn(bi);
    } else {
      reinterpret_cast<__nv_bfloat16*>(out_scales)[grp] = __float2bfloat16_rn(s);
      reinterpret_cast<__nv_bfloat16*>(out_biases)[grp] = __float2bfloat16_rn(bi);
    }
  }
}

}  // namespace
}  // namespace cachalot

using namespace cachalot;

extern "C" int cachalot_requant_fp4_to_affine(const uint8_t* packed, const uint8_t* scales, int n, int k, int bits, int group,
                                              int scale_dtype, int lsq_iters, uint32_t* out_words, void* out_scales,
                                              void* out_biases, cachalot_stream_t stream) {
  if (!packed || !scales || !out_words || !out_scales || !out_biases) return fail(CACHALOT_EINVAL, "requant: null pointer");
  if (n <= 0 || k <= 0 || k % 32) return fail(CACHALOT_EINVAL, "requant: K=%d must be a positive multiple of 32", k);
  if (bits != 2 && bits != 4) return fail(CACHALOT_EUNSUPPORTED, "requant: bits=%d (2 or 4)", bits);
  if (group != 64 && group != 128) return fail(CACHALOT_EUNSUPPORTED, "requant: group %d (64 or 128)", group);
  // the reference reshapes the fitted scales to [rows, K / group] (benchmarks/quant_affine.py:326-329): a row is a whole number of groups
  if (k % group) return fail(CACHALOT_EINVAL, "requant: K=%d is not a whole number of groups of %d", k, group);
  if (scale_dtype != CACHALOT_F16 && scale_dtype != CACHALOT_BF16) return fail(CACHALOT_EINVAL, "requant: scale dtype must be f16 or bf16");
  if (lsq_iters < 0 || lsq_iters > 64) return fail(CACHALOT_EINVAL, "requant: lsq_iters %d", lsq_iters);
  const long long groups = (long long)n * k / group;
  const unsigned blocks = (unsigned)((groups * 32 + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
#define CACHALOT_RQ(PERV, SDTV) \
  requant_kernel<PERV, SDTV><<<blocks, 256, 0, s>>>(packed, scales, groups, k, bits, lsq_iters, out_words, out_scales, out_biases)
  if (group == 128) {
    if (scale_dtype == CACHALOT_F16) CACHALOT_RQ(4, CACHALOT_F16); else CACHALOT_RQ(4, CACHALOT_BF16);
  } else {
    if (scale_dtype == CACHALOT_F16) CACHALOT_RQ(2, CACHALOT_F16); else CACHALOT_RQ(2, CACHALOT_BF16);
  }
#undef CACHALOT_RQ
  return check_launch("requant");
}
