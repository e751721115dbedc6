// Elementwise dequantisation kernels.  They exist to prove bit-exactness of the decode tables
// against the reference's numpy path; the GEMV kernels never materialise dense weights.
#include "common.cuh"

namespace cachalot {

// one thread per packed 32-bit word (8 codes); 4 words share a scale byte
__global__ void fp4_dequant_kernel(const uint32_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                                   long long n_words, int words_per_row, float* __restrict__ out) {
  long long w = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (w >= n_words) return;
  long long row = w / words_per_row;
  int col = (int)(w - row * words_per_row);
  float s = e8m0_to_f32(scales[row * (words_per_row / 4) + col / 4]);
  uint32_t v = packed[w];
  float4 lo, hi;
  lo.x = e2m1_to_f32(v) * s;
  lo.y = e2m1_to_f32(v >> 4) * s;
  lo.z = e2m1_to_f32(v >> 8) * s;
  lo.w = e2m1_to_f32(v >> 12) * s;
  hi.x = e2m1_to_f32(v >> 16) * s;
  hi.y = e2m1_to_f32(v >> 20) * s;
  hi.z = e2m1_to_f32(v >> 24) * s;
  hi.w = e2m1_to_f32(v >> 28) * s;
  float4* o = reinterpret_cast<float4*>(out + w * 8);
  o[0] = lo;
  o[1] = hi;
}

template <typename S>
__device__ __forceinline__ float load_scale(const void* p, long long i);
template <>
__device__ __forceinline__ float load_scale<__half>(const void* p, long long i) {
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
template <>
__device__ __forceinline__ float load_scale<__nv_bfloat16>(const void* p, long long i) {
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// one thread per output element; bits in {2,4,8} so a level never straddles a word
template <typename S>
__global__ void affine_dequant_kernel(const uint32_t* __restrict__ words, const void* __restrict__ scales,
                                      const void* __restrict__ biases, long long total, int k, int bits, int group,
                                      float* __restrict__ out) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= total) return;
  long long row = i / k;
  int col = (int)(i - row * k);
  int per_word = 32 / bits;
  uint32_t word = words[row * (k / per_word) + col / per_word];
  uint32_t q = (word >> ((col % per_word) * bits)) & ((1u << bits) - 1u);
  long long g = row * (k / group) + col / group;
  // product is exact in fp32 (<= 8 + 11 significant bits); one rounding in the add
  out[i] = __fadd_rn(__fmul_rn(load_scale<S>(scales, g), (float)q), load_scale<S>(biases, g));
}

}  // namespace cachalot

using namespace cachalot;

extern "C" int cachalot_fp4_dequant(const uint8_t* packed, const uint8_t* scales, int n, int k, float* out,
                                    cachalot_stream_t stream) {
  if (!packed || !scales || !out) return fail(CACHALOT_EINVAL, "fp4_dequant: null pointer");
  if (n < 0 || k <= 0 || k % 32) return fail(CACHALOT_EINVAL, "fp4_dequant: K=%d must be a positive multiple of 32", k);
  if (!aligned(packed, 4) || !aligned(out, 16)) return fail(CACHALOT_EALIGN, "fp4_dequant: packed needs 4-byte, out 16-byte alignment");
  if (n == 0) return CACHALOT_OK;
  long long n_words = (long long)n * (k / 8);
  int threads = 256;
  long long blocks = (n_words + threads - 1) / threads;
  fp4_dequant_kernel<<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const uint32_t*>(packed), scales, n_words, k / 8, out);
  return check_launch("fp4_dequant");
}

extern "C" int cachalot_affine_dequant(const uint32_t* words, const void* scales, const void* biases, int n, int k,
                                       int bits, int group, int scale_dtype, float* out,
                                       cachalot_stream_t stream) {
  if (!words || !scales || !biases || !out) return fail(CACHALOT_EINVAL, "affine_dequant: null pointer");
  if (bits != 2 && bits != 4 && bits != 8) return fail(CACHALOT_EUNSUPPORTED, "affine_dequant: bits=%d not in {2,4,8}", bits);
  if (group <= 0 || k <= 0 || k % group || (group * bits) % 32)
    return fail(CACHALOT_EINVAL, "affine_dequant: K=%d group=%d bits=%d is not a whole number of groups/words", k, group, bits);
  if (n == 0) return CACHALOT_OK;
  long long total = (long long)n * k;
  int threads = 256;
  long long blocks = (total + threads - 1) / threads;
  if (scale_dtype == CACHALOT_F16)
    affine_dequant_kernel<__half><<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(words, scales, biases, total, k, bits, group, out);
  else if (scale_dtype == CACHALOT_BF16)
    affine_dequant_kernel<__nv_bfloat16><<<(unsigned)blocks, threads, 0, (cudaStream_t)stream>>>(words, scales, biases, total, k, bits, group, out);
  else
    return fail(CACHALOT_EINVAL, "affine_dequant: scale_dtype must be f16 or bf16");
  return check_launch("affine_dequant");
}
