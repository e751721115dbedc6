// Prefill helpers: expert-major row grouping (a stable counting sort of the routed expert ids)
// and MXFP4 activation quantisation.
#include "kernels.cuh"

namespace cachalot {

constexpr int GROUP_CHUNK = 1024;  // ids per CTA of the counting sort

// CTA b counts the experts of ids [b*1024, (b+1)*1024): block_counts[b][e]
__global__ void __launch_bounds__(GROUP_CHUNK)
group_count_kernel(const int32_t* __restrict__ ids, int total, int n_experts, int32_t* __restrict__ block_counts,
                   int* __restrict__ status) {
  extern __shared__ int32_t hist[];
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int i = blockIdx.x * GROUP_CHUNK + threadIdx.x;
  if (i < total) {
    const int e = ids[i];
    if (e < 0 || e >= n_experts) {
      if (status) atomicOr(status, CACHALOT_STATUS_ID_RANGE);
    } else {
      atomicAdd(&hist[e], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) block_counts[(size_t)blockIdx.x * n_experts + e] = hist[e];
}

// single CTA: offsets[e] = rows of experts < e; block_counts[b][e] becomes the first position of CTA b's rows of
// expert e (experts ascending, CTAs ascending inside an expert: the order a stable sort gives)
__global__ void group_scan_kernel(int32_t* __restrict__ block_counts, int n_blocks, int n_experts, int32_t* __restrict__ offsets) {
  extern __shared__ int32_t sh[];  // [n_experts] totals, then [blockDim.x] partial sums
  int32_t* tot = sh;
  int32_t* part = sh + n_experts;
  const int t = threadIdx.x, n = blockDim.x;
  for (int e = t; e < n_experts; e += n) {
    int run = 0;
    for (int b = 0; b < n_blocks; ++b) {
      const int v = block_counts[(size_t)b * n_experts + e];
      block_counts[(size_t)b * n_experts + e] = run;
      run += v;
    }
    tot[e] = run;
  }
  __syncthreads();
  const int per = (n_experts + n - 1) / n;
  const int lo = min(t * per, n_experts), hi = min(lo + per, n_experts);
  int sum = 0;
  for (int e = lo; e < hi; ++e) sum += tot[e];
  part[t] = sum;
  __syncthreads();
  if (t == 0) {
    int run = 0;
    for (int i = 0; i < n; ++i) {
      const int v = part[i];
      part[i] = run;
      run += v;
    }
    offsets[n_experts] = run;
  }
  __syncthreads();
  int run = part[t];
  for (int e = lo; e < hi; ++e) {
    offsets[e] = run;
    const int base = run;
    run += tot[e];
    tot[e] = base;
  }
  __syncthreads();
  for (int e = t; e < n_experts; e += n)
    for (int b = 0; b < n_blocks; ++b) block_counts[(size_t)b * n_experts + e] += tot[e];
}

// CTA b places its ids in order: warps one after the other, lanes ranked inside a warp by match + popcount
__global__ void __launch_bounds__(GROUP_CHUNK)
group_place_kernel(const int32_t* __restrict__ ids, int total, int n_experts, const int32_t* __restrict__ block_base,
                   int32_t* __restrict__ perm) {
  extern __shared__ int32_t next[];  // next free position of every expert for this CTA
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) next[e] = block_base[(size_t)blockIdx.x * n_experts + e];
  __syncthreads();
  const int i = blockIdx.x * GROUP_CHUNK + threadIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int e = i < total ? ids[i] : -1;
  if (e >= n_experts) e = -1;
  for (int w = 0; w < GROUP_CHUNK / 32; ++w) {
    if (warp == w) {
      const unsigned same = __match_any_sync(0xffffffffu, e);
      if (e >= 0) {
        const int rank = __popc(same & ((1u << lane) - 1u));
        perm[next[e] + rank] = i;
      }
      __syncwarp();
      if (e >= 0 && (same & ((1u << lane) - 1u)) == 0) next[e] += __popc(same);  // the group's first lane moves the cursor on
    }
    __syncthreads();
  }
}

// one thread per 8 consecutive elements (one 16-byte load), four threads per 32-block
__global__ void mxfp4_quant_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ src_rows,
                                   long long rows, int k, uint8_t* __restrict__ codes, uint8_t* __restrict__ scales) {
  const int per_row = k / 8;
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const bool live = i < rows * per_row;
  const long long r = live ? i / per_row : 0;
  const int c = live ? (int)(i - r * per_row) : 0;
  const long long src = src_rows ? src_rows[r] : r;
  uint4 raw = make_uint4(0, 0, 0, 0);
  if (live) raw = *reinterpret_cast<const uint4*>(x + src * k + c * 8);
  const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
  float v[8];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[2 * j] = __uint_as_float(wds[j] << 16);
    v[2 * j + 1] = __uint_as_float(wds[j] & 0xffff0000u);
    amax = fmaxf(amax, fmaxf(fabsf(v[2 * j]), fabsf(v[2 * j + 1])));
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const int e = mxfp4_exponent(amax);
  const float inv = pow2f(-e);  // times 2**-e is the same rounding as over 2**e
  uint32_t packed = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) packed |= e2m1x2_byte(v[2 * j] * inv, v[2 * j + 1] * inv) << (8 * j);
  if (!live) return;
  *reinterpret_cast<uint32_t*>(codes + r * (k / 2) + c * 4) = packed;
  if ((c & 3) == 0) scales[r * (k / 32) + (c >> 2)] = (uint8_t)(e + 127);
}

template <typename T>
__global__ void mxfp4_roundtrip_kernel(const T* __restrict__ in, T* __restrict__ out, long long n_blocks) {
  long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= n_blocks) return;
  float v;
  if constexpr (sizeof(T) == 2) v = __bfloat162float(in[warp * 32 + lane]); else v = in[warp * 32 + lane];
  int e = mxfp4_exponent(warp_max(fabsf(v)));
  float s = pow2f(e);
  float q = fminf(fmaxf(__fdiv_rn(v, s), -6.0f), 6.0f);
  uint32_t code = e2m1_round_code(q);
  float y = e2m1_to_f32(code) * s;
  if (code == 8u || ((code & 7u) == 0u && (code & 8u))) y = -0.0f * s;  // signed zero kept
  if constexpr (sizeof(T) == 2) out[warp * 32 + lane] = __float2bfloat16_rn(y); else out[warp * 32 + lane] = y;
}

int launch_mxfp4_roundtrip_f32(float* data, long long rows, int k, cudaStream_t stream) {
  long long n_blocks = rows * (k / 32);
  if (n_blocks == 0) return CACHALOT_OK;
  unsigned blocks = (unsigned)((n_blocks * 32 + 255) / 256);
  mxfp4_roundtrip_kernel<float><<<blocks, 256, 0, stream>>>(data, data, n_blocks);
  return check_launch("mxfp4_roundtrip_f32");
}
int launch_mxfp4_roundtrip_bf16(const __nv_bfloat16* in, __nv_bfloat16* out, long long rows, int k, cudaStream_t stream) {
  long long n_blocks = rows * (k / 32);
  if (n_blocks == 0) return CACHALOT_OK;
  unsigned blocks = (unsigned)((n_blocks * 32 + 255) / 256);
  mxfp4_roundtrip_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(in, out, n_blocks);
  return check_launch("mxfp4_roundtrip_bf16");
}

}  // namespace cachalot

using namespace cachalot;

extern "C" size_t cachalot_group_rows_scratch_ints(int tokens, int k, int n_experts) {
  if (tokens < 0 || k <= 0 || n_experts <= 0) return 0;
  const long long total = (long long)tokens * k;
  return (size_t)((total + GROUP_CHUNK - 1) / GROUP_CHUNK + 1) * (size_t)n_experts;
}

extern "C" int cachalot_group_rows(const int32_t* expert_ids, int tokens, int k, int n_experts, int32_t* perm,
                                   int32_t* offsets, int32_t* counts_scratch, int* status,
                                   cachalot_stream_t stream) {
  if (!expert_ids || !perm || !offsets || !counts_scratch) return fail(CACHALOT_EINVAL, "group_rows: null pointer");
  if (tokens < 0 || k <= 0 || n_experts <= 0) return fail(CACHALOT_EINVAL, "group_rows: bad shape");
  long long total_ll = (long long)tokens * k;
  if (total_ll > 0x7fffffff) return fail(CACHALOT_EINVAL, "group_rows: tokens*k too large");
  int total = (int)total_ll;
  cudaStream_t s = (cudaStream_t)stream;
  if (n_experts > 8192) return fail(CACHALOT_EUNSUPPORTED, "group_rows: more than 8192 experts");
  const int n_blocks = (total + GROUP_CHUNK - 1) / GROUP_CHUNK;
  if (n_blocks > 0)
    group_count_kernel<<<n_blocks, GROUP_CHUNK, n_experts * sizeof(int32_t), s>>>(expert_ids, total, n_experts, counts_scratch, status);
  group_scan_kernel<<<1, 256, (n_experts + 256) * sizeof(int32_t), s>>>(counts_scratch, n_blocks, n_experts, offsets);
  if (n_blocks > 0)
    group_place_kernel<<<n_blocks, GROUP_CHUNK, n_experts * sizeof(int32_t), s>>>(expert_ids, total, n_experts, counts_scratch, perm);
  return check_launch("group_rows");
}

extern "C" int cachalot_mxfp4_act_quant(const void* x_bf16, const int32_t* src_rows, int rows, int k, uint8_t* codes,
                                        uint8_t* scales, cachalot_stream_t stream) {
  if (!x_bf16 || !codes || !scales) return fail(CACHALOT_EINVAL, "mxfp4_act_quant: null pointer");
  if (rows < 0 || k <= 0 || k % 32) return fail(CACHALOT_EINVAL, "last dimension %d must be divisible by block_size=32", k);
  if (rows == 0) return CACHALOT_OK;
  if (!aligned(x_bf16, 16) || !aligned(codes, 4)) return fail(CACHALOT_EALIGN, "mxfp4_act_quant: x must be 16-byte and codes 4-byte aligned");
  long long threads = (long long)rows * (k / 8);
  unsigned blocks = (unsigned)((threads + 255) / 256);
  mxfp4_quant_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x_bf16, src_rows, rows, k, codes, scales);
  return check_launch("mxfp4_act_quant");
}
