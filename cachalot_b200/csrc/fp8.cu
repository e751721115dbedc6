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

// SwiGLU of the shared expert fused with the act_quant of its result (model/shared_expert_metal.py:165-180):
// gate, up bf16 -> f32; up = clip(up, +-L), gate = min(gate, L) when L > 0; h = silu(gate) * up -> bf16 (the
// activation dtype) -> act_quant per block.  One warp per (row, block), as act_quant_kernel.
template <int PER>
__global__ void swiglu_act_quant_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up, long long ld,
                                        int rows, int k, int scale_rule, float limit, uint8_t* __restrict__ codes,
                                        float* __restrict__ scales) {
  constexpr int BLOCK = 32 * PER;
  const int nblk = k / BLOCK;
  long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)rows * nblk) return;
  const long long row = warp / nblk;
  const int col = (int)(warp - row * nblk) * BLOCK + lane * PER;
  float v[PER];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    float g = __bfloat162float(gate[row * ld + col + i]), u = __bfloat162float(up[row * ld + col + i]);
    v[i] = bf16_round(swiglu(g, u, limit));
    amax = fmaxf(amax, fabsf(v[i]));
  }
  amax = fmaxf(warp_max(amax), 1e-4f);
  float raw = __fdiv_rn(amax, 448.0f);
  float scale = raw;
  if (scale_rule == CACHALOT_SCALE_E8M0) scale = __uint_as_float((uint32_t)(ceil_log2(raw) + 127) << 23);
  const size_t base = (size_t)row * k + col;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    float q = fminf(fmaxf(__fdiv_rn(v[i], scale), -448.0f), 448.0f);
    codes[base + i] = (uint8_t)__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3);
  }
  if (lane == 0) scales[warp] = scale;
}

// ---- GEMV on the tensor cores -------------------------------------------------------------------
// Both operands are E4M3 codes, so the products can be formed by mma.sync.m16n8k32.e4m3 (exact in
// fp32) without decoding anything: weight bytes go from global memory straight into the A operand.
//   CTA  = 16 output rows (the MMA's M), KS warps (4, 8 or 16: enough to put ~12 warps on every SM) that each
//          take a slice of K, partial sums added through shared memory at the end
//   lane = (g, t): loads 8 bytes of rows g and g+8 per step; the quad covers 32 consecutive K = one
//          MMA, and never straddles a scale block (32 or 128)
//   N    = eight tokens per MMA (token g of the group in operand column g); more tokens loop over
//          groups of eight with the weight registers reused
// Per scale block the fp32 partial sum of the block is multiplied by act_scale * weight_scale and
// added to the row's accumulator: the reference's scale placement (model/fp8_ref.py:208-229).
constexpr int GEMV_MAX_TG = 8;   // token groups of eight handled by one launch (64 tokens)

__device__ __forceinline__ uint32_t e4m3x4_nan_to_zero(uint32_t w) {  // the codes 0x7F / 0xFF read as zero
  return w & ~__vcmpeq4(w & 0x7F7F7F7Fu, 0x7F7F7F7Fu);
}
__device__ __forceinline__ void qmma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// RT: 16-row tiles per warp.  With several token groups the activation fragments are the larger part of the loads;
// two row tiles share them.
template <int NTG, int BLOCK, int KS, int RT, typename OutT>
__global__ void __launch_bounds__(KS * 32)
fp8_gemv_mma_kernel(const uint8_t* __restrict__ codes, const float* __restrict__ act_scales,
                    const uint8_t* __restrict__ weight, const void* __restrict__ w_scales, int scale_rule, int rows,
                    int n_out, int k, OutT* __restrict__ out, long long ldo, const float* __restrict__ addend) {
  constexpr int MPB = BLOCK / 32;  // MMAs per scale block
  constexpr int UNR = BLOCK == 32 ? 8 / RT : 2;  // scale blocks in flight: about sixteen 8-byte weight loads per lane
  __shared__ float red[KS][RT][NTG][4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n0 = blockIdx.x * 16 * RT;
  const int nkb = k / BLOCK;
  // this warp's scale blocks
  const int kb_lo = nkb * warp / KS, kb_hi = nkb * (warp + 1) / KS;
  // rows past the end read the last row; their results are not stored
  const uint8_t* wa[RT];
  const uint8_t* wb[RT];
#pragma unroll
  for (int rt = 0; rt < RT; ++rt) {
    wa[rt] = weight + (size_t)min(n0 + rt * 16 + g, n_out - 1) * k + t * 8;
    wb[rt] = weight + (size_t)min(n0 + rt * 16 + g + 8, n_out - 1) * k + t * 8;
  }
  // weight scales: the CTA's 16*RT rows share a scale row (the block is 32 or 128 rows, n0 a multiple of 16*RT <= 32)
  const size_t srow = (size_t)(n0 / BLOCK) * nkb;
  // tokens of this lane: operand column g of group tg is token tg*8 + g; accumulator columns 2t, 2t+1
  const uint8_t* cb[NTG];
  bool tok_ok[NTG];
#pragma unroll
  for (int tg = 0; tg < NTG; ++tg) {
    const int tok = tg * 8 + g;
    tok_ok[tg] = tok < rows;
    cb[tg] = codes + (size_t)(tok_ok[tg] ? tok : 0) * k + t * 8;
  }
  float acc[RT][NTG][4];
#pragma unroll
  for (int rt = 0; rt < RT; ++rt)
#pragma unroll
    for (int tg = 0; tg < NTG; ++tg) acc[rt][tg][0] = acc[rt][tg][1] = acc[rt][tg][2] = acc[rt][tg][3] = 0.f;

#pragma unroll UNR
  for (int kb = kb_lo; kb < kb_hi; ++kb) {
    float d[RT][NTG][4];
#pragma unroll
    for (int rt = 0; rt < RT; ++rt)
#pragma unroll
      for (int tg = 0; tg < NTG; ++tg) d[rt][tg][0] = d[rt][tg][1] = d[rt][tg][2] = d[rt][tg][3] = 0.f;
#pragma unroll
    for (int m = 0; m < MPB; ++m) {
      const int ko = kb * BLOCK + m * 32;
      uint32_t a[RT][4];
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        const uint2 va = ld_stream_u2(wa[rt] + ko), vb = ld_stream_u2(wb[rt] + ko);
        a[rt][0] = e4m3x4_nan_to_zero(va.x), a[rt][2] = e4m3x4_nan_to_zero(va.y);
        a[rt][1] = e4m3x4_nan_to_zero(vb.x), a[rt][3] = e4m3x4_nan_to_zero(vb.y);
      }
#pragma unroll
      for (int tg = 0; tg < NTG; ++tg) {
        uint2 b = make_uint2(0u, 0u);
        if (tok_ok[tg]) b = __ldg(reinterpret_cast<const uint2*>(cb[tg] + ko));
#pragma unroll
        for (int rt = 0; rt < RT; ++rt) qmma_e4m3(d[rt][tg], a[rt][0], a[rt][1], a[rt][2], a[rt][3], b.x, b.y);
      }
    }
    const float ws = scale_rule == CACHALOT_SCALE_E8M0 ? e8m0_to_f32(reinterpret_cast<const uint8_t*>(w_scales)[srow + kb])
                                                        : reinterpret_cast<const float*>(w_scales)[srow + kb];
#pragma unroll
    for (int tg = 0; tg < NTG; ++tg) {
      const int t0 = tg * 8 + 2 * t;
      const float s0 = (t0 < rows ? act_scales[(size_t)t0 * nkb + kb] : 0.f) * ws;
      const float s1 = (t0 + 1 < rows ? act_scales[(size_t)(t0 + 1) * nkb + kb] : 0.f) * ws;
#pragma unroll
      for (int rt = 0; rt < RT; ++rt) {
        acc[rt][tg][0] = fmaf(d[rt][tg][0], s0, acc[rt][tg][0]);
        acc[rt][tg][1] = fmaf(d[rt][tg][1], s1, acc[rt][tg][1]);
        acc[rt][tg][2] = fmaf(d[rt][tg][2], s0, acc[rt][tg][2]);
        acc[rt][tg][3] = fmaf(d[rt][tg][3], s1, acc[rt][tg][3]);
      }
    }
  }
  // add the K slices (fixed order) and store
#pragma unroll
  for (int rt = 0; rt < RT; ++rt)
#pragma unroll
    for (int tg = 0; tg < NTG; ++tg)
#pragma unroll
      for (int i = 0; i < 4; ++i) red[warp][rt][tg][i][lane] = acc[rt][tg][i];
  __syncthreads();
  // warp w adds and stores the (row tile, token group) pairs w, w + KS, ...
  for (int pair = warp; pair < RT * NTG; pair += KS) {
    const int rt = pair / NTG, tg = pair - rt * NTG;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v = red[0][rt][tg][i][lane];
#pragma unroll
      for (int w = 1; w < KS; ++w) v += red[w][rt][tg][i][lane];
      const int tok = tg * 8 + 2 * t + (i & 1), row = n0 + rt * 16 + g + (i >> 1) * 8;
      if (tok < rows && row < n_out) {
        // with an addend the linear's own result is rounded to bf16 first (it is a bf16 tensor in the reference),
        // then added in fp32: (routed + shared.astype(f32)).astype(bf16) of model/moe_layer_metal.py:394-403
        if (addend) v = bf16_round(v) + addend[(size_t)tok * n_out + row];
        if constexpr (sizeof(OutT) == 2)
          out[(size_t)tok * ldo + row] = __float2bfloat16_rn(v);
        else
          out[(size_t)tok * ldo + row] = v;
      }
    }
  }
}

template <int BLOCK, typename OutT>
static void launch_gemv_mma(int ntg, cudaStream_t s, const uint8_t* codes, const float* act_scales, const uint8_t* weight,
                            const void* w_scales, int scale_rule, int rows, int n, int k, OutT* out, long long ldo,
                            const float* addend) {
  // warps per CTA: about twelve warps per SM in total (the reduction buffer limits it for many tokens)
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int rt = ntg >= 3 && ntg <= 4 ? 2 : 1;   // 32-row CTAs once the activation fragments outweigh the weight loads (registers allow it up to 32 tokens)
  const long long tiles = (n + 16 * rt - 1) / (16 * rt);
  const dim3 grid((unsigned)tiles);
  int ks = 4;
  if (tiles * 4 < 12LL * sms && ntg <= 4) ks = 8;
  if (tiles * 8 < 12LL * sms && ntg <= 2) ks = 16;
#define CACHALOT_GEMV(NTGV, KSV, RTV) \
  fp8_gemv_mma_kernel<NTGV, BLOCK, KSV, RTV, OutT><<<grid, KSV * 32, 0, s>>>(codes, act_scales, weight, w_scales, scale_rule, rows, n, k, out, ldo, addend)
  if (ntg == 1) {
    if (ks == 16) CACHALOT_GEMV(1, 16, 1); else if (ks == 8) CACHALOT_GEMV(1, 8, 1); else CACHALOT_GEMV(1, 4, 1);
  } else if (ntg == 2) {
    if (ks == 16) CACHALOT_GEMV(2, 16, 1); else if (ks == 8) CACHALOT_GEMV(2, 8, 1); else CACHALOT_GEMV(2, 4, 1);
  } else if (ntg <= 4) {
    if (ks == 8) CACHALOT_GEMV(4, 8, 2); else CACHALOT_GEMV(4, 4, 2);
  } else {
    CACHALOT_GEMV(8, 4, 1);
  }
#undef CACHALOT_GEMV
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

static int gemv_checked(const char* who, const uint8_t* codes, const float* act_scales, const uint8_t* weight, const void* w_scales,
                        int scale_rule, int block, int rows, int n, int k, void* out, int out_dtype, long long ldo,
                        const float* addend, cudaStream_t s) {
  if (!codes || !act_scales || !weight || !w_scales || !out) return fail(CACHALOT_EINVAL, "%s: null pointer", who);
  if (block != 32 && block != 128) return fail(CACHALOT_EUNSUPPORTED, "%s: block=%d (32 or 128)", who, block);
  if (rows < 0 || n <= 0 || k <= 0 || k % block) return fail(CACHALOT_EINVAL, "K=%d is not divisible by %d", k, block);
  if (scale_rule != CACHALOT_SCALE_E8M0 && scale_rule != CACHALOT_SCALE_F32) return fail(CACHALOT_EINVAL, "%s: unknown scale rule", who);
  if (out_dtype != CACHALOT_BF16 && out_dtype != CACHALOT_F32) return fail(CACHALOT_EINVAL, "%s: out dtype must be bf16 or f32", who);
  if (!aligned(weight, 8) || !aligned(codes, 8) || k % 8) return fail(CACHALOT_EALIGN, "%s: weight and codes need 8-byte alignment", who);
  if (ldo < n) return fail(CACHALOT_EINVAL, "%s: output row pitch %lld < %d", who, ldo, n);
  if (rows == 0) return CACHALOT_OK;
  // 64 tokens per launch; more tokens take more launches over the same weights
  for (int r0 = 0; r0 < rows; r0 += 8 * GEMV_MAX_TG) {
    const int nr = rows - r0 < 8 * GEMV_MAX_TG ? rows - r0 : 8 * GEMV_MAX_TG;
    const int ntg = (nr + 7) / 8;
    const uint8_t* c = codes + (size_t)r0 * k;
    const float* as = act_scales + (size_t)r0 * (k / block);
    const float* ad = addend ? addend + (size_t)r0 * n : nullptr;
    if (out_dtype == CACHALOT_BF16) {
      __nv_bfloat16* o = (__nv_bfloat16*)out + (size_t)r0 * ldo;
      if (block == 32) launch_gemv_mma<32>(ntg, s, c, as, weight, w_scales, scale_rule, nr, n, k, o, ldo, ad);
      else launch_gemv_mma<128>(ntg, s, c, as, weight, w_scales, scale_rule, nr, n, k, o, ldo, ad);
    } else {
      float* o = (float*)out + (size_t)r0 * ldo;
      if (block == 32) launch_gemv_mma<32>(ntg, s, c, as, weight, w_scales, scale_rule, nr, n, k, o, ldo, ad);
      else launch_gemv_mma<128>(ntg, s, c, as, weight, w_scales, scale_rule, nr, n, k, o, ldo, ad);
    }
  }
  return check_launch(who);
}

extern "C" int cachalot_fp8_gemv(const uint8_t* codes, const float* act_scales, const uint8_t* weight,
                                 const void* w_scales, int scale_rule, int block, int rows, int n, int k, void* out,
                                 int out_dtype, cachalot_stream_t stream) {
  return gemv_checked("fp8_gemv", codes, act_scales, weight, w_scales, scale_rule, block, rows, n, k, out, out_dtype, n, nullptr,
                      (cudaStream_t)stream);
}

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }

extern "C" size_t cachalot_shared_expert_workspace_bytes(int rows, int hidden, int inter, int block) {
  if (rows <= 0 || hidden <= 0 || inter <= 0 || block <= 0) return 0;
  const size_t kmax = (size_t)(hidden > inter ? hidden : inter);
  // codes and scales of the larger of the two activations (x, then h in the same place), gate|up as bf16
  return align256((size_t)rows * kmax) + align256((size_t)rows * (kmax / block + 1) * 4) + align256((size_t)rows * 2 * inter * 2);
}

extern "C" int cachalot_shared_expert(const void* x_bf16, int rows, int hidden, int inter, const uint8_t* w1,
                                      const void* w1_scales, const uint8_t* w3, const void* w3_scales, const uint8_t* w2,
                                      const void* w2_scales, int scale_rule, int block, float swiglu_limit,
                                      const float* addend, void* workspace, size_t workspace_bytes, void* out_bf16,
                                      cachalot_stream_t stream) {
  if (!x_bf16 || !w1 || !w1_scales || !w2 || !w2_scales || !out_bf16) return fail(CACHALOT_EINVAL, "shared_expert: null pointer");
  if (w3 && !w3_scales) return fail(CACHALOT_EINVAL, "shared_expert: w3 without scales");
  if (rows < 0 || hidden <= 0 || inter <= 0) return fail(CACHALOT_EINVAL, "shared_expert: bad shape");
  if (block != 32 && block != 128) return fail(CACHALOT_EUNSUPPORTED, "shared_expert: block=%d (32 or 128)", block);
  if (hidden % block || inter % block) return fail(CACHALOT_EINVAL, "shared_expert: hidden %d and inter %d must be multiples of the block %d", hidden, inter, block);
  if (rows == 0) return CACHALOT_OK;
  const size_t need = cachalot_shared_expert_workspace_bytes(rows, hidden, inter, block);
  if (!workspace || workspace_bytes < need) return fail(CACHALOT_ESCRATCH, "shared_expert: workspace %zu < %zu bytes", workspace_bytes, need);
  if (!aligned(workspace, 256)) return fail(CACHALOT_EALIGN, "shared_expert: workspace must be 256-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const size_t kmax = (size_t)(hidden > inter ? hidden : inter);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  uint8_t* codes = ws;
  float* scales = reinterpret_cast<float*>(ws + align256((size_t)rows * kmax));
  __nv_bfloat16* gu = reinterpret_cast<__nv_bfloat16*>(ws + align256((size_t)rows * kmax) + align256((size_t)rows * (kmax / block + 1) * 4));
  // one act_quant for both projections (model/shared_expert_metal.py:94-107, 160-163)
  int rc = cachalot_fp8_act_quant(x_bf16, rows, hidden, block, scale_rule, codes, scales, stream);
  if (rc) return rc;
  const long long ld = 2LL * inter;
  if (w3) {
    rc = gemv_checked("shared_expert w1", codes, scales, w1, w1_scales, scale_rule, block, rows, inter, hidden, gu, CACHALOT_BF16, ld, nullptr, s);
    if (rc) return rc;
    rc = gemv_checked("shared_expert w3", codes, scales, w3, w3_scales, scale_rule, block, rows, inter, hidden, gu + inter, CACHALOT_BF16, ld, nullptr, s);
  } else {  // w1 holds [2*inter, hidden] = w1 rows, then w3 rows
    rc = gemv_checked("shared_expert w13", codes, scales, w1, w1_scales, scale_rule, block, rows, 2 * inter, hidden, gu, CACHALOT_BF16, ld, nullptr, s);
  }
  if (rc) return rc;
  {
    const long long warps = (long long)rows * (inter / block);
    const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
    if (block == 32) swiglu_act_quant_kernel<1><<<blocks, 256, 0, s>>>(gu, gu + inter, ld, rows, inter, scale_rule, swiglu_limit, codes, scales);
    else swiglu_act_quant_kernel<4><<<blocks, 256, 0, s>>>(gu, gu + inter, ld, rows, inter, scale_rule, swiglu_limit, codes, scales);
    if ((rc = check_launch("shared_expert swiglu"))) return rc;
  }
  return gemv_checked("shared_expert w2", codes, scales, w2, w2_scales, scale_rule, block, rows, hidden, inter, out_bf16, CACHALOT_BF16, hidden, addend, s);
}
