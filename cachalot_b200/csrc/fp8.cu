// FP8 E4M3 trunk GEMV with dynamic activation quantisation (act_quant).
#include <cuda_fp8.h>

#include <cstdlib>
#include <mutex>
#include <set>
#include <utility>

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
  // a GEMV launched behind this kernel may start to stream its weights now (it waits for these codes itself)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
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
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
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

// ---- streaming GEMV: weight rows through a shared-memory ring --------------------------------------
// The same arithmetic with the weights brought in by bulk copies instead of per-lane loads: persistent CTAs (one
// per SM), a tile = 16 output rows over the whole K, cut along K into chunks of KC bytes per row.  Four copy warps
// (one lane each: the copies of one warp are issued one after the other, and a lane gets through a copy in about
// 60 ns + bytes / 46 B/ns, so the issuers have to be in different warps and the copies large) bring four rows each:
// one copy of 4 * K bytes when a stage holds whole rows, else one per row.  Eight MMA warps each take a slice of
// every stage's K (whole scale blocks) and add their partial sums through shared memory at the end of a tile.
// Rows 4c..4c+3 of a stage sit 64 bytes (mod 128) from the next four, and MMA row g is tile row
// (g >> 1) + 4 * (g & 1).  Up to eight tokens have their codes and scales staged in shared memory; more tokens
// read their codes through L1.  Under programmatic dependent launch the ring starts to fill while the activation
// quantiser that precedes this kernel is still running: only the staging waits for it.
constexpr int GS_PROD = 4;   // copy warps
constexpr int GS_WARPS = 8;  // MMA warps
constexpr int GS_THREADS = (GS_WARPS + GS_PROD) * 32;
constexpr int GS_MAX_STAGES = 8;
constexpr uint32_t GS_WAIT_LIMIT = 1u << 22;

struct GsGeo {
  int kc;         // bytes of K per stage and row
  int nkc;        // stages per tile
  int group_pitch;  // bytes between the four-row groups of a stage: 4 * kc + 64
  int stage_bytes, n_stage;
  int tok_pitch;  // bytes between staged tokens
  int off_ring, off_codes, off_as, off_red, off_bar, total;
};

__device__ __forceinline__ uint32_t gs_smem(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool gs_wait(uint64_t* b, uint32_t parity) {
  for (uint32_t i = 0; i < GS_WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok)
                 : "r"(gs_smem(b)), "r"(parity)
                 : "memory");
    if (ok) return true;
  }
  return false;
}
__host__ __device__ inline int gs_row_off(int r, int kc) { return (r >> 2) * (4 * kc + 64) + (r & 3) * kc; }

template <int NTG, int BLOCK, bool STAGED, typename OutT>
__global__ void __launch_bounds__(GS_THREADS, 1)
fp8_gemv_stream_kernel(GsGeo G, const uint8_t* __restrict__ codes, const float* __restrict__ act_scales,
                       const uint8_t* __restrict__ weight, const void* __restrict__ w_scales, int scale_rule, int rows,
                       int n_out, int k, OutT* __restrict__ out, long long ldo, const float* __restrict__ addend,
                       int* __restrict__ status) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* ring = smem + G.off_ring;
  uint8_t* s_codes = smem + G.off_codes;
  float* s_as = reinterpret_cast<float*>(smem + G.off_as);
  float* red = reinterpret_cast<float*>(smem + G.off_red);  // [GS_WARPS][NTG][4][32]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + G.off_bar);
  uint64_t* empty = full + GS_MAX_STAGES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int tiles = (n_out + 15) / 16;
  const int tile_lo = (int)((long long)tiles * blockIdx.x / gridDim.x), tile_hi = (int)((long long)tiles * (blockIdx.x + 1) / gridDim.x);
  const int nkb = k / BLOCK;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int s = 0; s < GS_MAX_STAGES; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gs_smem(&full[s])), "r"(GS_PROD));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(gs_smem(&empty[s])), "r"(GS_WARPS));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp < GS_PROD) {
    // ---- copies: warp p brings rows 4p..4p+3 of every stage (the weights do not depend on the previous kernel) ----
    if (lane == 0) {
      int s = 0;
      uint32_t round = 0;
      bool ok = true;
      for (int tile = tile_lo; tile < tile_hi && ok; ++tile) {
        const bool whole = G.nkc == 1 && tile * 16 + 16 <= n_out;  // four rows are one contiguous piece
        for (int c = 0; c < G.nkc; ++c) {
          if (round > 0 && !gs_wait(&empty[s], (round - 1u) & 1u)) {
            ok = false;
            break;
          }
          uint8_t* dst = ring + (size_t)s * G.stage_bytes + warp * G.group_pitch;
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(gs_smem(&full[s])), "r"(4u * (uint32_t)G.kc) : "memory");
          if (whole) {
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(gs_smem(dst)),
                         "l"(weight + (size_t)(tile * 16 + warp * 4) * k), "r"(4u * (uint32_t)G.kc), "r"(gs_smem(&full[s]))
                         : "memory");
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int row = min(tile * 16 + warp * 4 + j, n_out - 1);  // rows past the end repeat the last one; never stored
              asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                               gs_smem(dst + j * G.kc)),
                           "l"(weight + (size_t)row * k + (size_t)c * G.kc), "r"((uint32_t)G.kc), "r"(gs_smem(&full[s]))
                           : "memory");
            }
          }
          if (++s == G.n_stage) s = 0, ++round;
        }
      }
      if (!ok && status) atomicOr(status, CACHALOT_STATUS_WAIT_EXPIRED);
    }
    return;
  }
  // ---- MMA warps ----
  const int cw = warp - GS_PROD, tid = threadIdx.x - GS_PROD * 32;
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the codes and scales come from the kernel before this one
  if (STAGED) {
    const int per = k / 16;  // 16-byte pieces per token
    for (int i = tid; i < rows * per; i += GS_WARPS * 32) {
      const int tok = i / per, p = i - tok * per;
      *reinterpret_cast<uint4*>(s_codes + (size_t)tok * G.tok_pitch + p * 16) = __ldg(reinterpret_cast<const uint4*>(codes + (size_t)tok * k) + p);
    }
    for (int i = tid; i < 8 * nkb; i += GS_WARPS * 32) s_as[i] = i < rows * nkb ? act_scales[i] : 0.f;
    asm volatile("bar.sync 1, %0;" ::"r"(GS_WARPS * 32) : "memory");
  }
  constexpr int MPB = BLOCK / 32;  // MMAs per scale block
  const int n_u = G.kc / BLOCK;    // scale blocks per stage
  const int u_lo = n_u * cw / GS_WARPS, u_hi = n_u * (cw + 1) / GS_WARPS;
  const int wr = (g >> 1) + 4 * (g & 1);  // MMA row g is tile row wr; MMA row g + 8 is tile row wr + 8
  const int offA = gs_row_off(wr, G.kc) + t * 8, offB = gs_row_off(wr + 8, G.kc) + t * 8;
  int s = 0;
  uint32_t round = 0;
  bool ok = true;
  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    float acc[NTG][4];
#pragma unroll
    for (int tg = 0; tg < NTG; ++tg) acc[tg][0] = acc[tg][1] = acc[tg][2] = acc[tg][3] = 0.f;
    const int n0 = tile * 16;
    const size_t srow = (size_t)(n0 / BLOCK) * nkb;  // the tile's 16 rows share a row of weight scales
    for (int c = 0; c < G.nkc; ++c) {
      if (ok && !gs_wait(&full[s], round & 1u)) ok = false;
      const uint8_t* st = ring + (size_t)s * G.stage_bytes;
#pragma unroll 2
      for (int u = u_lo; u < u_hi; ++u) {
        const int kb = c * n_u + u;
        float d[NTG][4];
        // The two NaN codes of E4M3 (0x7F, 0xFF) read as zero.  Masking them out of every weight word would be most of
        // the loop's instructions, and real weights hold none: the block runs unmasked first, a NaN code shows as a
        // NaN in the block's sums (NaN times anything, zero included), and only then the block is redone masked.
        bool masked = false;
        for (;;) {
#pragma unroll
          for (int tg = 0; tg < NTG; ++tg) d[tg][0] = d[tg][1] = d[tg][2] = d[tg][3] = 0.f;
#pragma unroll
          for (int m = 0; m < MPB; ++m) {
            const int ko = u * BLOCK + m * 32;
            uint2 va = *reinterpret_cast<const uint2*>(st + offA + ko);
            uint2 vb = *reinterpret_cast<const uint2*>(st + offB + ko);
            if (masked) {
              va.x = e4m3x4_nan_to_zero(va.x), va.y = e4m3x4_nan_to_zero(va.y);
              vb.x = e4m3x4_nan_to_zero(vb.x), vb.y = e4m3x4_nan_to_zero(vb.y);
            }
#pragma unroll
            for (int tg = 0; tg < NTG; ++tg) {
              uint2 b = make_uint2(0u, 0u);
              const int tok = tg * 8 + g;
              if (tok < rows) {
                if (STAGED) b = *reinterpret_cast<const uint2*>(s_codes + (size_t)tok * G.tok_pitch + c * G.kc + ko + t * 8);
                else b = __ldg(reinterpret_cast<const uint2*>(codes + (size_t)tok * k + c * G.kc + ko + t * 8));
              }
              qmma_e4m3(d[tg], va.x, vb.x, va.y, vb.y, b.x, b.y);
            }
          }
          if (masked) break;
          float chk = 0.f;
#pragma unroll
          for (int tg = 0; tg < NTG; ++tg) chk += (d[tg][0] + d[tg][1]) + (d[tg][2] + d[tg][3]);
          if (!__any_sync(0xffffffffu, chk != chk)) break;
          masked = true;
        }
        const float ws = scale_rule == CACHALOT_SCALE_E8M0 ? e8m0_to_f32(__ldg(reinterpret_cast<const uint8_t*>(w_scales) + srow + kb))
                                                            : __ldg(reinterpret_cast<const float*>(w_scales) + srow + kb);
#pragma unroll
        for (int tg = 0; tg < NTG; ++tg) {
          const int t0 = tg * 8 + 2 * t;
          float s0, s1;
          if (STAGED) {
            s0 = s_as[t0 * nkb + kb] * ws, s1 = s_as[(t0 + 1) * nkb + kb] * ws;  // zero for tokens past the end
          } else {
            s0 = (t0 < rows ? __ldg(act_scales + (size_t)t0 * nkb + kb) : 0.f) * ws;
            s1 = (t0 + 1 < rows ? __ldg(act_scales + (size_t)(t0 + 1) * nkb + kb) : 0.f) * ws;
          }
          acc[tg][0] = fmaf(d[tg][0], s0, acc[tg][0]);
          acc[tg][1] = fmaf(d[tg][1], s1, acc[tg][1]);
          acc[tg][2] = fmaf(d[tg][2], s0, acc[tg][2]);
          acc[tg][3] = fmaf(d[tg][3], s1, acc[tg][3]);
        }
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(gs_smem(&empty[s])) : "memory");
      if (++s == G.n_stage) s = 0, ++round;
    }
    // add the eight K slices in a fixed order and store.  Two buffers by tile parity: one barrier per tile is enough,
    // because a warp cannot write the buffer of tile i + 2 before every warp has passed the barrier of tile i + 1,
    // that is, has read tile i.
    float* rbuf = red + ((tile - tile_lo) & 1) * (GS_WARPS * NTG * 4 * 32);
#pragma unroll
    for (int tg = 0; tg < NTG; ++tg)
#pragma unroll
      for (int i = 0; i < 4; ++i) rbuf[((cw * NTG + tg) * 4 + i) * 32 + lane] = acc[tg][i];
    asm volatile("bar.sync 1, %0;" ::"r"(GS_WARPS * 32) : "memory");
    // warp w adds and stores accumulator element w & 3 of token group w >> 2
    for (int job = cw; job < NTG * 4; job += GS_WARPS) {
      const int tg = job >> 2, i = job & 3;
      {
        float v = rbuf[((0 * NTG + tg) * 4 + i) * 32 + lane];
#pragma unroll
        for (int w = 1; w < GS_WARPS; ++w) v += rbuf[((w * NTG + tg) * 4 + i) * 32 + lane];
        const int tok = tg * 8 + 2 * t + (i & 1), row = n0 + wr + (i >> 1) * 8;
        if (tok < rows && row < n_out) {
          if (addend) v = bf16_round(v) + addend[(size_t)tok * n_out + row];
          if constexpr (sizeof(OutT) == 2)
            out[(size_t)tok * ldo + row] = __float2bfloat16_rn(v);
          else
            out[(size_t)tok * ldo + row] = v;
        }
      }
    }
  }
  if (!ok && lane == 0 && status) atomicOr(status, CACHALOT_STATUS_WAIT_EXPIRED);
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

constexpr int GS_SMEM_LIMIT = 227 * 1024 - 256;

// false when the shape is outside what the streaming kernel takes (the per-lane kernel runs then)
static bool gs_geometry(int rows, int k, int block, int ntg, bool* staged, GsGeo* out) {
  if (k % block || k % 16) return false;
  int nkc = 0;
  for (int n = (k + 4095) / 4096; n <= k / 1024 + 1 && n <= 64; ++n)
    if (k % n == 0 && (k / n) % block == 0 && (k / n) % 16 == 0) {
      nkc = n;
      break;
    }
  if (!nkc || k / nkc < 1024) return false;  // short rows: copies of under 1 KB cannot keep HBM busy
  GsGeo G = {};
  G.kc = k / nkc, G.nkc = nkc;
  G.group_pitch = 4 * G.kc + 64;
  G.stage_bytes = (4 * G.group_pitch + 127) / 128 * 128;
  G.tok_pitch = k + 32;
  const int nkb = k / block;
  int p = 256;  // the barriers
  G.off_bar = 0;
  G.off_red = p, p += 2 * GS_WARPS * ntg * 4 * 32 * 4;  // two buffers
  G.off_as = p, p += (8 * nkb * 4 + 127) / 128 * 128;
  *staged = rows <= 8 && ntg == 1;
  G.off_codes = p;
  if (*staged) p += (rows * G.tok_pitch + 127) / 128 * 128;
  G.off_ring = p;
  G.n_stage = (GS_SMEM_LIMIT - p) / G.stage_bytes;
  if (G.n_stage > GS_MAX_STAGES) G.n_stage = GS_MAX_STAGES;
  if (G.n_stage < 3) {  // too little room next to the staged tokens: read them through L1 instead
    if (!*staged) return false;
    *staged = false;
    p = G.off_codes, G.off_ring = p;
    G.n_stage = (GS_SMEM_LIMIT - p) / G.stage_bytes;
    if (G.n_stage > GS_MAX_STAGES) G.n_stage = GS_MAX_STAGES;
    if (G.n_stage < 3) return false;
  }
  G.total = p + G.n_stage * G.stage_bytes;
  *out = G;
  return true;
}

template <int BLOCK, typename OutT>
static cudaError_t launch_gemv_stream(const GsGeo& G, bool staged, bool pdl, int ntg, cudaStream_t s, const uint8_t* codes,
                                      const float* act_scales, const uint8_t* weight, const void* w_scales, int scale_rule,
                                      int rows, int n, int k, OutT* out, long long ldo, const float* addend, int* status) {
  int dev = 0, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return e;
  const int tiles = (n + 15) / 16;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles < sms ? tiles : sms));
  cfg.blockDim = dim3(GS_THREADS);
  cfg.dynamicSmemBytes = (size_t)G.total;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl ? 1 : 0;
  auto go = [&](auto kern) {
    static std::mutex mu;
    static std::set<std::pair<const void*, int>> done;  // the shared-memory opt-in is per kernel and device
    {
      std::lock_guard<std::mutex> lock(mu);
      if (!done.count({(const void*)kern, dev})) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GS_SMEM_LIMIT);
        if (e != cudaSuccess) return;
        done.insert({(const void*)kern, dev});
      }
    }
    e = cudaLaunchKernelEx(&cfg, kern, G, codes, act_scales, weight, w_scales, scale_rule, rows, n, k, out, ldo, addend, status);
  };
  if (ntg == 1) {
    if (staged) go(fp8_gemv_stream_kernel<1, BLOCK, true, OutT>);
    else go(fp8_gemv_stream_kernel<1, BLOCK, false, OutT>);
  } else if (ntg == 2) {
    go(fp8_gemv_stream_kernel<2, BLOCK, false, OutT>);
  } else if (ntg <= 4) {
    go(fp8_gemv_stream_kernel<4, BLOCK, false, OutT>);
  } else {
    go(fp8_gemv_stream_kernel<8, BLOCK, false, OutT>);
  }
  return e;
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

// pdl: the kernel directly before this call in the stream is one of this file's quantisers (it writes the codes and
// scales only), so the GEMV may start streaming weights while it runs
static int gemv_checked(const char* who, const uint8_t* codes, const float* act_scales, const uint8_t* weight, const void* w_scales,
                        int scale_rule, int block, int rows, int n, int k, void* out, int out_dtype, long long ldo,
                        const float* addend, cudaStream_t s, bool pdl = false, int* status = nullptr) {
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
    static const bool no_stream = [] { const char* e = std::getenv("CACHALOT_FP8_PER_LANE"); return e && e[0] == '1'; }();
    GsGeo G;
    bool staged = false;
    // up to eight tokens; beyond that the activation fragments outweigh the weights and the per-lane kernel, which
    // shares them between two row tiles, is the faster one (measured at 32 tokens)
    if (!no_stream && ntg == 1 && gs_geometry(nr, k, block, 1, &staged, &G)) {
      cudaError_t e;
      if (out_dtype == CACHALOT_BF16) {
        __nv_bfloat16* o = (__nv_bfloat16*)out + (size_t)r0 * ldo;
        e = block == 32 ? launch_gemv_stream<32>(G, staged, pdl, ntg, s, c, as, weight, w_scales, scale_rule, nr, n, k, o, ldo, ad, status)
                        : launch_gemv_stream<128>(G, staged, pdl, ntg, s, c, as, weight, w_scales, scale_rule, nr, n, k, o, ldo, ad, status);
      } else {
        float* o = (float*)out + (size_t)r0 * ldo;
        e = block == 32 ? launch_gemv_stream<32>(G, staged, pdl, ntg, s, c, as, weight, w_scales, scale_rule, nr, n, k, o, ldo, ad, status)
                        : launch_gemv_stream<128>(G, staged, pdl, ntg, s, c, as, weight, w_scales, scale_rule, nr, n, k, o, ldo, ad, status);
      }
      if (e != cudaSuccess) return fail(CACHALOT_ECUDA, "%s: %s", who, cudaGetErrorString(e));
      pdl = false;  // a further launch of this call follows a GEMV, not the quantiser
      continue;
    }
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

extern "C" int cachalot_fp8_linear(const void* x_bf16, int rows, int k, int block, int scale_rule, uint8_t* codes, float* scales,
                                   const uint8_t* weight, const void* w_scales, int n, void* out, int out_dtype,
                                   cachalot_stream_t stream) {
  int rc = cachalot_fp8_act_quant(x_bf16, rows, k, block, scale_rule, codes, scales, stream);
  if (rc) return rc;
  return gemv_checked("fp8_linear", codes, scales, weight, w_scales, scale_rule, block, rows, n, k, out, out_dtype, n, nullptr,
                      (cudaStream_t)stream, true);
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
    rc = gemv_checked("shared_expert w1", codes, scales, w1, w1_scales, scale_rule, block, rows, inter, hidden, gu, CACHALOT_BF16, ld, nullptr, s, true);
    if (rc) return rc;
    rc = gemv_checked("shared_expert w3", codes, scales, w3, w3_scales, scale_rule, block, rows, inter, hidden, gu + inter, CACHALOT_BF16, ld, nullptr, s);
  } else {  // w1 holds [2*inter, hidden] = w1 rows, then w3 rows
    rc = gemv_checked("shared_expert w13", codes, scales, w1, w1_scales, scale_rule, block, rows, 2 * inter, hidden, gu, CACHALOT_BF16, ld, nullptr, s, true);
  }
  if (rc) return rc;
  {
    const long long warps = (long long)rows * (inter / block);
    const unsigned blocks = (unsigned)((warps * 32 + 255) / 256);
    if (block == 32) swiglu_act_quant_kernel<1><<<blocks, 256, 0, s>>>(gu, gu + inter, ld, rows, inter, scale_rule, swiglu_limit, codes, scales);
    else swiglu_act_quant_kernel<4><<<blocks, 256, 0, s>>>(gu, gu + inter, ld, rows, inter, scale_rule, swiglu_limit, codes, scales);
    if ((rc = check_launch("shared_expert swiglu"))) return rc;
  }
  return gemv_checked("shared_expert w2", codes, scales, w2, w2_scales, scale_rule, block, rows, hidden, inter, out_bf16, CACHALOT_BF16, hidden, addend, s, true);
}
