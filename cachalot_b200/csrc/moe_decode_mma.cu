// Decode-time routed experts, tensor-core path.
//
// The kernels are HBM-bound dequant-GEMVs; the tensor cores are used only because they do the
// multiply-accumulate for free next to the integer work of unpacking codes.  Each warp owns a
// 16-row weight tile (the A operand of mma.sync m16n8k16, f16 in / f32 accumulate); the eight B
// columns are the activation rows that share the expert.  A lane (g = lane/4, t = lane%4) reads
// 16/8/4 contiguous bytes of rows g and g+8 per step, so the four lanes of a quad cover one
// contiguous 64/32/16-byte run of a weight row.
//
//   FP4 bank   : E2M1 byte -> f16x2 with cvt.rn.f16x2.e2m1x2, times 2**(scale - centre) as an
//                f16x2 multiply (exact); the result is scaled by 2**(centre-127) at the end.
//   2-bit bank : codes stay in place inside an f16 mantissa, (word & mask) | 0x6400 gives
//                1024 + q*4**n; the activation operand is pre-divided by 4**n and the 1024 offset
//                is removed with a pre-computed sum, then scale and bias are applied in fp32 per
//                64 or 128 columns:  acc += s*(T - 1024*xj) + b*xs.
//
// Activations are converted to f16 after a per-row power-of-two prescale (exact for bf16 inputs
// within 2**27 of the row maximum) and kept in shared memory in a padded layout that makes the
// 128-bit operand loads bank-conflict free.
#include "kernels.cuh"

namespace cachalot {
namespace {

constexpr int SEG_BYTES = 80;  // 32 halves (64 B) + 16 B pad: quad lanes land in distinct bank groups
constexpr int MAX_COLS = 8;

__host__ __device__ inline int xrow_bytes(int K) {
  int b = (K / 32) * SEG_BYTES;
  return b + ((64 - b % 128) + 128) % 128;  // row stride == 64 (mod 128) bytes
}
__device__ __forceinline__ int xoff(int k) { return (k >> 5) * SEG_BYTES + (k & 31) * 2; }

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1, const float (&c)[4]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// four E2M1 bytes (8 codes) -> four f16x2, each times the f16x2 multiplier
__device__ __forceinline__ void fp4_word(uint32_t w, uint32_t mul, uint32_t (&h)[4]) {
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "mul.rn.f16x2 %0, %0, %5;\n"
      "mul.rn.f16x2 %1, %1, %5;\n"
      "mul.rn.f16x2 %2, %2, %5;\n"
      "mul.rn.f16x2 %3, %3, %5;\n"
      "}\n"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w), "r"(mul));
}

// 2-bit: sixteen codes of a word -> eight f16x2 (field f in the low half, field f+8 in the high
// half), value 1024 + q * 4**pos with pos = {2,3,2,3,4,2,3,4}[f]
// M = 0x64006400 arrives through a kernel parameter so that it lives in a register: (x & imm) | reg is
// one LOP3, whereas with two immediates each field would cost two instructions.
__device__ __forceinline__ void q2_word(uint32_t w, uint32_t M, uint32_t (&h)[8]) {
  const uint32_t s1 = w << 4, s2 = w >> 6;
  h[0] = (s1 & 0x00300030u) | M;
  h[1] = (s1 & 0x00C000C0u) | M;
  h[2] = (w & 0x00300030u) | M;
  h[3] = (w & 0x00C000C0u) | M;
  h[4] = (w & 0x03000300u) | M;
  h[5] = (s2 & 0x00300030u) | M;
  h[6] = (s2 & 0x00C000C0u) | M;
  h[7] = (s2 & 0x03000300u) | M;
}
__device__ __forceinline__ float q2_div(int f) {  // 4**pos of field f (f in 0..7)
  const int pos = (0x43243232 >> (4 * f)) & 15;    // nibble f = {2,3,2,3,4,2,3,4}[f]
  return (float)(1 << (2 * pos));
}

template <int FMT, int KCH>
struct Geo {
  // 32-bit words each lane reads per row per chunk, and MMAs per word
  static constexpr int WORDS = FMT == CACHALOT_BANK_FP4 ? KCH / 32 : KCH / 64;
  static constexpr int MMA_PER_WORD = FMT == CACHALOT_BANK_FP4 ? 2 : 4;
  static constexpr int LANE_K = KCH / 4;            // activations per lane per chunk
  static constexpr int LANE_BYTES = WORDS * 4;      // weight bytes per lane per row per chunk
  static constexpr int XQ = LANE_K / 8;             // 128-bit operand loads per lane per chunk
};

template <int WORDS>
struct Wv {
  uint32_t w[WORDS];
};
template <int WORDS>
__device__ __forceinline__ Wv<WORDS> ld_words(const uint8_t* p) {
  Wv<WORDS> r;
  if constexpr (WORDS == 4) {
    uint4 v = ld_stream_u4(p);
    r.w[0] = v.x, r.w[1] = v.y, r.w[2] = v.z, r.w[3] = v.w;
  } else if constexpr (WORDS == 2) {
    uint2 v = ld_stream_u2(p);
    r.w[0] = v.x, r.w[1] = v.y;
  } else {
    r.w[0] = ld_stream_u32(p);
  }
  return r;
}

// One chunk of one weight matrix for rows g and g+8 of the tile: D = C + A(16 x KCH) * B(KCH x 8).
// xq: the lane's B operand (XQ x uint4).  FP4: mula/mulb are the f16x2 scale multipliers.
template <int FMT, int KCH>
__device__ __forceinline__ void chunk_mma(float (&D)[4], const float (&C)[4], const Wv<Geo<FMT, KCH>::WORDS>& ra,
                                          const Wv<Geo<FMT, KCH>::WORDS>& rb, uint32_t mula, uint32_t mulb,
                                          const uint4 (&xq)[Geo<FMT, KCH>::XQ]) {
  // affine: mula carries the 0x64006400 magic
  using G = Geo<FMT, KCH>;
#pragma unroll
  for (int wd = 0; wd < G::WORDS; ++wd) {
    if constexpr (FMT == CACHALOT_BANK_FP4) {
      uint32_t ha[4], hb[4];
      fp4_word(ra.w[wd], mula, ha);
      fp4_word(rb.w[wd], mulb, hb);
      const uint4 q = xq[wd];  // 8 activations = this word's 8 codes
      if (wd == 0)
        mma16816(D, ha[0], hb[0], ha[1], hb[1], q.x, q.y, C);
      else
        mma16816(D, ha[0], hb[0], ha[1], hb[1], q.x, q.y, D);
      mma16816(D, ha[2], hb[2], ha[3], hb[3], q.z, q.w, D);
    } else {
      uint32_t ha[8], hb[8];
      q2_word(ra.w[wd], mula, ha);
      q2_word(rb.w[wd], mula, hb);
      const uint4 q0 = xq[2 * wd], q1 = xq[2 * wd + 1];  // 16 activations, permuted and pre-divided
      if (wd == 0)
        mma16816(D, ha[0], hb[0], ha[1], hb[1], q0.x, q0.y, C);
      else
        mma16816(D, ha[0], hb[0], ha[1], hb[1], q0.x, q0.y, D);
      mma16816(D, ha[2], hb[2], ha[3], hb[3], q0.z, q0.w, D);
      mma16816(D, ha[4], hb[4], ha[5], hb[5], q1.x, q1.y, D);
      mma16816(D, ha[6], hb[6], ha[7], hb[7], q1.z, q1.w, D);
    }
  }
}

// ---- activation staging --------------------------------------------------------------------
// All warps of the CTA convert up to MAX_COLS source rows of K floats into the f16 operand layout.
// Warps are split evenly over the rows; a lane converts one 16-column region per step and the
// loads of a step are issued before any of them is used.
//   FP4   : natural order, value v*P (+ the residual v*P - hi in `lo` for a second MMA pass)
//   2-bit : per region the eight pairs (v[r], v[r+8]) / 4**pos(r); xs/xj get the per-chunk sums
//           of v*P and of the rounded, divided values
// P is a power of two per row that puts the row maximum in [2**13, 2**14).
// load16(row, k, float (&v)[16]) reads 16 consecutive source values.  Contains __syncthreads.
template <int FMT, int KCH, int NWARPS, typename Load16>
__device__ __forceinline__ void stage_rows(uint8_t* hi, uint8_t* lo, int xrow, int ncol, int K, Load16 load16,
                                           float* inv_p, float* xsj /* (xs, -1024 xj) per column and chunk */, int nch,
                                           float* wmax /*[MAX_COLS*NWARPS]*/) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nreg = K / 16;
  const int wpc = NWARPS / ncol;                 // warps per row (ncol <= MAX_COLS <= NWARPS)
  const int c = warp / wpc, wi = warp - c * wpc;  // this warp's row and its index among the row's warps
  const bool active = c < ncol;
  const int stride = wpc * 32;
  const int steps = (nreg + stride - 1) / stride;
  for (int i = threadIdx.x; i < MAX_COLS * NWARPS; i += blockDim.x) wmax[i] = 0.f;
  __syncthreads();
  if (active) {
    float amax = 0.f;
    for (int s = 0; s < steps; s += 2) {
      const int r0 = (s * wpc + wi) * 32 + lane, r1 = r0 + stride;
      float v0[16], v1[16];
      const bool ok0 = r0 < nreg, ok1 = (s + 1 < steps) && r1 < nreg;
      if (ok0) load16(c, r0 * 16, v0);
      if (ok1) load16(c, r1 * 16, v1);
      if (ok0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v0[i]));
      }
      if (ok1) {
#pragma unroll
        for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v1[i]));
      }
    }
    amax = warp_max(amax);
    if (lane == 0) wmax[c * NWARPS + wi] = amax;
  }
  __syncthreads();
  if (active) {
    float amax = 0.f;
    for (int w = 0; w < wpc; ++w) amax = fmaxf(amax, wmax[c * NWARPS + w]);
    float P = 1.f, invP = 1.f;
    const int ex = (int)((__float_as_uint(amax) >> 23) & 0xffu);
    if (ex > 0 && ex < 255) {  // finite, normal, non-zero
      const int e = min(max(13 - (ex - 127), -120), 120);
      P = __uint_as_float((uint32_t)(e + 127) << 23);
      invP = __uint_as_float((uint32_t)(127 - e) << 23);
    }
    if (wi == 0 && lane == 0) inv_p[c] = invP;
    uint8_t* hrow = hi + c * xrow;
    uint8_t* lrow = lo ? lo + c * xrow : nullptr;
    for (int s = 0; s < steps; ++s) {  // warp-uniform trip count: the chunk sums use shuffles
      const int reg = (s * wpc + wi) * 32 + lane;
      const bool valid = reg < nreg;
      float v[16];
      if (valid) {
        load16(c, reg * 16, v);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] *= P;
      uint32_t pk[8], pl[8];
      float sum = 0.f, jsum = 0.f;
      if constexpr (FMT == CACHALOT_BANK_FP4) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
          pk[i] = *reinterpret_cast<uint32_t*>(&h);
          float2 f = __half22float2(h);
          __half2 l = __floats2half2_rn(v[2 * i] - f.x, v[2 * i + 1] - f.y);
          pl[i] = *reinterpret_cast<uint32_t*>(&l);
        }
      } else {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const int pos = (0x43243232 >> (4 * r)) & 15;
          const float inv = 1.0f / (float)(1 << (2 * pos));  // a constant after unrolling
          __half2 h = __floats2half2_rn(v[r] * inv, v[r + 8] * inv);
          pk[r] = *reinterpret_cast<uint32_t*>(&h);
          float2 f = __half22float2(h);
          sum += v[r] + v[r + 8];
          jsum += f.x + f.y;
          pl[r] = 0;
        }
      }
      if (valid) {
        uint4* dst = reinterpret_cast<uint4*>(hrow + xoff(reg * 16));
        dst[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        dst[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        if (FMT == CACHALOT_BANK_FP4 && lrow) {
          uint4* dl = reinterpret_cast<uint4*>(lrow + xoff(reg * 16));
          dl[0] = make_uint4(pl[0], pl[1], pl[2], pl[3]);
          dl[1] = make_uint4(pl[4], pl[5], pl[6], pl[7]);
        }
      }
      if constexpr (FMT == CACHALOT_BANK_AFFINE) {
        // a chunk is KCH/16 consecutive regions = consecutive lanes of this warp
#pragma unroll
        for (int o = KCH / 32; o > 0; o >>= 1) {
          sum += __shfl_xor_sync(0xffffffffu, sum, o);
          jsum += __shfl_xor_sync(0xffffffffu, jsum, o);
        }
        if (valid && (lane & (KCH / 16 - 1)) == 0) {
          reinterpret_cast<float2*>(xsj)[c * nch + reg / (KCH / 16)] = make_float2(sum, -1024.f * jsum);
        }
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void load16_bf16(const __nv_bfloat16* p, float (&v)[16]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p), b = *reinterpret_cast<const uint4*>(p + 8);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void load16_f32(const float* p, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 a = reinterpret_cast<const float4*>(p)[i];
    v[4 * i] = a.x, v[4 * i + 1] = a.y, v[4 * i + 2] = a.z, v[4 * i + 3] = a.w;
  }
}

// warp-level copy of `bytes` from global to shared; 16-byte cp.async when both sides allow it
__device__ __forceinline__ void warp_copy_async(uint8_t* dst, const uint8_t* src, int bytes, int lane) {
  if (((reinterpret_cast<uintptr_t>(src) | (uintptr_t)__cvta_generic_to_shared(dst)) & 15) == 0) {
    const int n16 = bytes >> 4;
    for (int i = lane; i < n16; i += 32) {
      const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst + i * 16);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src + i * 16));
    }
    for (int i = (n16 << 4) + lane; i < bytes; i += 32) dst[i] = src[i];
  } else {
    for (int i0 = 0; i0 < bytes; i0 += 128) {  // four independent byte loads per lane before the stores
      uint8_t v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = i0 + j * 32 + lane;
        v[j] = i < bytes ? src[i] : 0;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = i0 + j * 32 + lane;
        if (i < bytes) dst[i] = v[j];
      }
    }
  }
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ---- the streaming kernel --------------------------------------------------------------------
// PHASE 0 (gate/up): unit = (group, 8 intermediate indices); MMA rows 0..7 are the gate rows,
//   rows 8..15 the up rows of the same indices, so a lane ends with gate (c0,c1) and up (c2,c3) of
//   its index and applies SwiGLU and the router weight itself.
// PHASE 1 (down):    unit = (group, 16 output rows); each routed row's 16 results go to a global
//   [rows, H] buffer; the warp that delivers the last of a token's k contributions for the tile
//   (an atomic counter per token and tile) sums them in route-slot order and writes the output.
// A unit is streamed over the whole K by ONE warp: no cross-warp reduction, no block barrier in
// the loop.  A CTA takes a contiguous range of units, stages the activation rows of a group once
// (skipped when the same single row is already staged, as in batch 1 where every group shares the
// token) and hands tiles to its warps round-robin.  A warp issues the first PF chunks of its unit
// and the copy of the unit's scales before the staging barrier, so the weight stream starts at once.

constexpr int ST_WARPS = 8;

template <int FMT, int KCH>
struct Pf {  // chunks in flight per warp
#ifndef CB_PF_DIV
#define CB_PF_DIV 1
#endif
#ifndef CB_MINB
#define CB_MINB 2
#endif
  static constexpr int N = (FMT == CACHALOT_BANK_FP4 ? 512 : 1024) / KCH / CB_PF_DIV;
};

struct StSmem {
  int xrow;     // bytes per operand row
  int n_raw;    // affine: raw scale halves per warp (the raw biases follow at raw_half); FP4: raw scale bytes
  int raw_half; // affine: bytes of the raw scale array
  int sc_warp;  // bytes of a warp's scale area: raw copy, then converted values
  int off_cv;   // offset of the converted values inside the warp area
  int off_hi, off_lo, off_invp, off_xsj, off_wmax, off_sc, total;
};
__host__ __device__ inline StSmem st_layout(int fmt, int K, int kch, int cols, bool hilo) {
  StSmem s;
  s.xrow = xrow_bytes(K);
  int p = 0;
  s.off_hi = p, p += cols * s.xrow;
  s.off_lo = p, p += hilo ? cols * s.xrow : 0;
  s.off_invp = p, p += MAX_COLS * 4;
  p = (p + 15) & ~15;
  const int nch = K / kch;
  s.off_xsj = p, p += (fmt == CACHALOT_BANK_AFFINE ? cols * nch * 8 : 0);  // float2 (xs, -1024 xj) per column and chunk
  s.off_wmax = p, p += MAX_COLS * ST_WARPS * 4;
  p = (p + 15) & ~15;
  if (fmt == CACHALOT_BANK_FP4) {
    s.n_raw = 16 * (K / 32);
    s.raw_half = 0;
    s.off_cv = (s.n_raw + 15) & ~15;
    s.sc_warp = s.off_cv + s.n_raw * 2;  // one f16 multiplier per (tile row, block)
  } else {
    s.n_raw = 16 * K / 128 + 16;  // two runs of 8 rows, or one of 16, each 16-byte aligned with a spare group
    s.raw_half = (s.n_raw * 2 + 15) & ~15;
    s.off_cv = 2 * s.raw_half;
    s.sc_warp = s.off_cv + 16 * nch * 8;  // float2 (scale, bias) per (tile row, chunk)
  }
  s.sc_warp = (s.sc_warp + 15) & ~15;
  s.off_sc = p, p += ST_WARPS * s.sc_warp;
  s.total = p;
  return s;
}

template <int FMT, int KCH, int PHASE, bool HILO, bool ONECOL, typename OutT>
__global__ void __launch_bounds__(ST_WARPS * 32, CB_MINB)
stream_kernel(BankView bank, const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ slots,
              const float* __restrict__ gate_w, Plan plan, int R, int k, int cols, float limit, int numerics,
              float* __restrict__ hidden, float* __restrict__ ybuf, int* __restrict__ counters, OutT* __restrict__ out,
              int* __restrict__ status, uint32_t magic /* 0x64006400, see q2_word */) {
  using G = Geo<FMT, KCH>;
  constexpr int PF = Pf<FMT, KCH>::N;
  constexpr int TILE = PHASE == 0 ? 8 : 16;  // outputs per unit
  constexpr int CHUNK_BYTES = KCH / (FMT == CACHALOT_BANK_FP4 ? 2 : 4);
  constexpr int XSTEP = (KCH / 32) * SEG_BYTES;  // operand bytes per chunk
  extern __shared__ __align__(16) uint8_t smem[];
  const int H = bank.hidden, I = bank.inter;
  const int K = PHASE == 0 ? H : I;   // reduction length
  const int N = PHASE == 0 ? I : H;   // outputs
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int n_groups = plan.n_groups ? *plan.n_groups : R;
  const int tiles = N / TILE;
  const long long U = (long long)n_groups * tiles;
  const long long u_begin = U * blockIdx.x / gridDim.x, u_end = U * (blockIdx.x + 1) / gridDim.x;
  if constexpr (PHASE == 0) {  // the down launch's arrival counters start at zero
    const int n_cnt = (R / k) * (H / 16);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_cnt; i += gridDim.x * blockDim.x) counters[i] = 0;
  }
  if (u_end <= u_begin) return;
  const StSmem L = st_layout(FMT, K, KCH, cols, HILO);
  float* invp = reinterpret_cast<float*>(smem + L.off_invp);
  float2* xsj = reinterpret_cast<float2*>(smem + L.off_xsj);
  float* wmax = reinterpret_cast<float*>(smem + L.off_wmax);
  uint8_t* my_sc = smem + L.off_sc + warp * L.sc_warp;
  const int nch = K / KCH;
  const int row_bytes = FMT == CACHALOT_BANK_FP4 ? K / 2 : K / 4;
  // tensors of the record: weight / scale (/ bias) of the A rows 0..7 and 8..15
  const int tA = PHASE == 0 ? 0 : (FMT == CACHALOT_BANK_FP4 ? 2 : 3);
  const int tB = PHASE == 0 ? (FMT == CACHALOT_BANK_FP4 ? 4 : 6) : tA;
  const int lane_off = t * G::LANE_BYTES;
  int staged_row = -1;  // >= 0: column 0 holds exactly this source row
  int range_flag = 0;

  for (int grp = (int)(u_begin / tiles); grp <= (int)((u_end - 1) / tiles); ++grp) {
    const long long gbase = (long long)grp * tiles;
    const int tile_lo = (int)(max(u_begin, gbase) - gbase), tile_hi = (int)(min(u_end, gbase + tiles) - gbase);
    int r_begin, r_end, slot;
    if (plan.order) {
      r_begin = plan.group_start[grp], r_end = plan.group_start[grp + 1], slot = plan.group_slot[grp];
    } else {
      r_begin = grp, r_end = grp + 1, slot = slots[grp];
    }
    const bool absent = slot < 0 || slot >= bank.n_slots;  // zero contribution, never an out-of-range read
    if (PHASE == 0 && slot >= bank.n_slots && status && threadIdx.x == 0) atomicOr(status, CACHALOT_STATUS_SLOT_RANGE);
    const uint8_t* rec = bank.base + (size_t)(absent ? 0 : slot) * bank.record_bytes;
    const uint8_t* WA = rec + bank.off[tA];
    const uint8_t* WB = rec + bank.off[tB];

    for (int tc = r_begin; tc < r_end; tc += cols) {
      const int ncol = min(cols, r_end - tc);
      const int r0 = plan.order ? plan.order[tc] : tc;
      const int src0 = PHASE == 0 ? r0 / k : r0;  // source row of column 0 (token for gate/up, routed row for down)

      Wv<G::WORDS> bufa[PF], bufb[PF];
      const uint8_t* pa = nullptr;
      const uint8_t* pb = nullptr;
      int n_a = 0;         // affine: pairs in the first run (the second run starts there)
      long long gf = 0;    // affine: first flattened group of the tile
      int tile = tile_lo + warp;
      // issue: the first PF chunks of the unit, and the copy of its raw scales
      auto issue = [&](int tl) {
        const long long ra = PHASE == 0 ? (long long)tl * 8 + g : (long long)tl * 16 + g;
        const long long rb = PHASE == 0 ? ra : ra + 8;
        pa = WA + ra * row_bytes + lane_off;
        pb = WB + rb * row_bytes + lane_off;
#pragma unroll
        for (int j = 0; j < PF; ++j) {
          if (j < nch) {
            bufa[j] = ld_words<G::WORDS>(pa + j * CHUNK_BYTES);
            bufb[j] = ld_words<G::WORDS>(pb + j * CHUNK_BYTES);
          }
        }
        __syncwarp();  // the previous unit's scale reads are done
        if constexpr (FMT == CACHALOT_BANK_FP4) {
          const int per_row = K / 32;
          if constexpr (PHASE == 0) {
            warp_copy_async(my_sc, rec + bank.off[tA + 1] + (size_t)tl * 8 * per_row, 8 * per_row, lane);
            warp_copy_async(my_sc + 8 * per_row, rec + bank.off[tB + 1] + (size_t)tl * 8 * per_row, 8 * per_row, lane);
          } else {
            warp_copy_async(my_sc, rec + bank.off[tA + 1] + (size_t)tl * 16 * per_row, 16 * per_row, lane);
          }
        } else {
          // groups of 128 over the flattened matrix: rows [row0, row0 + n) touch groups [glo, ghi]
          const long long row0 = (long long)tl * TILE;
          const int nrows = PHASE == 0 ? 8 : 16;
          const long long glo = (row0 * K) >> 7, ghi = ((row0 + nrows) * (long long)K - 1) >> 7;
          gf = glo;
          n_a = (int)(ghi - glo + 1);
          warp_copy_async(my_sc, rec + bank.off[tA + 1] + glo * 2, n_a * 2, lane);
          warp_copy_async(my_sc + L.raw_half, rec + bank.off[tA + 2] + glo * 2, n_a * 2, lane);
          if constexpr (PHASE == 0) {
            const int o2 = (n_a * 2 + 15) & ~15;
            warp_copy_async(my_sc + o2, rec + bank.off[tB + 1] + glo * 2, n_a * 2, lane);
            warp_copy_async(my_sc + L.raw_half + o2, rec + bank.off[tB + 2] + glo * 2, n_a * 2, lane);
          }
        }
      };
      bool have = tile < tile_hi && !absent;
      if (have) issue(tile);

      if (!absent && !(ncol == 1 && staged_row == src0)) {
        __syncthreads();  // every warp is done with the previous operand rows
        float* xs_tmp = reinterpret_cast<float*>(xsj);  // filled as [col][chunk] pairs below
        if constexpr (PHASE == 0) {
          stage_rows<FMT, KCH, ST_WARPS>(
              smem + L.off_hi, nullptr, L.xrow, ncol, K,
              [&](int c, int kk, float(&v)[16]) {
                const int r = plan.order ? plan.order[tc + c] : tc + c;
                load16_bf16(x + (size_t)(r / k) * K + kk, v);
              },
              invp, xs_tmp, nch, wmax);
        } else {
          stage_rows<FMT, KCH, ST_WARPS>(
              smem + L.off_hi, HILO ? smem + L.off_lo : nullptr, L.xrow, ncol, K,
              [&](int c, int kk, float(&v)[16]) {
                const int r = plan.order ? plan.order[tc + c] : tc + c;
                load16_f32(hidden + (size_t)r * K + kk, v);
              },
              invp, xs_tmp, nch, wmax);
        }
        staged_row = ncol == 1 ? src0 : -1;
      }

      if (absent) {
        // zero rows: PHASE 0 clears the hidden rows of its tiles; PHASE 1 delivers zeros below
        if constexpr (PHASE == 0) {
          const int span = (tile_hi - tile_lo) * 8;
          for (int idx = threadIdx.x; idx < ncol * span; idx += blockDim.x) {
            const int rr = tc + idx / span;
            const int r = plan.order ? plan.order[rr] : rr;
            hidden[(size_t)r * I + tile_lo * 8 + idx % span] = 0.f;
          }
        }
      }

      for (; tile < tile_hi; tile += ST_WARPS) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        if (!absent) {
          if (!have) issue(tile);
          have = false;
          cp_async_wait_all();
          __syncwarp();
          // convert the raw scales once per unit into one entry per (tile row, chunk)
          if constexpr (FMT == CACHALOT_BANK_FP4) {
            const uint32_t* raw = reinterpret_cast<const uint32_t*>(my_sc);
            uint2* cvw = reinterpret_cast<uint2*>(my_sc + L.off_cv);
            for (int i = lane; i < L.n_raw / 4; i += 32) {
              const uint32_t w = raw[i];
              uint32_t m[4];
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                int e = (int)((w >> (8 * b)) & 0xffu) - bank.scale_centre + 15;
                if (e < 1 || e > 28) range_flag = 1, e = min(max(e, 1), 28);  // 6 * 2**13 is the largest product f16 holds
                m[b] = (uint32_t)e << 10;
              }
              cvw[i] = make_uint2(m[0] | (m[1] << 16), m[2] | (m[3] << 16));
            }
          } else {
            const uint16_t* S = reinterpret_cast<const uint16_t*>(my_sc);
            const uint16_t* Bv = reinterpret_cast<const uint16_t*>(my_sc + L.raw_half);
            float2* cvw = reinterpret_cast<float2*>(my_sc + L.off_cv);
            const bool f16s = bank.scale_dtype == CACHALOT_F16;
            const int o2 = ((n_a * 2 + 15) & ~15) / 2;  // the second run (up rows) in the raw arrays
            const long long row0 = (long long)tile * TILE;
            for (int i = lane; i < 16 * nch; i += 32) {
              const int lr = i / nch, c = i - lr * nch;  // tile row 0..15 (PHASE 0: 0..7 gate, 8..15 up), chunk
              const long long row = PHASE == 0 ? row0 + (lr & 7) : row0 + lr;
              const int src = (int)(((row * K + (long long)c * KCH) >> 7) - gf) + ((PHASE == 0 && lr >= 8) ? o2 : 0);
              const uint16_t sv = S[src], bv = Bv[src];
              float2 v;
              if (f16s) {
                v.x = __half2float(__ushort_as_half(sv)), v.y = __half2float(__ushort_as_half(bv));
              } else {
                v.x = __uint_as_float((uint32_t)sv << 16), v.y = __uint_as_float((uint32_t)bv << 16);
              }
              cvw[i] = v;
            }
          }
          __syncwarp();

          // Per-lane pointers of the chunk loop; every address inside it is pointer + constant.
          // Operand columns at or beyond ncol are never stored and columns do not mix in the MMA, so
          // their lanes simply read the last valid row.
          const int brow = min(g, ncol - 1);
          const uint8_t* xp = smem + L.off_hi + brow * L.xrow + xoff(t * G::LANE_K);
          const float2* cva = reinterpret_cast<const float2*>(my_sc + L.off_cv) + g * nch;
          const float2* cvb = cva + 8 * nch;
          const float2* z0p = xsj + min(2 * t, ncol - 1) * nch;
          const float2* z1p = xsj + min(2 * t + 1, ncol - 1) * nch;
          const uint16_t* mula_p = reinterpret_cast<const uint16_t*>(my_sc + L.off_cv) + g * (K / 32) + ((t * G::LANE_K) >> 5);
          const uint16_t* mulb_p = mula_p + 8 * (K / 32);
          const float zero4[4] = {0.f, 0.f, 0.f, 0.f};

          for (int c0 = 0; c0 < nch; c0 += PF) {
            pa += PF * CHUNK_BYTES, pb += PF * CHUNK_BYTES;  // now the addresses of chunk c0 + PF
#pragma unroll
            for (int j = 0; j < PF; ++j) {
              if (c0 + j < nch) {
                uint4 xq[G::XQ];
#pragma unroll
                for (int q = 0; q < G::XQ; ++q) xq[q] = *reinterpret_cast<const uint4*>(xp + j * XSTEP + q * 16);
                if constexpr (FMT == CACHALOT_BANK_FP4) {
                  const uint32_t ma = (uint32_t)mula_p[j * (KCH / 32)] * 0x00010001u;
                  const uint32_t mb = (uint32_t)mulb_p[j * (KCH / 32)] * 0x00010001u;
                  chunk_mma<FMT, KCH>(acc, acc, bufa[j], bufb[j], ma, mb, xq);
                  if constexpr (HILO) {
                    uint4 xl[G::XQ];
#pragma unroll
                    for (int q = 0; q < G::XQ; ++q)
                      xl[q] = *reinterpret_cast<const uint4*>(xp + (L.off_lo - L.off_hi) + j * XSTEP + q * 16);
                    chunk_mma<FMT, KCH>(acc, acc, bufa[j], bufb[j], ma, mb, xl);
                  }
                } else {
                  float T[4];
                  chunk_mma<FMT, KCH>(T, zero4, bufa[j], bufb[j], magic, 0, xq);
                  const float2 sa = cva[j], sb = cvb[j];
                  const float2 z0 = z0p[j];
                  acc[0] = fmaf(sa.x, T[0] + z0.y, fmaf(sa.y, z0.x, acc[0]));
                  acc[2] = fmaf(sb.x, T[2] + z0.y, fmaf(sb.y, z0.x, acc[2]));
                  if constexpr (!ONECOL) {
                    const float2 z1 = z1p[j];
                    acc[1] = fmaf(sa.x, T[1] + z1.y, fmaf(sa.y, z1.x, acc[1]));
                    acc[3] = fmaf(sb.x, T[3] + z1.y, fmaf(sb.y, z1.x, acc[3]));
                  }
                }
                // the words of chunk c0 + j are consumed: refill the slot with chunk c0 + j + PF
                if (c0 + j + PF < nch) {
                  bufa[j] = ld_words<G::WORDS>(pa + j * CHUNK_BYTES);
                  bufb[j] = ld_words<G::WORDS>(pb + j * CHUNK_BYTES);
                }
              }
            }
            xp += PF * XSTEP;
            cva += PF, cvb += PF, z0p += PF, z1p += PF;
            mula_p += PF * (KCH / 32), mulb_p += PF * (KCH / 32);
          }
        }
        // epilogue: this lane holds rows g, g+8 x columns 2t, 2t+1
        float post_fmt = 1.f;
        if constexpr (FMT == CACHALOT_BANK_FP4) post_fmt = e8m0_to_f32((uint32_t)bank.scale_centre);
        if constexpr (PHASE == 0) {
          if (!absent) {
#pragma unroll
            for (int e = 0; e < (ONECOL ? 1 : 2); ++e) {
              const int col = 2 * t + e;
              if (col < ncol) {
                const float post = invp[col] * post_fmt;
                float gv = acc[e] * post, uv = acc[2 + e] * post;
                if (numerics != CACHALOT_NUMERICS_F32) gv = bf16_round(gv), uv = bf16_round(uv);
                const int r = plan.order ? plan.order[tc + col] : tc + col;
                float h = swiglu(gv, uv, limit) * gate_w[r];
                if (numerics == CACHALOT_NUMERICS_BF16) h = bf16_round(h);
                hidden[(size_t)r * I + tile * 8 + g] = h;
              }
            }
          }
        } else {
          const int n0 = tile * 16;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = 2 * t + (e & 1), row = g + (e >> 1) * 8;
            if (col < ncol && !(ONECOL && (e & 1))) {
              float y = absent ? 0.f : acc[e] * invp[col] * post_fmt;
              if (numerics != CACHALOT_NUMERICS_F32) y = bf16_round(y);
              const int r = plan.order ? plan.order[tc + col] : tc + col;
              ybuf[(size_t)r * H + n0 + row] = y;
            }
          }
          __threadfence();
          __syncwarp();
          // one lane per column reports the arrival; the last of a token's k combines in slot order
          int last_tok = -1;
          if (lane < ncol) {
            const int r = plan.order ? plan.order[tc + lane] : tc + lane;
            const int tok = r / k;
            const int old = atomicAdd(&counters[tok * tiles + tile], 1);
            if (old == k - 1) last_tok = tok;
          }
#pragma unroll 1
          for (int c = 0; c < ncol; ++c) {
            const int tok = __shfl_sync(0xffffffffu, last_tok, c);
            if (tok >= 0) {
              __threadfence();
              if (lane < 16) {
                float total = 0.f;
                for (int j = 0; j < k; ++j) total += __ldcg(ybuf + (size_t)(tok * k + j) * H + n0 + lane);
                if constexpr (sizeof(OutT) == 2)
                  out[(size_t)tok * H + n0 + lane] = __float2bfloat16_rn(total);
                else
                  out[(size_t)tok * H + n0 + lane] = total;
              }
              if (lane == 0) counters[tok * tiles + tile] = 0;
            }
          }
        }
      }
    }
  }
  if (range_flag && status) atomicOr(status, CACHALOT_STATUS_SCALE_RANGE);
}

// ---- grouping (rows > 1) --------------------------------------------------------------------
// Single CTA: stable rank of every routed row by slot, then runs of equal slot become groups.
__global__ void plan_kernel(const int32_t* __restrict__ slots, int R, int32_t* __restrict__ n_groups,
                            int32_t* __restrict__ group_start, int32_t* __restrict__ order,
                            int32_t* __restrict__ group_slot) {
  extern __shared__ int32_t sh[];  // [R] slots, [R] sorted slot
  int32_t* s_in = sh;
  int32_t* s_sorted = sh + R;
  for (int i = threadIdx.x; i < R; i += blockDim.x) s_in[i] = slots[i];
  __syncthreads();
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const int v = s_in[i];
    int rank = 0;
    for (int j = 0; j < R; ++j) {
      const int o = s_in[j];
      rank += (o < v || (o == v && j < i)) ? 1 : 0;
    }
    order[rank] = i;
    s_sorted[rank] = v;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int ng = 0;
    for (int i = 0; i < R; ++i) {
      if (i == 0 || s_sorted[i] != s_sorted[i - 1]) {
        group_start[ng] = i;
        group_slot[ng] = s_sorted[i];
        ++ng;
      }
    }
    group_start[ng] = R;
    *n_groups = ng;
  }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  }
  return n;
}

}  // namespace

static int kch_for(int K) { return K % 128 == 0 ? 128 : 64; }

bool decode_mma_supported(const BankView& v, int rows, int k) {
  const long long R = (long long)rows * k;
  if (v.hidden % 64 || v.inter % 64) return false;
  if (R > 1024) return false;  // the grouping kernel is a single CTA
  if (v.format == CACHALOT_BANK_AFFINE && (v.group != 128 || v.bits != 2)) return false;
  if (st_layout(v.format, v.inter, kch_for(v.inter), MAX_COLS, true).total > 200 * 1024) return false;
  if (st_layout(v.format, v.hidden, kch_for(v.hidden), MAX_COLS, false).total > 200 * 1024) return false;
  return true;
}

// hidden [R, I] f32 | ybuf [R, H] f32 | counters [rows * H/16] i32 | plan (3R + 8) i32
size_t decode_mma_workspace_bytes(int hidden, int inter, int rows, int k) {
  const size_t R = (size_t)rows * k;
  return align_up(R * inter * sizeof(float), 256) + align_up(R * hidden * sizeof(float), 256) +
         align_up((size_t)rows * (hidden / 16 + 1) * sizeof(int32_t), 256) + align_up((3 * R + 8) * sizeof(int32_t), 256);
}

template <int FMT>
static int launch_fmt(const BankView& v, const void* x, const int32_t* slots, const float* gate_w, int rows, int k,
                      float limit, int numerics_flags, void* workspace, void* out, int out_dtype, int* status,
                      cudaStream_t stream) {
  const int numerics = numerics_flags & 0xff;
  const bool do_gate_up = !(numerics_flags & CACHALOT_DECODE_ONLY_DOWN);
  const bool do_down = !(numerics_flags & CACHALOT_DECODE_ONLY_GATE_UP);
  const int H = v.hidden, I = v.inter, R = rows * k;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* hidden = reinterpret_cast<float*>(ws);
  ws += align_up((size_t)R * I * sizeof(float), 256);
  float* ybuf = reinterpret_cast<float*>(ws);
  ws += align_up((size_t)R * H * sizeof(float), 256);
  int32_t* counters = reinterpret_cast<int32_t*>(ws);
  ws += align_up((size_t)rows * (H / 16 + 1) * sizeof(int32_t), 256);
  int32_t* pl = reinterpret_cast<int32_t*>(ws);
  Plan plan = {nullptr, nullptr, nullptr, nullptr};
  if (rows > 1) {
    plan.n_groups = pl;
    plan.group_start = pl + 4;
    plan.order = pl + 4 + (R + 1);
    plan.group_slot = pl + 4 + (R + 1) + R;
    const int threads = R < 1024 ? ((R + 31) / 32) * 32 : 1024;
    plan_kernel<<<1, threads, 2 * R * sizeof(int32_t), stream>>>(slots, R, pl, pl + 4, pl + 4 + (R + 1), pl + 4 + (R + 1) + R);
  }
  const int cols = rows < MAX_COLS ? rows : MAX_COLS;
  const int max_ctas = 2 * sm_count();
  auto grid_for = [&](long long units) {
    const long long want = (units + ST_WARPS - 1) / ST_WARPS;  // about one unit per warp
    return dim3((unsigned)(want < max_ctas ? (want > 0 ? want : 1) : max_ctas));
  };
#define CACHALOT_ST(KCHV, PH, HL, OT, KK)                                                                              \
  do {                                                                                                                \
    if (cols == 1) CACHALOT_ST1(KCHV, PH, HL, true, OT, KK); else CACHALOT_ST1(KCHV, PH, HL, false, OT, KK);           \
  } while (0)
#define CACHALOT_ST1(KCHV, PH, HL, OC, OT, KK)                                                                         \
  do {                                                                                                                \
    auto kern = stream_kernel<FMT, KCHV, PH, HL, OC, OT>;                                                             \
    const StSmem L = st_layout(FMT, KK, KCHV, cols, HL);                                                              \
    smem_optin_once(kern, 200 * 1024);                                                                                \
    kern<<<grid_for((long long)R * ((PH) == 0 ? I / 8 : H / 16)), ST_WARPS * 32, L.total, stream>>>(                  \
        v, (const __nv_bfloat16*)x, slots, gate_w, plan, R, k, cols, limit, numerics, hidden, ybuf, counters,          \
        (OT*)out, status, 0x64006400u);                                                                                          \
  } while (0)
  int rc = CACHALOT_OK;
  if (do_gate_up) {
    if (kch_for(H) == 128)
      CACHALOT_ST(128, 0, false, float, H);
    else
      CACHALOT_ST(64, 0, false, float, H);
    rc = check_launch("moe_decode gate_up (mma)");
    if (rc) return rc;
  }
  if (!do_down) return rc;
  // the low-order pass is only needed when the hidden activation is not already bf16-rounded
  const bool hilo = numerics == CACHALOT_NUMERICS_F32 && FMT == CACHALOT_BANK_FP4;
  const int kch = kch_for(I);
  if (out_dtype == CACHALOT_BF16) {
    if (kch == 128) { if (hilo) CACHALOT_ST(128, 1, true, __nv_bfloat16, I); else CACHALOT_ST(128, 1, false, __nv_bfloat16, I); }
    else { if (hilo) CACHALOT_ST(64, 1, true, __nv_bfloat16, I); else CACHALOT_ST(64, 1, false, __nv_bfloat16, I); }
  } else {
    if (kch == 128) { if (hilo) CACHALOT_ST(128, 1, true, float, I); else CACHALOT_ST(128, 1, false, float, I); }
    else { if (hilo) CACHALOT_ST(64, 1, true, float, I); else CACHALOT_ST(64, 1, false, float, I); }
  }
#undef CACHALOT_ST
#undef CACHALOT_ST1
  return check_launch("moe_decode down (mma)");
}

int launch_decode_mma(const BankView& v, const void* x, const int32_t* slots, const float* gate_w, int rows, int k,
                      float limit, int numerics_flags, void* workspace, void* out, int out_dtype, int* status,
                      cudaStream_t stream) {
  if (!decode_mma_supported(v, rows, k)) return CACHALOT_EUNSUPPORTED;
  if (v.format == CACHALOT_BANK_FP4)
    return launch_fmt<CACHALOT_BANK_FP4>(v, x, slots, gate_w, rows, k, limit, numerics_flags, workspace, out, out_dtype, status, stream);
  return launch_fmt<CACHALOT_BANK_AFFINE>(v, x, slots, gate_w, rows, k, limit, numerics_flags, workspace, out, out_dtype, status, stream);
}

}  // namespace cachalot
