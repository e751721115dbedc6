// Decode-time routed experts for ONE token in ONE launch (cooperative, one CTA per SM).
//
//   phase 0 : hidden[j, i] = silu(min(g,L)) * clip(u,+-L) * gate_w[j]     g = W1_j x, u = W3_j x
//   (hidden crosses the CTAs through L2 as self-validating words: see below)
//   phase 1 : out[n]       = sum_j W2_j[n, :] . hidden[j, :]               j in routing order
//
// There is no grid barrier between the phases.  A hidden value travels through L2 as one 32-bit word that carries
// its own validity: the fp32 value rounded to 15 mantissa bits (exact for the bf16 numerics; the consumer turns it
// into 15-bit fixed point or f16 anyway) with the launch's 8-bit tag in the low byte, written and read with relaxed
// GPU-scope accesses, which are single-copy atomic per word.  A CTA that finds another launch's tag reads the word
// again (bounded).  Every launch writes all k rows (tag only, for an expert that is absent), so the tag a word held
// before is the previous launch's.  No release fence is needed, and a fence is what a barrier costs here: at GPU
// scope it waits for the SM's copies in flight, 2-3 us with the ring full.
// The experts are taken in two groups (about two thirds of the present experts, then the rest).  Every CTA owns
// a slice of the inter rows of EVERY expert and walks them expert by expert, so group A's hidden rows are long
// written by every CTA when a CTA, through with all its phase-0 units, converts them into operand form and runs
// A's part of phase 1; group B's rows are converted by the copy warps meanwhile: the skew between the CTAs and the
// second conversion hide under work.
//
// The kernel is a stream of weight bytes: HBM -> cp.async.bulk -> a ring of shared-memory stages -> registers ->
// mma.sync.  Warps 0..3 issue the copies (one lane each) and run ahead of the consumers by the depth of the ring.
// In phase 0 every copy warp brings four rows (and one scale array) of every unit; in phase 1, where a unit's 16
// rows are contiguous in the bank, two of the copy warps bring whole units, turn about: the down projection's rows
// are all on their way shortly after phase 0 ends.  The copy warps then help with the hidden rows.
// Warps 4..11 are the MMA warps.  In phase 0 they work as four pairs: a pair takes one unit, each warp of the
// pair does half of the reduction dimension and the two partial sums meet in shared memory (gate and up must be
// complete before SwiGLU).  In phase 1 every warp works alone on its half of a unit's reduction dimension and
// leaves its partial sums in shared memory; the closing sum adds halves and experts in a fixed order.
// Code that only a few warps run on their own is slow here (the kernel is larger than the instruction cache, and a
// lone warp pays every miss itself): work that several roles share goes through one non-inlined function.
//
//   unit, phase 0 : 8 rows of W1 (MMA rows 0..7) + the same 8 rows of W3 (MMA rows 8..15) of one expert
//   unit, phase 1 : 16 rows of W2 of one expert; a CTA owns whole 16-row output tiles and walks
//                   the experts in routing order, so the sum over experts needs no atomics.
//
// A lane (g = lane/4, t = lane%4) reads 16 contiguous bytes of rows g and g+8 per step, so a quad
// covers 64 contiguous bytes of a row: four "sub-blocks" that each have their own scale (FP4: a
// 32-code E8M0 block; 2-bit: 64 codes, half a scale group).  The MMA would add the four
// sub-blocks up; to keep them apart the activation operand of lane t is placed in operand column
// 2t (and 2t+1) and is zero in the others, so accumulator column 2t holds exactly the partial sum
// of the codes lane t loaded, and the scale is applied per sub-block in fp32 afterwards.
//
//   2-bit bank : codes stay packed: w & (0x03030303 << 2c) puts codes c, c+4, c+8, c+12 of a word
//                into the four u8 lanes of an IMMA operand (m16n8k32, u8 x s8 -> s32, exact) scaled
//                by 4**c; the four classes c have their own accumulators and are combined as
//                integers.  Activations are fixed point per sub-block: X = rint(x * 2**e),
//                |X| < 2**14, X = 256*hi + lo in operand columns 2t and 2t+1.
//                acc += s * 2**-e * (256*T_hi + T_lo) + b * sum(x).
//   FP4 bank   : E2M1 byte -> f16x2 (cvt.rn.f16x2.e2m1x2), HMMA m16n8k16 with f16 activations
//                scaled per sub-block by 2**e;  acc += 2**(scale-127) * 2**-e * T.
#include <cstdlib>
#include <mutex>
#include <set>
#include <utility>

#include "kernels.cuh"

#ifndef CB_UNROLL
#define CB_UNROLL 2
#endif

namespace cachalot {
namespace {

constexpr int kUnroll = CB_UNROLL;  // steps of the reduction loop unrolled together
constexpr int NPROD = 4;                          // producer warps (one issuing lane each; a lane's copies do not overlap)
constexpr int KMAX = 8;                           // routed experts per token
constexpr int MAX_TILES = 8;                      // phase-1 output tiles one CTA may own
constexpr int NISSUE1 = 2;                        // copy warps that issue phase 1's copies (the others start on the hidden rows)
constexpr int KP1 = 2;                            // parts the reduction dimension of a phase-1 unit is cut into (one warp each)
constexpr uint32_t WAIT_LIMIT = 1u << 20;         // polls before a wait gives up and flags an error
constexpr uint32_t HIDDEN_TRIES = 1u << 16;       // reads of a hidden block before a CTA gives up on the others (about 10 ms)
constexpr int SMEM_LIMIT = 227 * 1024;

template <int FMT>
struct Fm {
  // consumer warps work in pairs: the two warps of a pair split the reduction of one unit in halves and
  // share its ring stage.  An even number of pairs puts two consumer warps on every scheduler of the SM.
  // four pairs for both banks (measured: FP4 35 us per layer with four pairs, 41 us with two, 63 us with six; 2-bit
  // 25.5 us with four, 26.0 us with six)
  static constexpr int NPAIR = 4;
  static constexpr int NCW = 2 * NPAIR;
  static constexpr int NTHREADS = (NPROD + NCW) * 32;
  static constexpr int STEP = FMT == CACHALOT_BANK_FP4 ? 128 : 256;    // codes of a row per step (64 B)
  static constexpr int SUB = FMT == CACHALOT_BANK_FP4 ? 32 : 64;       // codes per sub-block (16 B)
};


// The hidden rows between the phases: KMAX rows of up to INTER_MAX tagged words (value & ~0xff | tag).  In the
// library image, zero at load, so a word is either zero (no launch has tag 0) or what an earlier launch wrote: never
// garbage that could pass for this launch's.  Every device that loads the library has its own copy; one launch at a
// time per device uses it (a launch holds every SM, so two cannot overlap).
constexpr int INTER_MAX = 8192;
__device__ uint32_t fused_hidden[KMAX * INTER_MAX];
// Layout of a row (one routed expert): 16-value blocks in chunks of 32; inside a chunk the words are ordered
// [quarter of the block 0..3][block 0..31][4 values], so that the 32 lanes of a warp, one block each, read 512
// contiguous bytes per 16-byte load.  A row is padded to whole chunks.
__device__ __forceinline__ int hidden_row_words(int inter) { return ((inter / 16 + 31) / 32) * 512; }
__device__ __forceinline__ int hidden_word(int i) {  // position of value i of a row
  const int b = i >> 4, v = i & 15;
  return (((b >> 5) * 4 + (v >> 2)) << 7) + ((b & 31) << 2) + (v & 3);
}
// {number of the next launch (never 0), CTAs of the current launch that have read it and taken their ticket}
__device__ unsigned fused_epoch[2] = {1u, 0u};

// Routing done inside the kernel (logits == nullptr: the caller passes slots and weights instead).
struct RouteArgs {
  const float* logits;        // f32 [E]
  const float* bias;          // f32 [E] or null
  const int32_t* slot_table;  // i32 [layers, E] or null (slot = expert id)
  int32_t* indices_out;       // i32 [k] or null
  float* weights_out;         // f32 [k] or null
  int layer, n_experts, mode, norm, weights_bf16;
  float gate_temp, route_scale;
};

struct Geo {
  int K[2];           // reduction length: hidden, inter
  int nsteps[2];      // steps along K (the last may be partial)
  int row_bytes[2];   // bytes of a weight row in the bank
  int sc_bytes[2];    // bytes of one scale (or bias) array of a unit
  int skew[2];        // bytes between the two 4-row halves of an 8-row tile in a stage (bank-conflict skew)
  int sc_off[2];      // offset of the scale arrays inside a stage
  int act_stride[2];  // bytes of one operand row (padded to whole steps)
  int unit_bytes[2];  // bytes copied per unit
  int tiles0;         // inter / 8
  int tiles1;         // hidden / 16
  int stage_bytes[2], nst[2];  // ring geometry per phase (the same memory, cut into stages of the phase's unit size)
  int off_ring, off_act, off_pe, off_part, off_bar, total;
  int x_off;          // x's operand row inside the operand area: at its end, clear of the first hidden rows
  int xpe_off;        // the same for x's per-sub-block entries (in entries)
  int max_tiles;      // phase-1 output tiles a CTA owns at most (sizes the partial-sum area)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, int n) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(n));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(smem_u32(b)), "r"(parity)
      : "memory");
  return ok != 0;
}
// One look at the barrier that never suspends the thread (try_wait may hold it for a while before it says no).
__device__ __forceinline__ bool mbar_test(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(smem_u32(b)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: false after WAIT_LIMIT polls (the caller flags the error and carries on).
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
    if (mbar_try(b, parity)) return true;
  return false;
}
// A long wait of a whole warp: one lane looks, with pauses, so that the waiting warps leave the shared-memory pipe to
// the warps that are being waited for; the other lanes learn of it at the warp barrier.
__device__ __forceinline__ bool mbar_wait_quiet(uint64_t* b, uint32_t parity, int lane) {
  int ok = 1;
  if (lane == 0) {
    ok = 0;
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
      if (mbar_test(b, parity)) {
        ok = 1;
        break;
      }
      __nanosleep(40);
    }
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

__device__ __forceinline__ void imma_u8s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void hmma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// four E2M1 bytes (8 codes) -> four f16x2 (low nibble in the low half)
__device__ __forceinline__ void fp4_word(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "}\n"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}

__device__ __forceinline__ void st_relaxed_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_relaxed_v4(const uint32_t* p) {
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ void unpack16_bf16(const uint4 a, const uint4 b, float (&v)[16]) {
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// Converts one 16-element block of an activation row into operand form and stores it.  Operand
// rows are laid out per step so that the eight lanes that load real data in one LDS.128 read 128
// (FP4: 64) contiguous bytes:
//   2-bit : step c = 512 B = [w 0..3][t 0..3][hi | lo][q 0..3][4 B]; the 16 values of (sub-block 4c+t,
//           16-block q) are s8 in the 4x4-transposed order [0,4,8,12 | 1,5,9,13 | 2,6,10,14 | 3,7,11,15]
//           (byte i of word w is code 4i+w of a weight word), and word w of the four blocks sits side by side
//   FP4   : step c = 256 B = [q 0..3][t 0..3][16 B]; (sub-block 4c+t, chunk q) holds 8 f16 in natural order
// and, for the first block of a sub-block, pexs = (2**-e [/64 for the 2-bit class sum], sum of x).
// The lanes that share a sub-block (4 for 2-bit, 2 for FP4) are adjacent and call this together.
template <int FMT>
__device__ __forceinline__ void convert_block(uint8_t* act_row, float2* pexs_row, int b, bool valid, float (&v)[16]) {
  constexpr int LPS = Fm<FMT>::SUB / 16;  // lanes per sub-block
  float amax = 0.f, sum = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i])), sum += v[i];
#pragma unroll
  for (int o = LPS >> 1; o > 0; o >>= 1) {
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
  }
  // 2**e * amax in [2**13, 2**14) (2-bit) or [2**10, 2**11) (FP4)
  const int ex = (int)((__float_as_uint(amax) >> 23) & 0xffu);
  int e = 0;
  if (ex > 0 && ex < 255) e = (FMT == CACHALOT_BANK_FP4 ? 10 : 13) - (ex - 127);
  e = min(max(e, -100), 100);
  const float P = __uint_as_float((uint32_t)(e + 127) << 23);
  if (!valid) return;
  if constexpr (FMT == CACHALOT_BANK_FP4) {
    uint32_t pk[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      __half2 h = __floats2half2_rn(v[2 * i] * P, v[2 * i + 1] * P);
      pk[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    const int sub = b >> 1, q0 = (b & 1) * 2;
    uint8_t* dst = act_row + (sub >> 2) * 256 + (sub & 3) * 16 + q0 * 64;
    *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    *reinterpret_cast<uint4*>(dst + 64) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
    if ((b & (LPS - 1)) == 0) pexs_row[sub] = make_float2(__uint_as_float((uint32_t)(127 - e) << 23), sum);
  } else {
    // X = rint(x * 2**e) = 256 * hi + lo with lo in [-128, 127].  With Y = X + 128, hi is byte 1 of Y and lo is byte 0
    // of Y with its top bit flipped, so the bytes are picked straight out of Y by byte permutes.
    int Y[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) Y[i] = __float2int_rn(v[i] * P) + 128;
    uint32_t ph[4], pl[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {  // word c = elements c, c+4, c+8, c+12
      ph[c] = __byte_perm(__byte_perm(Y[c], Y[c + 4], 0x0051), __byte_perm(Y[c + 8], Y[c + 12], 0x0051), 0x5410);
      pl[c] = __byte_perm(__byte_perm(Y[c], Y[c + 4], 0x0040), __byte_perm(Y[c + 8], Y[c + 12], 0x0040), 0x5410) ^ 0x80808080u;
    }
    // word c of block q goes to [c][sub-block][hi|lo][q]: a lane of the MMA loop reads its sub-block's 16 bytes of
    // every c with one load and finds the words of blocks 0..3 side by side (two MMA operand register pairs)
    const int sub = b >> 2, q = b & 3;
    uint8_t* dst = act_row + (sub >> 2) * 512 + (sub & 3) * 32 + q * 4;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      *reinterpret_cast<uint32_t*>(dst + c * 128) = ph[c];
      *reinterpret_cast<uint32_t*>(dst + c * 128 + 16) = pl[c];
    }
    // the class sum of the IMMA accumulators carries a factor 64
    if (q == 0) pexs_row[sub] = make_float2(__uint_as_float((uint32_t)(127 - e - 6) << 23), sum);
  }
}

// Makes operand rows of phase 1 from the other CTAs' hidden values.  A chunk is 32 consecutive 16-value blocks of one
// row, one block per lane (the conversion shuffles between the lanes that share a sub-block).  Warps take chunks off
// a shared counter, fetch the next chunk's words while they convert the current one's, read a chunk again until every
// word carries this launch's tag (bounded), and arrive once per finished chunk on `ready` (count = chunks of the
// group).  One copy of the code for every warp that calls it: code that few warps run on their own is fetched slowly.
// Returns true if some CTA did not deliver in time (the chunk is converted from what was there).
template <int FMT>
__device__ __noinline__ bool convert_chunks(int* next, uint64_t* ready, int nchunk, int nblk, int roww, const int* route,
                                            uint8_t* act_rows, float2* pexs_rows, int row_stride, int nsub, unsigned tag8, int lane) {
  const int per_row = roww >> 9;  // chunks of a row (padded: the last one may hold blocks past the row's end)
  bool late = false;
  auto grab = [&]() {
    int c = 0;
    if (lane == 0) c = atomicAdd(next, 1);
    return __shfl_sync(0xffffffffu, c, 0);
  };
  auto fetch = [&](int c, uint4 (&q)[4]) {
    const int r = c / per_row, ch = c - r * per_row;
    const uint32_t* src = fused_hidden + (size_t)route[r] * roww + (ch << 9) + (lane << 2);
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = ld_relaxed_v4(src + 128 * i);
  };
  uint4 qc[4], qn[4];
  int c = grab();
  if (c < nchunk) fetch(c, qc);
  while (c < nchunk) {
    const int cn = grab();
    if (cn < nchunk) fetch(cn, qn);
    const int r = c / per_row, bk = (c - r * per_row) * 32 + lane;
    const bool ok = bk < nblk;
    for (uint32_t tries = 0;; ++tries) {
      uint32_t diff = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) diff |= ((qc[i].x ^ tag8) | (qc[i].y ^ tag8) | (qc[i].z ^ tag8) | (qc[i].w ^ tag8)) & 0xffu;
      if (!__any_sync(0xffffffffu, ok && diff != 0)) break;
      if (tries >= HIDDEN_TRIES) {
        late = true;
        break;
      }
      if (tries > 4) __nanosleep(100);
      fetch(c, qc);
    }
    float v[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[4 * i] = __uint_as_float(qc[i].x & 0xffffff00u), v[4 * i + 1] = __uint_as_float(qc[i].y & 0xffffff00u);
      v[4 * i + 2] = __uint_as_float(qc[i].z & 0xffffff00u), v[4 * i + 3] = __uint_as_float(qc[i].w & 0xffffff00u);
    }
    convert_block<FMT>(act_rows + (size_t)r * row_stride, pexs_rows + r * nsub, ok ? bk : 0, ok, v);
    __syncwarp();
    if (lane == 0) mbar_arrive(ready);
    c = cn;
#pragma unroll
    for (int i = 0; i < 4; ++i) qc[i] = qn[i];
  }
  return late;
}

// d = a * b (no accumulator input: the first MMA of a chain)
__device__ __forceinline__ void imma_u8s8_z(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void hmma_f16_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

template <int SDT>
__device__ __forceinline__ float scale_f32(uint16_t raw) {
  if constexpr (SDT == CACHALOT_F16) return __half2float(__ushort_as_half(raw));
  return __uint_as_float((uint32_t)raw << 16);
}

// One step (64 bytes of rows g and g+8 per quad) of the 2-bit bank.  pb: the lane's operand bytes
// (64 B: four 16-element blocks in 4x4-transposed order), pxs = (2**-e / 64, sum x) of its sub-block.
template <int SDT, bool GUARD>
__device__ __forceinline__ void step_affine(float& accA, float& accB, const uint8_t* pa, const uint8_t* pbrow, const uint8_t* pb,
                                            const float2* ppx, const uint16_t* psA, const uint16_t* psB, int arr, bool valid) {
  const uint4 va = *reinterpret_cast<const uint4*>(pa);
  const uint4 vb = *reinterpret_cast<const uint4*>(pbrow);
  uint4 b[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) b[q] = (!GUARD || valid) ? *reinterpret_cast<const uint4*>(pb + q * 128) : make_uint4(0, 0, 0, 0);
  const float2 pxs = (!GUARD || valid) ? *ppx : make_float2(0.f, 0.f);
  const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
  const uint32_t bw[4][4] = {{b[0].x, b[0].y, b[0].z, b[0].w}, {b[1].x, b[1].y, b[1].z, b[1].w},
                             {b[2].x, b[2].y, b[2].z, b[2].w}, {b[3].x, b[3].y, b[3].z, b[3].w}};
  int T[4][4];
#pragma unroll
  for (int cl = 0; cl < 4; ++cl) {
    const uint32_t M = 0x03030303u << (2 * cl);
    // b[cl] = word cl of the lane's four 16-element blocks: each MMA's two operand registers come out of one load
    imma_u8s8_z(T[cl], wa[0] & M, wb[0] & M, wa[1] & M, wb[1] & M, bw[cl][0], bw[cl][1]);
    imma_u8s8(T[cl], wa[2] & M, wb[2] & M, wa[3] & M, wb[3] & M, bw[cl][2], bw[cl][3]);
  }
  // 64 * (T0 + T1/4 + T2/16 + T3/64) per accumulator element, then 256*hi + lo
  int R[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) R[i] = ((T[0][i] * 4 + T[1][i]) * 4 + T[2][i]) * 4 + T[3][i];
  const float fa = (float)(R[0] * 256 + R[1]) * pxs.x;
  const float fb = (float)(R[2] * 256 + R[3]) * pxs.x;
  float sa = scale_f32<SDT>(psA[0]), ba = scale_f32<SDT>(psA[arr]);
  float sb = scale_f32<SDT>(psB[0]), bb = scale_f32<SDT>(psB[arr]);
  if (GUARD && !valid) sa = ba = sb = bb = 0.f;  // entries past the row: whatever was read is discarded
  accA = fmaf(sa, fa, fmaf(ba, pxs.y, accA));
  accB = fmaf(sb, fb, fmaf(bb, pxs.y, accB));
}

template <bool GUARD>
__device__ __forceinline__ void step_fp4(float& accA, float& accB, const uint8_t* pa, const uint8_t* pbrow, const uint8_t* pb,
                                         const float2* ppx, const uint8_t* psA, const uint8_t* psB, bool valid) {
  const uint4 va = *reinterpret_cast<const uint4*>(pa);
  const uint4 vb = *reinterpret_cast<const uint4*>(pbrow);
  uint4 b[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) b[q] = (!GUARD || valid) ? *reinterpret_cast<const uint4*>(pb + q * 64) : make_uint4(0, 0, 0, 0);
  const float pe = (!GUARD || valid) ? ppx->x : 0.f;
  const uint32_t wa[4] = {va.x, va.y, va.z, va.w}, wb[4] = {vb.x, vb.y, vb.z, vb.w};
  const uint32_t bw[4][4] = {{b[0].x, b[0].y, b[0].z, b[0].w}, {b[1].x, b[1].y, b[1].z, b[1].w},
                             {b[2].x, b[2].y, b[2].z, b[2].w}, {b[3].x, b[3].y, b[3].z, b[3].w}};
  float T[4];
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    uint32_t ha[4], hb[4];
    fp4_word(wa[wd], ha);
    fp4_word(wb[wd], hb);
    if (wd == 0)
      hmma_f16_z(T, ha[0], hb[0], ha[1], hb[1], bw[wd][0], bw[wd][1]);
    else
      hmma_f16(T, ha[0], hb[0], ha[1], hb[1], bw[wd][0], bw[wd][1]);
    hmma_f16(T, ha[2], hb[2], ha[3], hb[3], bw[wd][2], bw[wd][3]);
  }
  float sa = e8m0_to_f32(*psA), sb = e8m0_to_f32(*psB);
  if (GUARD && !valid) sa = sb = 0.f;  // entries past the row: whatever was read is discarded
  accA = fmaf(T[0], sa * pe, accA);
  accB = fmaf(T[2], sb * pe, accB);
}

// One unit of one consumer warp: the lane's partial sums of MMA rows g and g+8 over the warp's part of the
// reduction (its own sub-block of every step).  stage: the unit's 16 rows then its scale arrays;
// act_row / pexs_row: the operand row (activation in operand form, per sub-block constants);
// zeros: 64 zero bytes for the lanes whose operand column belongs to another lane's sub-block.
template <int FMT, int PHASE, int SDT>
__device__ __forceinline__ float2 unit_dot(const uint8_t* stage, const Geo& G, const uint8_t* act_row, const float2* pexs_row,
                                           const uint8_t* zeros, int g, int t, int part, int nparts) {
  constexpr int SUB = Fm<FMT>::SUB, STEP = Fm<FMT>::STEP;
  const int K = G.K[PHASE];
  const int rb = G.row_bytes[PHASE];
  const int full = K / STEP;  // whole steps; one more, partial, when K is not a multiple of STEP
  const int nsub = K / SUB;
  // the steps (the partial one included, which costs as much as a whole one) are cut into `nparts` runs
  const bool has_tail = full * STEP < K;
  const int all = full + (has_tail ? 1 : 0);
  const int c_begin = all * part / nparts, c_end_all = all * (part + 1) / nparts;
  const bool tail = has_tail && c_end_all == all && c_begin < all;  // only the last non-empty run reaches it
  const int c_end = tail ? full : c_end_all;
  // MMA row g is row wr = (g >> 1) + 4 * (g & 1) of its 8-row tile: the two rows a quarter-warp
  // reads in one LDS come from different 4-row halves, which sit `skew` bytes apart modulo 128
  const int wr = (g >> 1) + 4 * (g & 1);
  const int half = 4 * rb + G.skew[PHASE];
  const uint8_t* pa = stage + (g & 1) * half + (g >> 1) * rb + t * 16 + c_begin * 64;
  const uint8_t* pbrow = pa + 2 * half;  // 4 * rb + skew + 4 * rb + skew
  const uint8_t* sc = stage + G.sc_off[PHASE];
  // the lane's operand column g carries its own sub-block only: 2-bit g = 2t (hi), 2t+1 (lo); FP4 g = 2t
  const bool mine = FMT == CACHALOT_BANK_FP4 ? (g == 2 * t) : ((g >> 1) == t);
  const int bstep = mine ? (FMT == CACHALOT_BANK_FP4 ? 256 : 512) : 0;
  const uint8_t* pb = (mine ? act_row + (FMT == CACHALOT_BANK_FP4 ? t * 16 : t * 32 + (g & 1) * 16) : zeros) + c_begin * bstep;
  const float2* ppx = pexs_row + t + c_begin * 4;
  float accA = 0.f, accB = 0.f;

  if constexpr (FMT == CACHALOT_BANK_AFFINE) {
    // scale / bias entries of the two rows at the lane's sub-block of step 0; +2 entries per step
    const uint16_t* S = reinterpret_cast<const uint16_t*>(sc);
    const int arr = G.sc_bytes[PHASE] / 2;
    int ia, ib;
    if constexpr (PHASE == 0) {
      ia = wr * (K >> 7) + (t >> 1);  // rows are whole groups (hidden is a multiple of 128)
      ib = 2 * arr + ia;              // [s1 | b1 | s3 | b3]
    } else {
      ia = (wr * K + t * 64) >> 7;    // groups run over the flattened [16, K] tile
      ib = ((wr + 8) * K + t * 64) >> 7;
    }
    const uint16_t* psA = S + ia + 2 * c_begin;
    const uint16_t* psB = S + ib + 2 * c_begin;
#pragma unroll kUnroll
    for (int c = c_begin; c < c_end; ++c) {
      step_affine<SDT, false>(accA, accB, pa, pbrow, pb, ppx, psA, psB, arr, true);
      pa += 64, pbrow += 64, pb += bstep, ppx += 4, psA += 2, psB += 2;
    }
    if (tail) step_affine<SDT, true>(accA, accB, pa, pbrow, pb, ppx, psA, psB, arr, full * 4 + t < nsub);
  } else {
    const int nblk = K >> 5;  // E8M0 bytes per row: [rows 0..15][K/32]
    const uint8_t* psA = sc + wr * nblk + t + 4 * c_begin;
    const uint8_t* psB = psA + 8 * nblk;
#pragma unroll kUnroll
    for (int c = c_begin; c < c_end; ++c) {
      step_fp4<false>(accA, accB, pa, pbrow, pb, ppx, psA, psB, true);
      pa += 64, pbrow += 64, pb += bstep, ppx += 4, psA += 4, psB += 4;
    }
    if (tail) step_fp4<true>(accA, accB, pa, pbrow, pb, ppx, psA, psB, full * 4 + t < nsub);
  }
  return make_float2(accA, accB);
}

// k rounds of a warp-wide arg-best over the experts' order keys (shared memory).  Lane l keeps experts l, l + 32, ...
// in registers (NE of them); a taken expert's key drops to 0 (below every real one).  Returns the expert of output
// position `lane` (-1: none).
template <int NE>
__device__ __forceinline__ int topk_rounds(const uint32_t* r_ord, int n_experts, int k, bool low_wins, bool ascending, int lane) {
  uint32_t ord[NE];
#pragma unroll
  for (int i = 0; i < NE; ++i) ord[i] = (i * 32 + lane < n_experts) ? r_ord[i * 32 + lane] : 0u;
  int my_e = -1;
  for (int r = 0; r < k; ++r) {
    uint32_t bo = 0u;
    int bi = -1;
#pragma unroll
    for (int i = 0; i < NE; ++i) {
      const bool better = low_wins ? ord[i] > bo : (ord[i] >= bo && ord[i] != 0u);
      if (better) bo = ord[i], bi = i * 32 + lane;
    }
    const uint32_t wo = __reduce_max_sync(0xffffffffu, bo);
    const bool cand = bo == wo && bi >= 0;
    const int win = low_wins ? (int)__reduce_min_sync(0xffffffffu, cand ? (unsigned)bi : 0x7fffffffu)
                             : (int)__reduce_max_sync(0xffffffffu, cand ? (unsigned)(bi + 1) : 0u) - 1;
    if (wo == 0u) break;  // fewer than k experts
#pragma unroll
    for (int i = 0; i < NE; ++i)
      if (i * 32 + lane == win) ord[i] = 0u;
    if (lane == (ascending ? k - 1 - r : r)) my_e = win;
  }
  return my_e;
}

template <int FMT, int SDT, typename OutT>
__global__ void __launch_bounds__(Fm<FMT>::NTHREADS, 1)
fused_decode_kernel(BankView bank, Geo G, RouteArgs R, const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ slots,
                    const float* __restrict__ gate_w, int k, float limit, int numerics, float* __restrict__ hidden,
                    OutT* __restrict__ out, int* __restrict__ status, PeerLink P) {
  constexpr int SUB = Fm<FMT>::SUB, NCW = Fm<FMT>::NCW, NCT = NCW * 32;
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ int s_route[KMAX];   // routing position of the p-th present expert
  __shared__ int s_slot[KMAX];    // its bank slot
  __shared__ float s_gw[KMAX];    // its router weight
  __shared__ int s_np;
  __shared__ unsigned s_tag;
  __shared__ unsigned s_absent;           // routing positions < k whose expert is not in the bank
  __shared__ int s_ta[KMAX], s_tb[KMAX];  // this CTA's inter tiles [ta, tb) of the p-th present expert
  __shared__ int s_n0;                    // its phase-0 units
  uint8_t* ring = smem + G.off_ring;
  uint8_t* act = smem + G.off_act;
  float2* pexs = reinterpret_cast<float2*>(smem + G.off_pe);
  float* ybuf = reinterpret_cast<float*>(smem + G.off_part);  // [tiles of this CTA][KMAX][KP1][16]
  // mbarriers: full / empty per ring stage and phase (the ring is re-cut into smaller stages for phase 1)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + G.off_bar);
  uint64_t* full0 = bars, *empty0 = bars + 16, *full1 = bars + 32, *empty1 = bars + 48;
  const uint8_t* zeros = smem + G.off_bar + 512;  // 512 zero bytes
  float2* xch = reinterpret_cast<float2*>(smem + G.off_bar + 1024);  // [NPAIR][2][8] partial sums between the warps of a pair
  // phase 0 is over in this CTA (x's operand row may be overwritten); the operand rows of group A / B are in place
  uint64_t* p0done = reinterpret_cast<uint64_t*>(smem + G.off_bar + 1536), *op_ready = p0done + 1;
  int* work = reinterpret_cast<int*>(smem + G.off_bar + 1600);  // next chunk of group A / B to convert
  uint8_t* act_x = act + G.x_off;
  float2* pexs_x = pexs + G.xpe_off;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int H = bank.hidden, I = bank.inter;
  int err = 0;
  (void)hidden;  // the hidden rows live in the library image (fused_hidden)
  // Under programmatic dependent launch the next kernel of the stream may be set up while this one runs (it cannot
  // become resident before this CTA leaves: a CTA fills the SM).  Until griddepcontrol.wait returns, only shared
  // memory is touched: the inputs may still be in the making by the previous kernel.  Both are no-ops otherwise.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x < 128) reinterpret_cast<uint32_t*>(smem + G.off_bar + 512)[threadIdx.x] = 0u;
  // one thread per barrier (a single thread would spend most of a microsecond on the 65 of them)
  if (threadIdx.x >= 128 && threadIdx.x < 193) {
    const int i = threadIdx.x - 128;  // bars: full0[16], empty0[16], full1[16], empty1[16]; then p0done
    if (i < 64) {
      mbar_init(&bars[i], i < 16 ? NPROD : i < 32 ? 2 : i < 48 ? 1 : KP1);
    } else {
      mbar_init(p0done, 1);
      work[0] = work[1] = 0;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // number of this exchange: every CTA reads the counter before any CTA can move it on (the last one to finish does)
  const uint32_t xe = P.world > 0 ? *reinterpret_cast<volatile const uint32_t*>(P.epoch) + 1u : 0u;

  // Number of this launch.  A CTA takes a ticket as it reads the number; the CTA with the last ticket moves the number
  // on when it is through - every CTA has read it by then, whatever else happens.  The ticket is asked for here and
  // looked at only at the end, so nobody waits for the atomic's round trip.
  unsigned ticket = 0;
  if (threadIdx.x == 0) {
    unsigned now;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(now) : "l"(&fused_epoch[0]) : "memory");
    s_tag = now;
    ticket = atomicAdd(&fused_epoch[1], 1u);
  }
  // consumers fetch their part of x before anything else (up to XB 16-element blocks per thread)
  constexpr int XB = 3;
  const int tid = threadIdx.x - NPROD * 32;
  uint4 xa[XB], xb[XB];
  if (warp >= NPROD) {
#pragma unroll
    for (int j = 0; j < XB; ++j) {
      const int b = tid + j * NCT;
      xa[j] = xb[j] = make_uint4(0, 0, 0, 0);
      if (b < H / 16) {
        xa[j] = *reinterpret_cast<const uint4*>(x + b * 16);
        xb[j] = *reinterpret_cast<const uint4*>(x + b * 16 + 8);
      }
    }
  }
  // routing inside the kernel: every CTA selects the top-k itself (same arithmetic and tie rules as
  // route_topk_kernel), so no launch and no round trip through global memory sits before the first copy
  uint32_t* r_ord = reinterpret_cast<uint32_t*>(smem + G.off_act);  // scratch in the operand area (x is converted into it later)
  float* r_score = reinterpret_cast<float*>(r_ord + 1024);
  int32_t* r_slot = reinterpret_cast<int32_t*>(r_ord + 2048);
  if (R.logits) {
    for (int e = threadIdx.x; e < R.n_experts; e += blockDim.x) {
      // the three loads are independent: one round trip to L2 for the whole routing tail
      const float raw = R.logits[e];
      const float b = R.bias ? R.bias[e] : 0.f;
      const int32_t sl = R.slot_table ? R.slot_table[(size_t)R.layer * R.n_experts + e] : e;
      float sc, ky;
      router_score_key(R.mode, raw, b, R.gate_temp, sc, ky);
      // "better" as an unsigned order: the sigmoid router prefers the lower key, the other the higher
      const uint32_t u = __float_as_uint(R.mode == CACHALOT_ROUTER_SIGMOID ? -ky : ky);
      r_ord[e] = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
      r_score[e] = sc, r_slot[e] = sl;
    }
    __syncthreads();
  }
  // warp 0: the present experts in routing order
  if (warp == 0) {
    int my_slot = -1;
    float my_w = 0.f;
    if (R.logits) {
      // k rounds of a warp-wide arg-best.  Lane l keeps experts l, l + 32, ... in registers; a taken expert's
      // order drops to 0 (below every real one).  Ties: the sigmoid router prefers the lower index, the other
      // the larger one, as route_topk_kernel does.
      const bool low_wins = R.mode == CACHALOT_ROUTER_SIGMOID;
      const bool ascending = !low_wins;  // the sqrt-softplus router writes the weakest first
      // the rounds are unrolled over the entries a lane keeps: as few as the expert count needs
      int my_e = -1;
      if (R.n_experts <= 128) my_e = topk_rounds<4>(r_ord, R.n_experts, k, low_wins, ascending, lane);
      else if (R.n_experts <= 384) my_e = topk_rounds<12>(r_ord, R.n_experts, k, low_wins, ascending, lane);
      else my_e = topk_rounds<32>(r_ord, R.n_experts, k, low_wins, ascending, lane);
      // lane r holds output position r; the total is added up in output order as route_topk_kernel does
      float total = 0.f;
      for (int r = 0; r < k; ++r) {
        const int e = __shfl_sync(0xffffffffu, my_e, r);
        total += e >= 0 ? r_score[e] : 0.f;
      }
      if (lane < k && my_e >= 0) {
        const float den = total + 1e-20f;
        float w = r_score[my_e];
        if (R.mode == CACHALOT_ROUTER_SIGMOID) {
          w = (w / den) * R.route_scale;
        } else {
          if (R.norm && k > 1) w = w / den;
          w = w * R.route_scale;
        }
        if (R.weights_bf16) w = bf16_round(w);
        my_w = w;
        my_slot = r_slot[my_e];
        if (blockIdx.x == 0) {
          if (R.indices_out) R.indices_out[lane] = my_e;
          if (R.weights_out) R.weights_out[lane] = w;
        }
      }
    } else if (lane < k) {
      my_slot = slots[lane];
      my_w = gate_w[lane];
    }
    const bool present = my_slot >= 0 && my_slot < bank.n_slots;
    const unsigned pmask = __ballot_sync(0xffffffffu, present);
    if (present) {
      const int p = __popc(pmask & ((1u << lane) - 1u));
      s_route[p] = lane, s_slot[p] = my_slot, s_gw[p] = my_w;
    }
    const bool oob = lane < k && my_slot >= bank.n_slots;
    if (__any_sync(0xffffffffu, oob) && lane == 0 && blockIdx.x == 0 && status) atomicOr(status, CACHALOT_STATUS_SLOT_RANGE);
    const bool bad_w = lane < k && !(fabsf(my_w) <= 3.0e38f);  // NaN or infinite
    if (__any_sync(0xffffffffu, bad_w) && lane == 0 && blockIdx.x == 0 && status) atomicOr(status, CACHALOT_STATUS_BAD_WEIGHT);
    // Phase-0 split: unit (routing position r, inter tile) has the number tile * k + r; CTA b takes the numbers
    // [V b / n, V (b+1) / n), V = tiles0 * k - a run of consecutive tiles of every expert, the totals of two CTAs
    // at most one unit apart.  (Numbered by routing position, not by present expert, so an absent expert only
    // leaves holes.)
    const int npres = __popc(pmask);
    int cnt = 0;
    if (present) {
      const unsigned V = (unsigned)G.tiles0 * (unsigned)k;
      const unsigned v0 = V * blockIdx.x / gridDim.x, v1 = V * (blockIdx.x + 1u) / gridDim.x;
      const int ta = (int)((v0 + (unsigned)(k - 1 - lane)) / (unsigned)k), tb = (int)((v1 + (unsigned)(k - 1 - lane)) / (unsigned)k);
      const int p = __popc(pmask & ((1u << lane) - 1u));
      s_ta[p] = ta, s_tb[p] = tb;
      cnt = tb - ta;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    const unsigned absent = __ballot_sync(0xffffffffu, lane < k && !present);
    if (lane == 0) {
      s_np = npres, s_n0 = cnt, s_absent = absent;
      // one arrival per converted chunk of a group's hidden rows (the groups: see below)
      const int b_ = npres >= 3 ? npres / 3 : (npres == 2 ? 1 : 0), a_ = npres - b_;
      const int per_row = hidden_row_words(I) >> 9;
      mbar_init(&op_ready[0], a_ > 0 ? a_ * per_row : 1), mbar_init(&op_ready[1], b_ > 0 ? b_ * per_row : 1);
    }
  }
  __syncthreads();
  const int np = s_np;
  // experts of the two groups: about two thirds, then the rest (6 experts: 4 + 2, so that a CTA with two output tiles
  // has 8 and 4 phase-1 units for its four pairs of MMA warps)
  const int nB = np >= 3 ? np / 3 : (np == 2 ? 1 : 0), nA = np - nB;
  const int t_begin = (int)((unsigned)G.tiles1 * blockIdx.x / gridDim.x), t_end = (int)((unsigned)G.tiles1 * (blockIdx.x + 1u) / gridDim.x);
  const int ntl = t_end - t_begin;                  // phase-1 output tiles of this CTA
  const int n0 = s_n0;                              // phase-0 units of this CTA
  const unsigned tag32 = s_tag;                     // number of this launch
  const unsigned tag8 = tag32 % 255u + 1u;          // marks this launch's hidden values (never 0)
  const int roww = hidden_row_words(I);             // words of a hidden row in fused_hidden
  const int n1 = ntl * np;                          // phase-1 units of this CTA
  const int nst0 = G.nst[0], nst1 = G.nst[1];

  // The operand rows of phase 1 (row p = p-th present expert) are made from the other CTAs' hidden values by whichever
  // warps have time: convert_chunks.  Group A's rows lie clear of x when the operand area is large enough (k rows of
  // inter against one of hidden): then a warp starts on them as soon as its own phase-0 work is done.  Otherwise, and
  // for group B's rows, which overlap x, the end of phase 0 in this CTA is waited for.
  const int row_stride1 = G.act_stride[1], nsub1 = I / SUB;
  const bool early = nA * row_stride1 <= G.x_off && nA * nsub1 <= G.xpe_off;
  auto convert_group = [&](int grp) {
    const int pa = grp ? nA : 0, pn = grp ? nB : nA;
    if (convert_chunks<FMT>(&work[grp], &op_ready[grp], pn * (roww >> 9), I / 16, roww, s_route + pa, act + (size_t)pa * row_stride1,
                            pexs + pa * nsub1, row_stride1, nsub1, tag8, lane))
      err = 2;
  };

  if (warp < NPROD) {
    // ---------------- producers: four rows (and one scale array) of every unit per warp ----------------
    const bool fp4 = FMT == CACHALOT_BANK_FP4;
    const int t_w1 = 0, t_w3 = fp4 ? 4 : 6, t_w2 = fp4 ? 2 : 3;
    const int n_sc = fp4 ? 1 : 2;  // scale arrays per matrix
    if (lane == 0) {
      // phase 0
      {
        const int rb = G.row_bytes[0], sb = G.sc_bytes[0];
        const int tw = warp < 2 ? t_w1 : t_w3;
        const int n_arr = 2 * n_sc;  // arrays in stage order: W1's, then W3's
        // the CTA's units in (present expert, tile) order; experts of which it owns no tile are skipped
        int p = 0, tile = 0, tend = 0;
        while (p < np && (tile = s_ta[p]) >= (tend = s_tb[p])) ++p;
        // One thread issues every copy of its warp, so its scalar code is on the critical path of the stream:
        // stage index and round are counted, nothing is divided inside the loops.
        const uint8_t* rec = p < np ? bank.base + (size_t)s_slot[p] * bank.record_bytes : bank.base;
        const long long off_w = bank.off[tw] + (long long)(warp & 1) * 4 * rb;
        long long off_s = -1;
        if (warp < n_arr) {
          const int m = warp / n_sc, a = warp - m * n_sc;
          off_s = bank.off[(m == 0 ? t_w1 : t_w3) + 1 + a];
        }
        const uint32_t tx = (uint32_t)(4 * rb + (off_s >= 0 ? sb : 0));
        const int dst_w = warp * (4 * rb + G.skew[0]), dst_s = G.sc_off[0] + warp * sb;
        int idx = 0;
        uint32_t round = 0;  // times the ring has wrapped
        for (int i = 0; i < n0 && !err; ++i) {
          if (round > 0 && !mbar_wait(&empty0[idx], (round - 1u) & 1u)) {
            err = 1;  // the consumers stopped releasing stages: give up on the rest of the stream
            break;
          }
          uint8_t* dst = ring + (size_t)idx * G.stage_bytes[0];
          uint64_t* bar = &full0[idx];
          // stage: [W1 rows 0-3 | skew | W1 rows 4-7 | skew | W3 rows 0-3 | skew | W3 rows 4-7 | skew | scale arrays]
          mbar_expect_tx(bar, tx);
          bulk_g2s(dst + dst_w, rec + off_w + (size_t)tile * 8 * rb, (uint32_t)(4 * rb), bar);
          if (off_s >= 0) bulk_g2s(dst + dst_s, rec + off_s + (size_t)tile * sb, (uint32_t)sb, bar);
          if (++tile == tend) {
            ++p;
            while (p < np && (tile = s_ta[p]) >= (tend = s_tb[p])) ++p;
            if (p < np) rec = bank.base + (size_t)s_slot[p] * bank.record_bytes;
          }
          if (++idx == nst0) idx = 0, ++round;
        }
      }
      // phase 1: the ring is cut into nst1 stages of the smaller unit.  Before a stage is first used, the
      // phase-0 stages it overlaps must have been released by their last phase-0 unit.  A unit's 16 rows are contiguous
      // in the bank: copy warp w < NISSUE1 brings the whole of units w, w + NISSUE1, ... (one copy of the rows, one per
      // scale array); the other copy warps go on to the hidden rows at once.
      {
        const int rb = G.row_bytes[1], sb = G.sc_bytes[1];
        const int S0 = G.stage_bytes[0], S1 = G.stage_bytes[1];
        // unit order: group A (tile by tile, its experts inside), then group B the same way
        const int n1a = ntl * nA;
        // phase-0 stage s was used uses(s) = full + (s < rest) times
        const int full = n0 / nst0, rest = n0 - full * nst0;
        const uint32_t tx = (uint32_t)(16 * rb + n_sc * sb);
        int idx = warp % nst1;
        uint32_t round = 0;  // NISSUE1 <= nst1
        int waited = -1;             // phase-0 stages 0..waited are known to be free
        int end_byte = warp * S1;    // end of the previous unit's phase-1 stage inside the ring
        int s_end = 0, s_end_byte = 0;  // first phase-0 stage that starts at or behind end_byte, and its start
        for (int q = warp; warp < NISSUE1 && q < n1 && !err; q += NISSUE1) {
          if (round > 0) {
            if (!mbar_wait(&empty1[idx], (round - 1u) & 1u)) err = 1;
          } else {
            end_byte += S1;
            while (s_end_byte < end_byte) s_end_byte += S0, ++s_end;  // stages waited+1 .. s_end-1 overlap this or an earlier stage
            for (int s0 = waited + 1; s0 < s_end && s0 < nst0 && !err; ++s0) {
              const int uses = full + (s0 < rest ? 1 : 0);
              if (uses > 0 && !mbar_wait(&empty0[s0], (uint32_t)(uses - 1) & 1u)) err = 1;
              waited = s0;
            }
            end_byte += (NISSUE1 - 1) * S1;
          }
          if (err) break;
          const bool in_a = q < n1a;
          const int qq = in_a ? q : q - n1a, pn = in_a ? nA : nB;
          const int tl = qq / pn, p = (in_a ? 0 : nA) + (qq - tl * pn);
          const uint8_t* rec = bank.base + (size_t)s_slot[p] * bank.record_bytes;
          uint8_t* dst = ring + (size_t)idx * S1;
          uint64_t* bar = &full1[idx];
          mbar_expect_tx(bar, tx);
          bulk_g2s(dst, rec + bank.off[t_w2] + (size_t)(t_begin + tl) * 16 * rb, (uint32_t)(16 * rb), bar);
          for (int a = 0; a < n_sc; ++a)
            bulk_g2s(dst + G.sc_off[1] + a * sb, rec + bank.off[t_w2 + 1 + a] + (size_t)(t_begin + tl) * sb, (uint32_t)sb, bar);
          idx += NISSUE1;
          while (idx >= nst1) idx -= nst1, ++round;
        }
      }
      if (err && status) atomicOr(status, CACHALOT_STATUS_WAIT_EXPIRED);
    }
    __syncwarp();
    // All copies are on their way: the copy warps help with the operand rows.  Group B's are theirs alone, converted
    // while the MMA warps work on group A.
    auto wait_phase0 = [&]() {
      if (!mbar_wait_quiet(p0done, 0u, lane)) err = 1;
    };
    if (!early) wait_phase0();
    convert_group(0);
    if (nB > 0) {
      if (early) wait_phase0();
      convert_group(1);
    }
    if (err && lane == 0 && status) atomicOr(status, CACHALOT_STATUS_WAIT_EXPIRED);
    // the launch number moves on once per launch (the next launch reads it after this grid has completed)
    if (threadIdx.x == 0 && ticket == gridDim.x - 1) {
      const unsigned nx = tag32 + 1u;
      fused_epoch[1] = 0u;
      fused_epoch[0] = nx ? nx : 1u;
    }
  } else {
    // ---------------- consumers: pair `pr` takes units pr, pr + NPAIR, ... of the CTA's stream ----------------
    constexpr int NPAIR = Fm<FMT>::NPAIR;
    const int cw = warp - NPROD;
    const int pr = cw >> 1, part = cw & 1;
    const int pair_bar = 2 + pr;  // named barrier of the pair (0 = __syncthreads, 1 = all consumers)
#pragma unroll
    for (int j = 0; j < XB; ++j) {
      const int b = tid + j * NCT;
      if (j * NCT < H / 16) {  // warp-uniform: the lanes of a sub-block convert together
        float v[16];
        unpack16_bf16(xa[j], xb[j], v);
        convert_block<FMT>(act_x, pexs_x, b < H / 16 ? b : 0, b < H / 16, v);
      }
    }
    named_bar_sync(1, NCT);
    // Rows of absent experts are not read in this launch, but their words get this launch's tag all the same (the CTA's
    // share of each): a word's previous tag is then always the previous launch's, never an old one that could recur.
    for (unsigned am = s_absent; am; am &= am - 1u) {
      const int r = __ffs(am) - 1;
      const int lo = (int)((unsigned)roww * blockIdx.x / gridDim.x), hi = (int)((unsigned)roww * (blockIdx.x + 1u) / gridDim.x);
      for (int i = lo + tid; i < hi; i += NCT) st_relaxed_u32(fused_hidden + (size_t)r * roww + i, tag8);
    }
    int n_done = 0;  // units of this pair so far (selects the exchange buffer)

    // -------- phase 0 --------
    // stage index and round of the pair's units are counted (no division per unit)
    int idx = pr % nst0;
    uint32_t rnd = (uint32_t)(pr / nst0);
    // expert and tile of the pair's current unit: the CTA's units in (present expert, tile) order, NPAIR apart
    int pu = 0, tu = 0, te = 0;
    auto skip_units = [&](int n) {
      while (pu < np) {
        if (tu + n < te) {
          tu += n;
          return;
        }
        n -= te - tu;
        ++pu;
        while (pu < np && (tu = s_ta[pu]) >= (te = s_tb[pu])) ++pu;
      }
    };
    while (pu < np && (tu = s_ta[pu]) >= (te = s_tb[pu])) ++pu;
    skip_units(pr);
    for (int i = pr; i < n0; i += NPAIR, ++n_done) {
      if (!err && !mbar_wait(&full0[idx], rnd & 1u)) err = 1;
      float2 r = unit_dot<FMT, 0, SDT>(ring + (size_t)idx * G.stage_bytes[0], G, act_x, pexs_x, zeros, g, t, part, 2);
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty0[idx]);
      r.x += __shfl_xor_sync(0xffffffffu, r.x, 1), r.y += __shfl_xor_sync(0xffffffffu, r.y, 1);
      r.x += __shfl_xor_sync(0xffffffffu, r.x, 2), r.y += __shfl_xor_sync(0xffffffffu, r.y, 2);
      float2* xb2 = xch + (pr * 2 + (n_done & 1)) * 8;
      if (part == 1 && t == 0) xb2[g] = r;
      named_bar_sync(pair_bar, 64);
      if (part == 0 && t == 0) {
        const float2 o = xb2[g];
        const int p = pu, tile = tu;
        float gv = r.x + o.x, uv = r.y + o.y;
        if (numerics != CACHALOT_NUMERICS_F32) gv = bf16_round(gv), uv = bf16_round(uv);
        float h = swiglu(gv, uv, limit) * s_gw[p];
        if (numerics == CACHALOT_NUMERICS_BF16) h = bf16_round(h);
        const size_t hi_ = (size_t)s_route[p] * roww + hidden_word(tile * 8 + (g >> 1) + 4 * (g & 1));
        // the value rounded to nearest at bit 8 (a bf16 value has nothing there), the tag in the low byte
        st_relaxed_u32(fused_hidden + hi_, ((__float_as_uint(h) + 0x80u) & 0xffffff00u) | tag8);
      }
      idx += NPAIR;
      while (idx >= nst0) idx -= nst0, ++rnd;
      skip_units(NPAIR);
    }
    // through with its phase-0 units, a warp helps with group A's operand rows (if they lie clear of x)
    if (early) convert_group(0);
    // every pair is through with x, whose operand row may now be overwritten with hidden rows
    named_bar_sync(1, NCT);
    if (tid == 0) mbar_arrive(p0done);
    if (!early) convert_group(0);

    const int kp = cw % KP1;               // the warp's part of the reduction dimension in phase 1
    constexpr int UPR = NCW / KP1;         // phase-1 units the consumer warps work on at a time
    static_assert(NCW % KP1 == 0, "the consumer warps must split into whole groups of KP1");
    int q_base = 0;                        // phase-1 units of the groups before this one
    for (int gsel = 0; gsel < 2; ++gsel) {
      const int pa = gsel ? nA : 0, pn = gsel ? nB : nA;  // the group's experts: pa .. pa + pn - 1
      if (pn == 0) break;
      // the group's operand rows: group B's are normally done by the copy warps by now (if those are still held up
      // in the ring, the chunks are still there to take)
      if (gsel == 1) convert_group(1);
      if (!err && !mbar_wait_quiet(&op_ready[gsel], 0u, lane)) err = 1;

      // -------- phase 1 of the group: unit u = (tile u / pn, expert pa + u % pn); a warp takes part kp of every
      // UPR-th unit and leaves its partial sums in shared memory --------
      const int n1g = ntl * pn;
      for (int u = cw / KP1; u < n1g; u += UPR) {
        const int q = q_base + u;
        const int sidx = q % nst1;
        const int tl = u / pn, p = pa + (u - tl * pn);
        if (!err && !mbar_wait(&full1[sidx], (uint32_t)(q / nst1) & 1u)) err = 1;
        float2 r = unit_dot<FMT, 1, SDT>(ring + (size_t)sidx * G.stage_bytes[1], G, act + (size_t)p * row_stride1, pexs + p * nsub1, zeros, g, t, kp, KP1);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty1[sidx]);
        r.x += __shfl_xor_sync(0xffffffffu, r.x, 1), r.y += __shfl_xor_sync(0xffffffffu, r.y, 1);
        r.x += __shfl_xor_sync(0xffffffffu, r.x, 2), r.y += __shfl_xor_sync(0xffffffffu, r.y, 2);
        if (t == 0) {
          const int wr = (g >> 1) + 4 * (g & 1);  // the weight row of MMA row g
          float* y = ybuf + (((size_t)tl * KMAX + p) * KP1 + kp) * 16;
          y[wr] = r.x, y[wr + 8] = r.y;
        }
      }
      q_base += n1g;
    }
    named_bar_sync(1, NCT);
    // sum over the experts in routing order; an expert's value is the sum of its KP1 partial sums in part order
    // (rounded to bf16 where the numerics ask for it)
    auto expert_sum = [&](int tl, int r) {
      float tot = 0.f;
      for (int p = 0; p < np; ++p) {
        const float* y = ybuf + ((size_t)tl * KMAX + p) * KP1 * 16 + r;
        float v = y[0];
#pragma unroll
        for (int c = 1; c < KP1; ++c) v += y[c * 16];
        if (numerics != CACHALOT_NUMERICS_F32) v = bf16_round(v);
        tot += v;
      }
      return tot;
    };
    const int n_mine = ntl * 16;
    if (P.world <= 0) {
      for (int o = tid; o < n_mine; o += NCT) {
        const int tl = o >> 4, r = o & 15;
        const float tot = expert_sum(tl, r);
        if constexpr (sizeof(OutT) == 2)
          out[(t_begin + tl) * 16 + r] = __float2bfloat16_rn(tot);
        else
          out[(t_begin + tl) * 16 + r] = tot;
      }
    } else if (n_mine > 0) {
      // Expert parallel: this rank's sum is a partial one.  A thread stores its output value into row `rank` of every
      // rank's inbox as ONE 64-bit word (value, number of this exchange): plain relaxed stores at system scope over
      // NVLink, single-copy atomic, so the word needs no flag and no fence behind it.  It then reads the same element
      // of every rank's row in its own inbox until the word carries this exchange's number (bounded), and adds the
      // values in rank order: no second launch, and every rank ends with the same bits.  Two inbox slots alternate: a
      // rank cannot be two exchanges ahead of a peer, because finishing one takes every peer's values of it.
      const int slot = (int)(xe & 1u), H1 = bank.hidden;
      for (int o = tid; o < n_mine; o += NCT) {
        const float mine = expert_sum(o >> 4, o & 15);
        const size_t el = (size_t)t_begin * 16 + o;
        const unsigned long long word = (unsigned long long)__float_as_uint(mine) | ((unsigned long long)xe << 32);
        const size_t at = ((size_t)slot * P.world + P.rank) * H1 + el;
        for (int q = 0; q < P.world; ++q)
          asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(P.inbox[q] + at), "l"(word) : "memory");
        float tot = 0.f;
        for (int q = 0; q < P.world; ++q) {
          const unsigned long long* src = P.inbox[P.rank] + ((size_t)slot * P.world + q) * H1 + el;
          unsigned long long got = 0ull;
          if (q == P.rank) {
            got = word;
          } else {
            for (uint32_t i = 0;; ++i) {
              asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(got) : "l"(src) : "memory");
              if ((uint32_t)(got >> 32) == xe) break;
              if (i >= (1u << 22)) {  // a peer did not show up: flag it and count its value as zero
                if (status) atomicOr(status, CACHALOT_STATUS_WAIT_EXPIRED);
                got = 0ull;
                break;
              }
              if (i > 64) __nanosleep(64);
            }
          }
          tot += __uint_as_float((uint32_t)got);
        }
        if constexpr (sizeof(OutT) == 2)
          out[t_begin * 16 + o] = __float2bfloat16_rn(tot);
        else
          out[t_begin * 16 + o] = tot;
      }
    }
    if (P.world > 0) {
      // the exchange counter moves on once per launch: by the CTA that takes the last ticket
      named_bar_sync(1, NCT);
      if (tid == 0) {
        const unsigned ticket = atomicAdd(P.epoch + 1, 1u);
        if (ticket == gridDim.x - 1) {
          P.epoch[1] = 0;
          __threadfence();
          P.epoch[0] = xe;
        }
      }
    }
    if (err && lane == 0 && status) atomicOr(status, CACHALOT_STATUS_WAIT_EXPIRED);
  }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

constexpr int MAX_DEVICES = 64;

// SM count of the current device (the grid size); 148 when there is no device to ask
int device_sms() {
  static int cached[MAX_DEVICES] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
    cached[dev] = n;
  }
  return cached[dev];
}

template <int FMT>
bool make_geo_fmt(const BankView& v, int k, int sms, Geo* out) {
  Geo G = {};
  constexpr bool fp4 = FMT == CACHALOT_BANK_FP4;
  constexpr int STEP = Fm<FMT>::STEP, SUB = Fm<FMT>::SUB;
  G.K[0] = v.hidden, G.K[1] = v.inter;
  for (int p = 0; p < 2; ++p) {
    if (G.K[p] % SUB) return false;
    G.nsteps[p] = (G.K[p] + STEP - 1) / STEP;
    G.row_bytes[p] = fp4 ? G.K[p] / 2 : G.K[p] / 4;
  }
  if (!fp4 && v.hidden % 128) return false;  // phase 0 indexes scale groups per row
  if (v.inter % 8 || v.hidden % 16 || v.inter > INTER_MAX) return false;
  if (v.hidden > 16 * 3 * Fm<FMT>::NCW * 32) return false;  // x is staged in at most three 16-element blocks per thread
  G.tiles0 = v.inter / 8, G.tiles1 = v.hidden / 16;
  int n_sc[2];
  if (fp4) {
    G.sc_bytes[0] = 8 * (v.hidden / 32), n_sc[0] = 2;
    G.sc_bytes[1] = 16 * (v.inter / 32), n_sc[1] = 1;
  } else {
    if ((16 * (long long)v.inter) % 128) return false;
    G.sc_bytes[0] = 8 * (v.hidden / 128) * 2, n_sc[0] = 4;
    G.sc_bytes[1] = (16 * v.inter / 128) * 2, n_sc[1] = 2;
  }
  int st[2];
  for (int p = 0; p < 2; ++p) {
    if (G.sc_bytes[p] % 16 || G.row_bytes[p] % 16) return false;
    G.unit_bytes[p] = 16 * G.row_bytes[p] + n_sc[p] * G.sc_bytes[p];
    G.act_stride[p] = G.nsteps[p] * (fp4 ? 256 : 512);
  }
  // phase 0 copies an 8-row tile as two 4-row halves; when a row is a multiple of 128 bytes the second half
  // is shifted by 64 bytes so that the two rows a quarter-warp reads together fall into different banks
  G.skew[0] = G.row_bytes[0] % 128 == 0 ? 64 : 0;
  G.skew[1] = 0;  // one copy for all 16 rows
  for (int p = 0; p < 2; ++p) {
    G.sc_off[p] = 16 * G.row_bytes[p] + 4 * G.skew[p];
    st[p] = G.sc_off[p] + n_sc[p] * G.sc_bytes[p] + 64;  // a partial last step reads up to 48 bytes past a row's end
    G.stage_bytes[p] = (int)align_up((size_t)st[p], 128);
  }
  // operand area: phase 0 one row of hidden, phase 1 k rows of inter
  const int act0 = G.act_stride[0], act1 = k * G.act_stride[1];
  const int act = (int)align_up((size_t)(act0 > act1 ? act0 : act1), 128);
  const int pe0 = (v.hidden / SUB) * 8, pe1 = k * (v.inter / SUB) * 8;
  const int pe = (int)align_up((size_t)(pe0 > pe1 ? pe0 : pe1), 128);
  int p = 0;
  G.off_bar = p, p += 2048;  // mbarriers (512 B), 512 zero bytes, pair exchange buffers
  G.off_act = p, p += act;
  G.off_pe = p, p += pe;
  G.x_off = act - act0, G.xpe_off = (pe - pe0) / 8;
  G.max_tiles = (G.tiles1 + sms - 1) / sms;
  if (G.max_tiles > MAX_TILES) return false;
  G.off_part = p, p += G.max_tiles * KMAX * KP1 * 16 * 4;  // partial sums of the CTA's output tiles per expert and part
  G.off_ring = p;
  const int room = SMEM_LIMIT - 256 /* static shared */ - p;
  for (int ph = 0; ph < 2; ++ph) {
    G.nst[ph] = room / G.stage_bytes[ph];
    if (G.nst[ph] > 16) G.nst[ph] = 16;
  }
  // a pair holds a stage while it works on it; at least one more must be in flight
  if (G.nst[0] < Fm<FMT>::NPAIR + 1 || G.nst[1] < Fm<FMT>::NPAIR + 1) return false;
  const int r0 = G.nst[0] * G.stage_bytes[0], r1 = G.nst[1] * G.stage_bytes[1];
  G.total = p + (r0 > r1 ? r0 : r1);
  *out = G;
  return true;
}

bool make_geo(const BankView& v, int k, Geo* out) {
  const int sms = device_sms();
  return v.format == CACHALOT_BANK_FP4 ? make_geo_fmt<CACHALOT_BANK_FP4>(v, k, sms, out) : make_geo_fmt<CACHALOT_BANK_AFFINE>(v, k, sms, out);
}

}  // namespace

bool decode_fused_supported(const BankView& v, int rows, int k) {
  if (rows != 1 || k < 1 || k > KMAX) return false;
  if (v.format == CACHALOT_BANK_AFFINE && (v.group != 128 || v.bits != 2)) return false;
  Geo G;
  return make_geo(v, k, &G);
}

// hidden [k, inter] f32
size_t decode_fused_workspace_bytes(int hidden, int inter, int rows, int k) {
  (void)hidden;
  return align_up((size_t)rows * k * inter * sizeof(float), 256);
}

template <int FMT>
static int launch_fused_fmt(const BankView& v, const Geo& G, const RouteArgs& R, const void* x, const int32_t* slots,
                            const float* gate_w, int k, float limit, int numerics, void* workspace, void* out, int out_dtype,
                            int* status, cudaStream_t stream, const PeerLink* peer = nullptr) {
  PeerLink P = {};
  if (peer) P = *peer;
  float* hidden = static_cast<float*>(workspace);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return fail(CACHALOT_ECUDA, "moe_decode (fused): no current device");
  const int sms = device_sms();
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
  const Geo& Gl = G;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)sms);
  cfg.blockDim = dim3(Fm<FMT>::NTHREADS);
  // Always the whole shared memory of an SM, also for small banks: one CTA per SM, so a second launch (from
  // another stream) cannot become resident, and cannot touch the hidden rows or the launch counter, before this
  // launch's CTAs have left.
  cfg.dynamicSmemBytes = (size_t)(SMEM_LIMIT - 256);
  (void)G.total;
  cfg.stream = stream;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident: they read each other's hidden values
  at[0].val.cooperative = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;  // the prologue may overlap the previous kernel's tail
  at[1].val.programmaticStreamSerializationAllowed = 1;
  // on unless CACHALOT_PDL=0 is set (the switch exists to time the difference: about 0.9 us per layer)
  static const bool pdl = [] { const char* e = std::getenv("CACHALOT_PDL"); return !(e && e[0] == '0'); }();
  cfg.attrs = at;
  cfg.numAttrs = pdl ? 2 : 1;
  cudaError_t e = cudaSuccess;
  auto go = [&](auto kern, auto* outp) {
    // the opt-in is an attribute of a kernel on a device: set once for each (the pointer types of different
    // instantiations coincide, so the record is keyed by the pointer)
    static std::mutex mu;
    static std::set<std::pair<const void*, int>> done;
    {
      std::lock_guard<std::mutex> lock(mu);
      if (!done.count({(const void*)kern, dev})) {
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_LIMIT - 256);
        if (e != cudaSuccess) return;
        done.insert({(const void*)kern, dev});
      }
    }
    e = cudaLaunchKernelEx(&cfg, kern, v, Gl, R, xb, slots, gate_w, k, limit, numerics, hidden, outp, status, P);
  };
  const bool bf16_scales = FMT == CACHALOT_BANK_AFFINE && v.scale_dtype == CACHALOT_BF16;
  if (out_dtype == CACHALOT_BF16) {
    if (bf16_scales) go(fused_decode_kernel<FMT, CACHALOT_BF16, __nv_bfloat16>, (__nv_bfloat16*)out);
    else go(fused_decode_kernel<FMT, CACHALOT_F16, __nv_bfloat16>, (__nv_bfloat16*)out);
  } else {
    if (bf16_scales) go(fused_decode_kernel<FMT, CACHALOT_BF16, float>, (float*)out);
    else go(fused_decode_kernel<FMT, CACHALOT_F16, float>, (float*)out);
  }
  if (e != cudaSuccess) return fail(CACHALOT_ECUDA, "moe_decode (fused): %s", cudaGetErrorString(e));
  return check_launch("moe_decode (fused)");
}

int launch_decode_fused(const BankView& v, const void* x, const int32_t* slots, const float* gate_w, int rows, int k,
                        float limit, int numerics_flags, void* workspace, void* out, int out_dtype, int* status,
                        cudaStream_t stream) {
  Geo G;
  if (rows != 1 || !make_geo(v, k, &G)) return CACHALOT_EUNSUPPORTED;
  const int numerics = numerics_flags & 0xff;
  const RouteArgs R = {};
  if (v.format == CACHALOT_BANK_FP4)
    return launch_fused_fmt<CACHALOT_BANK_FP4>(v, G, R, x, slots, gate_w, k, limit, numerics, workspace, out, out_dtype, status, stream);
  return launch_fused_fmt<CACHALOT_BANK_AFFINE>(v, G, R, x, slots, gate_w, k, limit, numerics, workspace, out, out_dtype, status, stream);
}

// The same launch with the routing tail inside: logits -> top-k -> slots, then the experts.
int launch_layer_fused(const BankView& v, const void* x, const float* logits, const float* bias, const int32_t* slot_table,
                       int layer, int n_experts, int k, int mode, float gate_temp, float route_scale, int norm,
                       int weights_bf16, float limit, int numerics_flags, void* workspace, void* out, int out_dtype,
                       int32_t* indices_out, float* weights_out, int* status, cudaStream_t stream, const PeerLink* peer) {
  Geo G;
  if (!make_geo(v, k, &G) || n_experts > 1024) return CACHALOT_EUNSUPPORTED;
  if (G.x_off + G.act_stride[0] < 12288) return CACHALOT_EUNSUPPORTED;  // the routing scratch (12 KB) borrows the operand area
  const int numerics = numerics_flags & 0xff;
  RouteArgs R = {};
  R.logits = logits, R.bias = bias, R.slot_table = slot_table, R.indices_out = indices_out, R.weights_out = weights_out;
  R.layer = layer, R.n_experts = n_experts, R.mode = mode, R.norm = norm, R.weights_bf16 = weights_bf16;
  R.gate_temp = gate_temp, R.route_scale = route_scale;
  if (v.format == CACHALOT_BANK_FP4)
    return launch_fused_fmt<CACHALOT_BANK_FP4>(v, G, R, x, nullptr, nullptr, k, limit, numerics, workspace, out, out_dtype, status, stream, peer);
  return launch_fused_fmt<CACHALOT_BANK_AFFINE>(v, G, R, x, nullptr, nullptr, k, limit, numerics, workspace, out, out_dtype, status, stream, peer);
}

bool layer_fused_supported(const BankView& v, int n_experts, int k) {
  Geo G;
  if (k < 1 || k > KMAX || n_experts < k || n_experts > 1024) return false;
  if (v.format == CACHALOT_BANK_AFFINE && (v.group != 128 || v.bits != 2)) return false;
  return make_geo(v, k, &G) && G.x_off + G.act_stride[0] >= 12288;
}

}  // namespace cachalot

