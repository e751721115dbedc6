// Prefill routed experts on the block-scaled FP4 tensor cores (tcgen05.mma kind::mxf4, E8M0 scale per 32).
//
// Rows are already grouped by expert (perm, offsets).  Two grouped GEMMs run per call, both with the
// weights as the M side of the MMA so that an expert with few rows wastes no tensor-core work:
//
//   gate/up : D_g, D_u [128 weight rows, <=96 routed rows] = W1/W3 tile . X^T      K = hidden
//             epilogue  h = silu(min(g,L)) * clip(u) * row weight  -> MXFP4 per 32 along the weight-row axis
//   down    : D   [128 weight rows, <=96 routed rows]        = W2 tile . H^T        K = inter
//             epilogue  y -> bf16, stored per routed row; a last kernel adds a token's k rows in slot order
//
// Work item = (unit, weight-row tile); a unit is up to 96 consecutive routed rows of one expert.  CTAs are
// persistent and take items round-robin, unit-major, so the CTAs that run together read different tiles of
// the same expert and share its activation rows in L2.
//
// Warp roles (448 threads): warp 0 issues the TMA tile loads (weights straight out of the bank through a
// 3-D tensor map {K bytes, rows, slot}; activations through a 2-D map), warp 1 owns TMEM and issues
// tcgen05.cp (scales, shared -> TMEM) and tcgen05.mma, warps 2-5 bring the E8M0 scale bytes of the stage
// from the bank's row-major arrays into the 32x16-byte pattern tcgen05.cp wants, warps 6-13 drain the
// accumulators (tcgen05.ld) while the next item's MMAs fill the other accumulator buffer.
//
// Every wait is bounded: when one gives up the CTA raises CACHALOT_STATUS_WAIT_EXPIRED, all roles leave
// their loops, TMEM is released and the kernel returns.
#include <cuda.h>

#include "kernels.cuh"

namespace cachalot {
namespace {

constexpr int BM = 128;          // weight rows per tile (MMA M)
constexpr int NTMAX = 96;        // routed rows per unit (MMA N <= 96, multiple of 16)
constexpr int BKB = 128;         // bytes of K per stage and row = 256 codes = 8 scale blocks = 4 MMAs of K=64
constexpr int A_TILE = BM * BKB;
constexpr int B_TILE = NTMAX * BKB;
constexpr int SF_TILE = 1024;    // 128 rows x 8 scale bytes, as two 512-byte groups of four blocks
constexpr int NTHREADS = 448;
constexpr int TMEM_COLS = 512;
constexpr int SF_COL = 2 * 2 * NTMAX;  // scale columns start behind the (up to) four accumulators
constexpr uint32_t WAIT_LIMIT = 1u << 20;


struct Unit {
  int32_t slot, row_start, ntok, pad;
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
// false when the wait gave up (it sets *abort) or another role already had
__device__ __forceinline__ bool mbar_wait(uint64_t* b, uint32_t parity, volatile int* abort) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try(b, parity)) return true;
    if ((i & 63u) == 63u && *abort) return false;
  }
  *abort = 1;
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::
          "r"(smem_u32(dst)),
      "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar,
                                            uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], "
      "%6;" ::"r"(smem_u32(dst)),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// contiguous bytes -> shared memory (both 16-byte aligned, size a multiple of 16), completion on an mbarrier
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src),
               "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// pulls one weight tile into L2 ahead of its load
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* map, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(map), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// shared-memory matrix descriptors (address and offsets in 16-byte units, descriptor version 1)
// operand tile: rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// scale group: 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes apart
__device__ __forceinline__ uint64_t desc_sf(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (8ull << 32) | (1ull << 46);
}
// instruction descriptor of kind::mxf4: E2M1 x E2M1, both K-major, E8M0 scales, M = 128, N = n
__device__ __forceinline__ uint32_t idesc_mxf4(int n) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tacc, uint64_t da, uint64_t db, uint32_t idesc, uint32_t tsfa, uint32_t tsfb,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4.block_scale.scale_vec::2X [%0], %1, %2, %3, [%5], [%6], p;\n}" ::"r"(tacc),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

struct GemmArgs {
  const uint8_t* bank;        // slot records
  long long record_bytes;
  long long off_sc[2];        // offsets of the weight matrices' scale arrays inside a record
  const uint8_t* act_scales;  // u8 [rows, K/32]
  const Unit* units;
  const int32_t* n_units;
  int n_rows;                 // weight rows N
  int k_codes;                // K
  int total_rows;             // routed rows R
  // gate/up epilogue
  const float* row_w;         // f32 [R] router weight of every grouped row
  float limit;
  uint8_t* h_codes;           // u8 [R, N/2]
  uint8_t* h_scales;          // u8 [R, N/32]
  // down epilogue
  __nv_bfloat16* y;           // bf16 [R, N]
  float* y32;                 // TERMS > 1: f32 [R / TERMS, N], one row per routed row
  int round_bf16;             // TERMS > 1: the reference's prefill rounding points (g, u, h and y rounded to bf16)
  int* status;
};

// Sixteen scale bytes of one row (one stage: two pieces of eight 32-blocks) starting at block kb0, for any
// even row pitch: one or two aligned 16-byte loads and a byte shift.  Blocks past the row's end read as 2**0
// (their codes are zero-filled), and no byte past the row's end is touched.
__device__ __forceinline__ uint4 load_sf16(const uint8_t* row, int kb0, int nkb, bool valid) {
  uint4 r = make_uint4(0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
  const int have = min(16, nkb - kb0);  // bytes of this stage that exist
  if (!valid || have <= 0) return r;
  const uintptr_t a = reinterpret_cast<uintptr_t>(row + kb0);
  const uint4* q = reinterpret_cast<const uint4*>(a & ~(uintptr_t)15);
  const int off = (int)(a & 15);
  const uint4 lo = __ldg(q);
  if (off == 0) {
    r = lo;
  } else {
    uint4 hi = make_uint4(0, 0, 0, 0);
    if (off + have > 16) hi = __ldg(q + 1);
    const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    const int ws = off >> 2, bs = (off & 3) * 8;
#pragma unroll
    for (int t = 0; t < 4; ++t)
      if (ws == t) {
        r.x = __funnelshift_r(w[t], w[t + 1], bs);
        r.y = __funnelshift_r(w[t + 1], w[t + 2], bs);
        r.z = __funnelshift_r(w[t + 2], w[t + 3], bs);
        r.w = __funnelshift_r(w[t + 3], w[t + 4], bs);
      }
  }
  if (have < 16) {
    uint32_t* v = &r.x;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int n = have - 4 * i;  // valid bytes of word i
      const uint32_t keep = n >= 4 ? 0xFFFFFFFFu : n <= 0 ? 0u : (1u << (8 * n)) - 1u;
      v[i] = (v[i] & keep) | (0x7F7F7F7Fu & ~keep);
    }
  }
  return r;
}

// NA = 2: gate and up tiles with the SwiGLU + MXFP4 epilogue; NA = 1: down tile with the bf16 store epilogue.
// A stage holds KSUB consecutive 128-byte pieces of every row (one swizzled tile each), so that a row's bytes
// of a stage are asked from DRAM back to back.
// RAW: the scale bytes of an item (contiguous in the bank: 128 rows of K/32 bytes per matrix, and the unit's
// rows of the activation scales) are bulk-copied into shared memory one item ahead and the loader warps read
// them from there; otherwise the loader warps read their rows from global memory (one row per lane).
// TERMS = 1: prefill numerics (activations are MXFP4 by definition; g, u rounded to bf16; outputs bf16).
// TERMS = 4: decode numerics.  Every routed row arrives as four consecutive MXFP4 rows whose sum is the row to
// within 6**-4 of its block maxima (each row quantises what the rows before it left over, with its own block
// scales), so the MMAs see the bf16 / fp32 activation almost exactly; the drain adds the four columns, keeps fp32
// throughout and writes the hidden activation as four residual rows again, the output as one fp32 row.
template <int NA, int NSTAGE, int KSUB, bool RAW, int TERMS = 1>
__global__ void __launch_bounds__(NTHREADS, 1)
grouped_mxf4_kernel(const __grid_constant__ CUtensorMap map_a0, const __grid_constant__ CUtensorMap map_a1,
                    const __grid_constant__ CUtensorMap map_b, GemmArgs A) {
  constexpr int STAGE_BYTES = KSUB * (NA * A_TILE + B_TILE + (NA + 1) * SF_TILE);
  constexpr int OFF_B = KSUB * NA * A_TILE, OFF_SF = OFF_B + KSUB * B_TILE;
  constexpr int ACC_COLS = NA * NTMAX;  // per accumulator buffer
  static_assert(SF_COL + (NA + 1) * KSUB * 8 <= TMEM_COLS, "scale columns do not fit");
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)NSTAGE * STAGE_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + NSTAGE;
  uint64_t* acc_full = bars + 2 * NSTAGE;
  uint64_t* acc_empty = bars + 2 * NSTAGE + 2;
  uint64_t* raw_full = bars + 2 * NSTAGE + 4;
  uint64_t* raw_empty = bars + 2 * NSTAGE + 6;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * NSTAGE + 8);
  volatile int* abort = reinterpret_cast<volatile int*>(tmem_holder + 1);
  uint8_t* raw_base = smem + (size_t)NSTAGE * STAGE_BYTES + 256;  // two slots of raw scale bytes behind the barriers

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) mbar_init(&full[s], 5), mbar_init(&empty[s], 1);
    for (int b = 0; b < 2; ++b) mbar_init(&acc_full[b], 1), mbar_init(&acc_empty[b], 8);
    for (int b = 0; b < 2; ++b) mbar_init(&raw_full[b], 1), mbar_init(&raw_empty[b], 4);
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_holder;

  const int n_units = *A.n_units;
  const int n_mt = (A.n_rows + BM - 1) / BM;
  const long long total = (long long)n_units * n_mt;
  const int k_bytes = A.k_codes / 2, nkb = A.k_codes / 32;
  const int nks = (k_bytes + KSUB * BKB - 1) / (KSUB * BKB);
  // raw scale slot: NA blocks of 128 rows, then the unit's activation rows (with up to 15 bytes of lead-in)
  const int raw_a = (BM * nkb + 15) & ~15, raw_b = (NTMAX * nkb + 15 + 15) & ~15;
  const int raw_slot = NA * raw_a + raw_b;

  if (warp == 0) {
    // ---- tile loads ------------------------------------------------------------------------
    if (lane == 0) {
      // weights are read once: first out of L2; activation rows are re-read by every tile of the expert
      uint64_t pol_w, pol_x;
      asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol_w));
      asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol_x));
      int s = 0;
      uint32_t ph = 0;
      bool wrapped = false, ok = true;
      // The shared-memory ring is only two or three stages deep, less than the HBM latency under load, so the
      // weight tiles of the next PFD stages are asked into L2 ahead of their loads (2 measured best of 0/2/4/8).
      constexpr int PFD = 2;
      long long pw = blockIdx.x;  // prefetch cursor (item, stage); the item's slot and row are looked up once per item
      int pks = 0, p_slot = 0, p_row = 0;
      auto prefetch_next = [&]() {
        if (pw >= total) return;
        if (pks == 0) {
          p_slot = A.units[pw / n_mt].slot;
          p_row = (int)(pw % n_mt) * BM;
        }
#pragma unroll
        for (int j = 0; j < KSUB; ++j) {
          const int kx = (pks * KSUB + j) * BKB;
          if (kx >= k_bytes) break;
          tma_prefetch_3d(&map_a0, kx, p_row, p_slot);
          if (NA == 2) tma_prefetch_3d(&map_a1, kx, p_row, p_slot);
        }
        if (++pks == nks) pks = 0, pw += gridDim.x;
      };
      for (int i = 0; i < PFD; ++i) prefetch_next();
      // raw scale bytes of item number `no` (work item wi) into slot no & 1
      auto raw_copy = [&](long long wi, long long no) -> bool {
        const int slot = (int)(no & 1);
        if (no >= 2 && !mbar_wait(&raw_empty[slot], (uint32_t)((no >> 1) - 1) & 1u, abort)) return false;
        const Unit u = A.units[wi / n_mt];
        const int mt = (int)(wi % n_mt);
        const int rows_a = min(BM, A.n_rows - mt * BM);
        const uint32_t bytes_a = (uint32_t)(rows_a * nkb + 15) & ~15u;
        const uint8_t* sb = A.act_scales + (size_t)u.row_start * nkb;
        const uint32_t lead = (uint32_t)(reinterpret_cast<uintptr_t>(sb) & 15);
        const uint32_t bytes_b = (lead + (uint32_t)(u.ntok * nkb) + 15) & ~15u;
        uint8_t* dst = raw_base + (size_t)slot * raw_slot;
        const uint8_t* rec = A.bank + (size_t)u.slot * A.record_bytes;
        mbar_expect_tx(&raw_full[slot], NA * bytes_a + bytes_b);
        bulk_load(dst, rec + A.off_sc[0] + (size_t)mt * BM * nkb, bytes_a, &raw_full[slot]);
        if (NA == 2) bulk_load(dst + raw_a, rec + A.off_sc[1] + (size_t)mt * BM * nkb, bytes_a, &raw_full[slot]);
        bulk_load(dst + NA * raw_a, sb - lead, bytes_b, &raw_full[slot]);
        return true;
      };
      long long item_no = 0;
      if (RAW && total > blockIdx.x) ok = raw_copy(blockIdx.x, 0);
      for (long long w = blockIdx.x; w < total && ok; w += gridDim.x, ++item_no) {
        const Unit u = A.units[w / n_mt];
        const int mt = (int)(w % n_mt);
        if (RAW && w + gridDim.x < total && !raw_copy(w + gridDim.x, item_no + 1)) { ok = false; break; }
        for (int ks = 0; ks < nks; ++ks) {
          if (wrapped && !mbar_wait(&empty[s], ph ^ 1u, abort)) { ok = false; break; }
          uint8_t* st = smem + (size_t)s * STAGE_BYTES;
          mbar_expect_tx(&full[s], KSUB * (NA * A_TILE + B_TILE));
#pragma unroll
          for (int j = 0; j < KSUB; ++j) {
            const int kx = (ks * KSUB + j) * BKB;
            tma_load_3d(st + j * A_TILE, &map_a0, kx, mt * BM, u.slot, &full[s], pol_w);
            if (NA == 2) tma_load_3d(st + (KSUB + j) * A_TILE, &map_a1, kx, mt * BM, u.slot, &full[s], pol_w);
          }
#pragma unroll
          for (int j = 0; j < KSUB; ++j) tma_load_2d(st + OFF_B + j * B_TILE, &map_b, (ks * KSUB + j) * BKB, u.row_start, &full[s], pol_x);
          if (++s == NSTAGE) s = 0, ph ^= 1u, wrapped = true;
          prefetch_next();
        }
      }
    }
  } else if (warp == 1) {
    // ---- scale copies into TMEM and the MMAs -------------------------------------------------
    // One thread issues everything, so its own instruction count is on the critical path: all descriptors are
    // the stage's base descriptor plus a compile-time constant (addresses are in 16-byte units in the low bits).
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      long long item = 0;
      bool ok = true;
      const uint64_t d_op0 = desc_sw128(smem_u32(smem));
      const uint64_t d_sf0 = desc_sf(smem_u32(smem) + OFF_SF);
      const uint32_t t_sf = tmem + SF_COL;
      for (long long w = blockIdx.x; w < total && ok; w += gridDim.x, ++item) {
        const Unit u = A.units[w / n_mt];
        const int buf = (int)(item & 1);
        const uint32_t id0 = idesc_mxf4((u.ntok + 15) & ~15);
        const uint32_t id2 = id0 | (2u << 29) | (2u << 4);  // scale bytes 2,3 of the column for the second K=64 of a pair
        const uint32_t t_acc = tmem + buf * ACC_COLS;
        uint32_t accumulate = 0;
        if (item >= 2 && !mbar_wait(&acc_empty[buf], (uint32_t)((item >> 1) - 1) & 1u, abort)) { ok = false; break; }
        tc_fence_after();
        for (int ks = 0; ks < nks; ++ks) {
          if (!mbar_wait(&full[s], ph, abort)) { ok = false; break; }
          tc_fence_after();
          const uint64_t so = (uint64_t)((uint32_t)(s * STAGE_BYTES) >> 4);
          const uint64_t dop = d_op0 + so, dsf = d_sf0 + so;
#pragma unroll
          for (int j = 0; j < KSUB; ++j) {
            if ((ks * KSUB + j) * BKB >= k_bytes) break;  // piece wholly behind the end of K: zeros, nothing to add
#pragma unroll
            for (int m = 0; m < NA + 1; ++m)
#pragma unroll
              for (int q = 0; q < 2; ++q)
                tc_cp_sf(t_sf + (m * KSUB + j) * 8 + q * 4, dsf + (uint64_t)(((m * KSUB + j) * SF_TILE + q * 512) >> 4));
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              // the allocation's lane field is zero, so adding the byte selector into bits 30-31 equals OR-ing it
              const uint32_t sel = (uint32_t)(kk & 1) << 31, q = (uint32_t)kk >> 1;
              const uint64_t db = dop + (uint64_t)((OFF_B + j * B_TILE + kk * 32) >> 4);
              const uint32_t tsfb = t_sf + (((NA * KSUB + j) * 8 + q * 4) | sel);
#pragma unroll
              for (int m = 0; m < NA; ++m) {
                const uint64_t da = dop + (uint64_t)(((m * KSUB + j) * A_TILE + kk * 32) >> 4);
                const uint32_t tsfa = t_sf + (((m * KSUB + j) * 8 + q * 4) | sel);
                tc_mma(t_acc + m * NTMAX, da, db, (kk & 1) ? id2 : id0, tsfa, tsfb, accumulate);
              }
              accumulate = 1;
            }
          }
          tc_commit(&empty[s]);
          if (++s == NSTAGE) s = 0, ph ^= 1u;
        }
        if (ok) tc_commit(&acc_full[buf]);
      }
    }
  } else if (warp < 6) {
    // ---- scale bytes: bank rows -> the stage's 32x16-byte groups --------------------------------
    // One flat walk over (item, stage) with the next stage's bytes already on their way, also across items;
    // the rows of the item after this one are pulled into L2 at the start of every item.
    const int m = (warp - 2) * 32 + lane;  // row of the tile
    const uint32_t sf_off = (uint32_t)((m & 31) * 16 + (m >> 5) * 4);
    const uint8_t *ra0 = nullptr, *ra1 = nullptr, *rb = nullptr;
    bool va = false, vb = false;
    auto point_at = [&](long long w) {
      const Unit u = A.units[w / n_mt];
      const int row_a = (int)(w % n_mt) * BM + m;
      va = row_a < A.n_rows;
      const uint8_t* rec = A.bank + (size_t)u.slot * A.record_bytes;
      ra0 = rec + A.off_sc[0] + (size_t)row_a * nkb;
      ra1 = rec + A.off_sc[NA - 1] + (size_t)row_a * nkb;
      vb = m < u.ntok;
      rb = A.act_scales + (size_t)(u.row_start + m) * nkb;
    };
    auto pull = [&](const uint8_t* p) {
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(p + nkb - 1));
    };
    auto pull_item = [&](long long w) {
      const Unit u = A.units[w / n_mt];
      const int row_a = (int)(w % n_mt) * BM + m;
      const uint8_t* rec = A.bank + (size_t)u.slot * A.record_bytes;
      if (row_a < A.n_rows) {
        pull(rec + A.off_sc[0] + (size_t)row_a * nkb);
        if (NA == 2) pull(rec + A.off_sc[1] + (size_t)row_a * nkb);
      }
      if (m < u.ntok) pull(A.act_scales + (size_t)(u.row_start + m) * nkb);
    };
    static_assert(KSUB == 2, "the scale loaders fetch sixteen bytes = two pieces per stage");
    // Three register sets in rotation: the bytes of stage i+2 are asked for before stage i is written, so a
    // load has two stage times to arrive.
    uint4 set_a[NA + 1], set_b[NA + 1], set_c[NA + 1];
    const long long n_mine = total > blockIdx.x ? (total - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    const long long n_stage = n_mine * nks;
    long long wf = blockIdx.x, fetched = 0;  // fetch cursor: item and stage count
    int ksf = 0;
    // RAW: sixteen bytes of the row at byte offset `at` of the slot (2-byte aligned), blocks past nkb as 2**0
    auto raw16 = [&](const uint8_t* base, int kb0, bool valid) -> uint4 {
      uint4 r = make_uint4(0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
      if (!valid) return r;
      const uint16_t* p = reinterpret_cast<const uint16_t*>(base + kb0);
      uint32_t* v = &r.x;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int n = nkb - kb0 - 4 * i;  // blocks left for word i
        if (n >= 4) v[i] = (uint32_t)p[2 * i] | ((uint32_t)p[2 * i + 1] << 16);
        else if (n > 0) {
          const uint32_t lo = p[2 * i], hi = n > 2 ? p[2 * i + 1] : 0u;
          const uint32_t keep = (1u << (8 * n)) - 1u;
          v[i] = ((lo | (hi << 16)) & keep) | (0x7F7F7F7Fu & ~keep);
        }
      }
      return r;
    };
    long long items_seen = 0;        // items whose raw bytes this warp has started to read
    const uint8_t* raw_slot_ptr = nullptr;
    uint32_t raw_lead = 0;
    bool raw_ok = true;
    auto fetch = [&](uint4 (&d)[NA + 1]) {
      if (fetched >= n_stage) return;
      if (RAW) {
        if (ksf == 0) {
          const Unit u = A.units[wf / n_mt];
          va = (int)(wf % n_mt) * BM + m < A.n_rows;
          vb = m < u.ntok;
          raw_lead = (uint32_t)(reinterpret_cast<uintptr_t>(A.act_scales + (size_t)u.row_start * nkb) & 15);
          const int slot = (int)(items_seen & 1);
          raw_slot_ptr = raw_base + (size_t)slot * raw_slot;
          if (!__all_sync(0xffffffffu, mbar_wait(&raw_full[slot], (uint32_t)(items_seen >> 1) & 1u, abort))) raw_ok = false;
          ++items_seen;
        }
        if (raw_ok) {
          d[0] = raw16(raw_slot_ptr + (size_t)m * nkb, ksf * 16, va);
          if (NA == 2) d[1] = raw16(raw_slot_ptr + raw_a + (size_t)m * nkb, ksf * 16, va);
          d[NA] = raw16(raw_slot_ptr + NA * raw_a + raw_lead + (size_t)m * nkb, ksf * 16, vb);
        }
        ++fetched;
        if (++ksf == nks) {
          ksf = 0, wf += gridDim.x;
          __syncwarp();
          if (lane == 0) mbar_arrive(&raw_empty[(items_seen - 1) & 1]);  // this warp is done with the slot
        }
        return;
      }
      if (ksf == 0) {
        point_at(wf);
        if (wf + gridDim.x < total) pull_item(wf + gridDim.x);
      }
      d[0] = load_sf16(ra0, ksf * 16, nkb, va);
      if (NA == 2) d[1] = load_sf16(ra1, ksf * 16, nkb, va);
      d[NA] = load_sf16(rb, ksf * 16, nkb, vb);
      ++fetched;
      if (++ksf == nks) ksf = 0, wf += gridDim.x;
    };
    int s = 0;
    uint32_t ph = 0;
    bool wrapped = false;
    // writes one stage from `cur` after asking for the stage two ahead into `far`; false when a wait gave up
    auto step = [&](uint4 (&cur)[NA + 1], uint4 (&far)[NA + 1]) -> bool {
      fetch(far);
      if (RAW && !raw_ok) return false;
      if (wrapped && !__all_sync(0xffffffffu, mbar_wait(&empty[s], ph ^ 1u, abort))) return false;
      uint8_t* sf = smem + (size_t)s * STAGE_BYTES + OFF_SF;
#pragma unroll
      for (int mm = 0; mm < NA + 1; ++mm) {
        *reinterpret_cast<uint32_t*>(sf + (mm * 2) * SF_TILE + sf_off) = cur[mm].x;
        *reinterpret_cast<uint32_t*>(sf + (mm * 2) * SF_TILE + 512 + sf_off) = cur[mm].y;
        *reinterpret_cast<uint32_t*>(sf + (mm * 2 + 1) * SF_TILE + sf_off) = cur[mm].z;
        *reinterpret_cast<uint32_t*>(sf + (mm * 2 + 1) * SF_TILE + 512 + sf_off) = cur[mm].w;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&full[s]);
      if (++s == NSTAGE) s = 0, ph ^= 1u, wrapped = true;
      return true;
    };
    fetch(set_a);
    fetch(set_b);
    for (long long i = 0; i < n_stage; i += 3) {
      if (!step(set_a, set_c)) break;
      if (i + 1 < n_stage && !step(set_b, set_a)) break;
      if (i + 2 < n_stage && !step(set_c, set_b)) break;
    }
    if (warp == 2 && lane == 0) {
    }
  } else {
    // ---- accumulators -> results ----------------------------------------------------------------
    // eight warps: two per TMEM lane quarter, taking alternate 16-column chunks
    const int q = warp & 3;  // TMEM lanes 32q .. 32q+31 belong to this warp
    const int half = (warp - 6) >> 2;
    const uint32_t lane_base = tmem + ((uint32_t)(q * 32) << 16);
    long long item = 0;
    bool ok = true;
    for (long long w = blockIdx.x; w < total && ok; w += gridDim.x, ++item) {
      const Unit u = A.units[w / n_mt];
      const int mt = (int)(w % n_mt);
      const int buf = (int)(item & 1);
      const int n = mt * BM + q * 32 + lane;           // weight row = output index
      const bool rows_ok = mt * BM + q * 32 < A.n_rows;  // whole warps: n_rows is a multiple of 32
      if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[buf], (uint32_t)(item >> 1) & 1u, abort))) { ok = false; break; }
      tc_fence_after();
      for (int j0 = 16 * half; j0 < u.ntok; j0 += 32) {
        uint32_t g[16], up[16];
        tc_ld16(lane_base + buf * ACC_COLS + j0, g);
        if (NA == 2) tc_ld16(lane_base + buf * ACC_COLS + NTMAX + j0, up);
        float wv = 0.f;
        if (TERMS == 1) {
          if (NA == 2 && lane < 16 && j0 + lane < u.ntok) wv = A.row_w[u.row_start + j0 + lane];
        } else {
          if (NA == 2 && lane < 16 / TERMS && j0 + lane * TERMS < u.ntok) wv = A.row_w[(u.row_start + j0) / TERMS + lane];
        }
        tc_ld_wait();
        if (!rows_ok) continue;
        if constexpr (TERMS > 1) {
#pragma unroll
          for (int r = 0; r < 16 / TERMS; ++r) {
            if (j0 + r * TERMS >= u.ntok) break;
            const size_t rr = (size_t)(u.row_start + j0) / TERMS + r;  // routed row
            float gs = 0.f, us = 0.f;
#pragma unroll
            for (int tt = 0; tt < TERMS; ++tt) {
              gs += __uint_as_float(g[r * TERMS + tt]);
              if (NA == 2) us += __uint_as_float(up[r * TERMS + tt]);
            }
            if (A.round_bf16) gs = bf16_round(gs), us = bf16_round(us);
            if (NA == 2) {
              float res = swiglu(gs, us, A.limit) * __shfl_sync(0xffffffffu, wv, r);
              if (A.round_bf16) res = bf16_round(res);
#pragma unroll
              for (int tt = 0; tt < TERMS; ++tt) {
                const float amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(res))));
                const int e = mxfp4_exponent(amax);
                const float qv = res * pow2f(-e);
                const float qn = __shfl_down_sync(0xffffffffu, qv, 1);
                const uint32_t byte = e2m1x2_byte(qv, qn);
                const uint32_t pair = __shfl_sync(0xffffffffu, byte, lane & ~1);
                const uint32_t code = (lane & 1) ? pair >> 4 : pair & 15u;
                res -= e2m1_to_f32(code) * pow2f(e);
                const size_t row = rr * TERMS + tt;
                if ((lane & 1) == 0) A.h_codes[row * (size_t)(A.n_rows / 2) + (n >> 1)] = (uint8_t)byte;
                if (lane == 0) A.h_scales[row * (size_t)(A.n_rows / 32) + (n >> 5)] = (uint8_t)(e + 127);
              }
            } else {
              A.y32[rr * (size_t)A.n_rows + n] = gs;
            }
          }
        } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (j0 + j >= u.ntok) break;
          const size_t row = (size_t)(u.row_start + j0 + j);
          if (NA == 2) {
            const float wj = __shfl_sync(0xffffffffu, wv, j);
            float gg = bf16_round(__uint_as_float(g[j])), uu = bf16_round(__uint_as_float(up[j]));
            if (A.limit > 0.f) {
              uu = fminf(fmaxf(uu, -A.limit), A.limit);
              gg = fminf(gg, A.limit);
            }
            const float h = __fdividef(gg, 1.0f + __expf(-gg)) * uu * wj;
            const float amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(h))));
            const int e = mxfp4_exponent(amax);
            const float qv = h * pow2f(-e);
            const float qn = __shfl_down_sync(0xffffffffu, qv, 1);
            if ((lane & 1) == 0) A.h_codes[row * (size_t)(A.n_rows / 2) + (n >> 1)] = (uint8_t)e2m1x2_byte(qv, qn);
            if (lane == 0) A.h_scales[row * (size_t)(A.n_rows / 32) + (n >> 5)] = (uint8_t)(e + 127);
          } else {
            A.y[row * (size_t)A.n_rows + n] = __float2bfloat16_rn(__uint_as_float(g[j]));
          }
        }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    if (warp == 6 && lane == 0) {
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort) {
    if (threadIdx.x == 0 && A.status) atomicOr(A.status, CACHALOT_STATUS_WAIT_EXPIRED);
    // give tile loads still in flight time to land before the shared memory goes away
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
  }
}

// ---- planning ---------------------------------------------------------------------------------

// one CTA per expert: inverse permutation and source token of every grouped row of a present expert
__global__ void plan_rows_kernel(const int32_t* __restrict__ perm, const int32_t* __restrict__ offsets,
                                 const int32_t* __restrict__ slot_of_expert, int n_slots, int k, const float* __restrict__ gate_w,
                                 int32_t* __restrict__ inv, int32_t* __restrict__ src_token, float* __restrict__ row_w,
                                 int* __restrict__ status) {
  const int e = blockIdx.x;
  const int s = slot_of_expert ? slot_of_expert[e] : e;
  const bool present = s >= 0 && s < n_slots;
  if (s >= n_slots && status && threadIdx.x == 0 && offsets[e + 1] > offsets[e]) atomicOr(status, CACHALOT_STATUS_SLOT_RANGE);
  for (int p = offsets[e] + threadIdx.x; p < offsets[e + 1]; p += blockDim.x) {
    const int r = perm[p];
    src_token[p] = r / k;
    row_w[p] = gate_w[r];
    if (present) inv[r] = p;
  }
}

// single CTA: units of up to NTMAX rows per present expert, experts ascending
__global__ void plan_units_kernel(const int32_t* __restrict__ offsets, const int32_t* __restrict__ slot_of_expert, int n_experts,
                                  int n_slots, Unit* __restrict__ units, int32_t* __restrict__ n_units) {
  extern __shared__ int32_t sh[];  // [blockDim.x] unit counts of each thread's span
  const int t = threadIdx.x, nt = blockDim.x;
  const int per = (n_experts + nt - 1) / nt;
  const int lo = min(t * per, n_experts), hi = min(lo + per, n_experts);
  auto units_of = [&](int e) {
    const int s = slot_of_expert ? slot_of_expert[e] : e;
    if (s < 0 || s >= n_slots) return 0;
    return (offsets[e + 1] - offsets[e] + NTMAX - 1) / NTMAX;
  };
  int sum = 0;
  for (int e = lo; e < hi; ++e) sum += units_of(e);
  sh[t] = sum;
  __syncthreads();
  if (t == 0) {
    int run = 0;
    for (int i = 0; i < nt; ++i) {
      const int v = sh[i];
      sh[i] = run;
      run += v;
    }
    *n_units = run;
  }
  __syncthreads();
  int at = sh[t];
  for (int e = lo; e < hi; ++e) {
    const int nu = units_of(e);
    const int s = slot_of_expert ? slot_of_expert[e] : e;
    const int begin = offsets[e], end = offsets[e + 1];
    for (int i = 0; i < nu; ++i) {
      Unit u;
      u.slot = s;
      u.row_start = begin + i * NTMAX;
      u.ntok = min(NTMAX, end - u.row_start);
      u.pad = 0;
      units[at++] = u;
    }
  }
}

// one CTA per segment: rows of a segment whose expert is absent give zeros
__global__ void zero_absent_rows_kernel(const int32_t* __restrict__ offsets, const int32_t* __restrict__ seg_slot, int n_slots,
                                        int hidden, __nv_bfloat16* __restrict__ y) {
  const int g = blockIdx.x;
  const int s = seg_slot ? seg_slot[g] : g;
  if (s >= 0 && s < n_slots) return;
  uint32_t* base = reinterpret_cast<uint32_t*>(y + (size_t)offsets[g] * hidden);
  const size_t words = (size_t)(offsets[g + 1] - offsets[g]) * hidden / 2;
  for (size_t i = threadIdx.x; i < words; i += blockDim.x) base[i] = 0u;
}

// out[t, :] = sum over the token's route slots j = 0..k-1 (in that order) of its row of y
__global__ void combine_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ inv, int k, int hidden,
                               float* __restrict__ out) {
  const int t = blockIdx.x;
  for (int n = threadIdx.x * 2; n < hidden; n += blockDim.x * 2) {
    float a = 0.f, b = 0.f;
    for (int j = 0; j < k; ++j) {
      const int p = inv[t * k + j];
      if (p < 0) continue;
      const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(y + (size_t)p * hidden + n);
      a += __bfloat162float(v.x);
      b += __bfloat162float(v.y);
    }
    out[(size_t)t * hidden + n] = a;
    out[(size_t)t * hidden + n + 1] = b;
  }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// byte matrix [planes][rows][row_bytes] with the given pitches; box = {128 bytes, box_rows, 1}, 128-byte swizzle
int make_map(CUtensorMap* m, const void* base, int row_bytes, long long row_pitch, int rows, long long plane_pitch, int planes,
             int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(CACHALOT_ECUDA, "moe_prefill: cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {(cuuint64_t)row_bytes, (cuuint64_t)rows, (cuuint64_t)planes};
  cuuint64_t strides[2] = {(cuuint64_t)row_pitch, (cuuint64_t)plane_pitch};
  cuuint32_t box[3] = {(cuuint32_t)BKB, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  const int rank = planes > 0 ? 3 : 2;
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(CACHALOT_ECUDA, "moe_prefill: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return CACHALOT_OK;
}

constexpr int KSUB = 2;
constexpr int STAGES_GU = 4 / KSUB, STAGES_DN = 6 / KSUB;
constexpr size_t SMEM_LIMIT = 227 * 1024;
// stages, 256 bytes of barriers, optionally two raw scale slots, 1 KB of alignment slack
size_t smem_bytes(int na, int nstage, int nkb, bool raw) {
  size_t b = (size_t)nstage * KSUB * (na * A_TILE + B_TILE + (na + 1) * SF_TILE) + 256 + 1024;
  if (raw) b += 2 * ((size_t)na * ((BM * nkb + 15) & ~15) + ((NTMAX * nkb + 30) & ~15));
  return b;
}

struct RowScratch {  // of the rows-level entry
  uint8_t *h_codes, *h_scales;
  int32_t* n_units;
  Unit* units;
  size_t total;
};
RowScratch carve_rows(uint8_t* base, int inter, size_t rows, int n_seg) {
  RowScratch s;
  size_t at = 0;
  auto take = [&](size_t bytes) {
    uint8_t* p = base ? base + at : nullptr;
    at += align_up(bytes, 256);
    return p;
  };
  s.h_codes = take(rows * (inter / 2));
  s.h_scales = take(rows * (inter / 32) + 32);
  // a segment with r rows gives ceil(r / NTMAX) units and an empty one none: at most rows / NTMAX + min(n_seg, rows)
  s.units = reinterpret_cast<Unit*>(take((rows / NTMAX + ((size_t)n_seg < rows ? (size_t)n_seg : rows) + 1) * sizeof(Unit)));
  s.n_units = reinterpret_cast<int32_t*>(take(256));
  s.total = at;
  return s;
}

struct Scratch {  // of the whole prefill call: quantised input, per-row arrays, then the rows-level scratch
  uint8_t *x_codes, *x_scales;
  __nv_bfloat16* y;
  int32_t *inv, *src_token;
  float* row_w;
  uint8_t* rows_ws;
  size_t total;
};
Scratch carve(uint8_t* base, int hidden, int inter, size_t rows, int n_experts) {
  Scratch s;
  size_t at = 0;
  auto take = [&](size_t bytes) {
    uint8_t* p = base ? base + at : nullptr;
    at += align_up(bytes, 256);
    return p;
  };
  s.x_codes = take(rows * (hidden / 2));
  s.x_scales = take(rows * (hidden / 32) + 32);
  s.y = reinterpret_cast<__nv_bfloat16*>(take(rows * hidden * 2));
  s.inv = reinterpret_cast<int32_t*>(take(rows * 4));
  s.src_token = reinterpret_cast<int32_t*>(take(rows * 4));
  s.row_w = reinterpret_cast<float*>(take(rows * 4));
  s.rows_ws = take(carve_rows(nullptr, inter, rows, n_experts).total);
  s.total = at;
  return s;
}

// ---- decode batches on the same grouped kernels ------------------------------------------------------

constexpr int DTERMS = 4;  // MXFP4 rows per routed row

// single CTA: routed rows (token * k + route slot) ordered by bank slot, stable; runs of one slot become segments of
// DTERMS rows per routed row.  seg_off i32 [R + 1] (in MXFP4 rows), seg_slot i32 [R] (-1 behind the last segment and
// for rows whose slot is absent or out of range), inv i32 [R] (position of a routed row in the order, -1 if absent),
// src_token i32 [R] and row_w f32 [R] in the order.
__global__ void decode_plan_kernel(const int32_t* __restrict__ slots, const float* __restrict__ gate_w, int R, int k, int n_slots,
                                   int32_t* __restrict__ seg_off, int32_t* __restrict__ seg_slot, int32_t* __restrict__ inv,
                                   int32_t* __restrict__ src_token, float* __restrict__ row_w, int* __restrict__ status) {
  extern __shared__ int32_t sh[];  // [R] slot of every row, [R] slot by position
  int32_t* s_in = sh;
  int32_t* s_sorted = sh + R;
  bool oob = false;
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    int v = slots[i];
    if (v >= n_slots) oob = true, v = -1;
    s_in[i] = v < 0 ? -1 : v;
  }
  if (oob && status) atomicOr(status, CACHALOT_STATUS_SLOT_RANGE);
  __syncthreads();
  for (int i = threadIdx.x; i < R; i += blockDim.x) {
    const int v = s_in[i];
    int rank = 0;
    for (int j = 0; j < R; ++j) {
      const int o = s_in[j];
      rank += (o < v || (o == v && j < i)) ? 1 : 0;
    }
    s_sorted[rank] = v;
    inv[i] = v < 0 ? -1 : rank;
    src_token[rank] = i / k;
    const float w = gate_w[i];
    if (!(fabsf(w) <= 3.0e38f) && status) atomicOr(status, CACHALOT_STATUS_BAD_WEIGHT);
    row_w[rank] = w;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int ng = 0;
    for (int i = 0; i < R; ++i)
      if (i == 0 || s_sorted[i] != s_sorted[i - 1]) {
        seg_off[ng] = i * DTERMS;
        seg_slot[ng] = s_sorted[i];
        ++ng;
      }
    for (int gidx = ng; gidx <= R; ++gidx) {
      seg_off[gidx] = R * DTERMS;
      if (gidx < R) seg_slot[gidx] = -1;
    }
  }
}

// One thread per 8 consecutive elements (one 16-byte load), four threads per 32-block: the block as DTERMS MXFP4
// blocks, each the quantisation (reference rule: model/fp4_act_mlx.py:101-250) of what the ones before it left over.
// x bf16 [tokens, K]; row p reads token src[p].
__global__ void mxfp4_residual_quant_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ src, int rows, int k,
                                            uint8_t* __restrict__ codes, uint8_t* __restrict__ scales) {
  const int per_row = k / 8;
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const bool live = i < (long long)rows * per_row;
  const long long p = live ? i / per_row : 0;
  const int c = live ? (int)(i - p * per_row) : 0;
  uint4 raw = make_uint4(0, 0, 0, 0);
  if (live) raw = *reinterpret_cast<const uint4*>(x + (size_t)src[p] * k + c * 8);
  const uint32_t wds[4] = {raw.x, raw.y, raw.z, raw.w};
  float res[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) res[2 * j] = __uint_as_float(wds[j] << 16), res[2 * j + 1] = __uint_as_float(wds[j] & 0xffff0000u);
#pragma unroll
  for (int tt = 0; tt < DTERMS; ++tt) {
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(res[j]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    const int e = mxfp4_exponent(amax);
    const float inv = pow2f(-e), sc = pow2f(e);
    uint32_t packed = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t byte = e2m1x2_byte(res[2 * j] * inv, res[2 * j + 1] * inv);
      packed |= byte << (8 * j);
      res[2 * j] -= e2m1_to_f32(byte & 15u) * sc;
      res[2 * j + 1] -= e2m1_to_f32(byte >> 4) * sc;
    }
    if (live) {
      const size_t row = (size_t)p * DTERMS + tt;
      *reinterpret_cast<uint32_t*>(codes + row * (size_t)(k / 2) + c * 4) = packed;
      if ((c & 3) == 0) scales[row * (size_t)(k / 32) + (c >> 2)] = (uint8_t)(e + 127);
    }
  }
}

// out[t, :] = sum over the token's route slots j = 0..k-1 (in that order) of its fp32 row
template <typename OutT>
__global__ void decode_combine_kernel(const float* __restrict__ y, const int32_t* __restrict__ inv, int k, int hidden, OutT* __restrict__ out) {
  const int t = blockIdx.x;
  for (int n = threadIdx.x; n < hidden; n += blockDim.x) {
    float a = 0.f;
    for (int j = 0; j < k; ++j) {
      const int p = inv[t * k + j];
      if (p >= 0) a += y[(size_t)p * hidden + n];
    }
    if constexpr (sizeof(OutT) == 2)
      out[(size_t)t * hidden + n] = __float2bfloat16_rn(a);
    else
      out[(size_t)t * hidden + n] = a;
  }
}

struct DecodeScratch {
  int32_t *seg_off, *seg_slot, *inv, *src_token, *n_units;
  float *row_w, *y32;
  uint8_t *x_codes, *x_scales, *h_codes, *h_scales;
  Unit* units;
  size_t total;
};
DecodeScratch carve_decode(uint8_t* base, int hidden, int inter, size_t R, size_t n_seg = 0) {
  DecodeScratch s;
  size_t at = 0;
  auto take = [&](size_t bytes) {
    uint8_t* p = base ? base + at : nullptr;
    at += align_up(bytes, 256);
    return p;
  };
  const size_t Q = R * DTERMS;
  const size_t S = n_seg > R ? n_seg : R;  // segments: one per routed row at most (decode), or one per expert (prefill)
  s.seg_off = reinterpret_cast<int32_t*>(take((S + 1) * 4));
  s.seg_slot = reinterpret_cast<int32_t*>(take(S * 4));
  s.inv = reinterpret_cast<int32_t*>(take(R * 4));
  s.src_token = reinterpret_cast<int32_t*>(take(R * 4));
  s.row_w = reinterpret_cast<float*>(take(R * 4));
  s.n_units = reinterpret_cast<int32_t*>(take(256));
  s.units = reinterpret_cast<Unit*>(take((Q / NTMAX + (S < R ? S : R) + R + 1) * sizeof(Unit)));
  s.x_codes = take(Q * (hidden / 2));
  s.x_scales = take(Q * (hidden / 32) + 32);
  s.h_codes = take(Q * (inter / 2));
  s.h_scales = take(Q * (inter / 32) + 32);
  s.y32 = reinterpret_cast<float*>(take(R * (size_t)hidden * 4));
  s.total = at;
  return s;
}

}  // namespace

bool decode_tc_supported(const BankView& v, int rows, int k) {
  return prefill_tc_supported(v) && rows >= 1 && (long long)rows * k <= 1024;
}
size_t decode_tc_workspace_bytes(int hidden, int inter, int rows, int k) { return carve_decode(nullptr, hidden, inter, (size_t)rows * k).total; }

// The two grouped GEMMs over DTERMS residual MXFP4 rows per routed row (gate/up with SwiGLU, router weight and the
// re-quantisation of h; down into s.y32).  seg_off is in MXFP4 rows; seg_slot may be null (segment e = slot e).
static int run_terms4(const BankView& v, const DecodeScratch& s, const int32_t* seg_off, const int32_t* seg_slot, int n_seg, long long Q,
                      float limit, bool round_bf16, int* status, cudaStream_t stream) {
  const int H = v.hidden, I = v.inter;
  plan_units_kernel<<<1, 256, 256 * sizeof(int32_t), stream>>>(seg_off, seg_slot, n_seg, v.n_slots, s.units, s.n_units);
  int rc;
  if ((rc = check_launch("moe (grouped, exact activations) plan"))) return rc;
  CUtensorMap m_w1, m_w3, m_w2, m_x, m_h;
  if ((rc = make_map(&m_w1, v.base + v.off[0], H / 2, H / 2, I, v.record_bytes, v.n_slots, BM))) return rc;
  if ((rc = make_map(&m_w3, v.base + v.off[4], H / 2, H / 2, I, v.record_bytes, v.n_slots, BM))) return rc;
  if ((rc = make_map(&m_w2, v.base + v.off[2], I / 2, I / 2, H, v.record_bytes, v.n_slots, BM))) return rc;
  if ((rc = make_map(&m_x, s.x_codes, H / 2, H / 2, (int)Q, 0, 0, NTMAX))) return rc;
  if ((rc = make_map(&m_h, s.h_codes, I / 2, I / 2, (int)Q, 0, 0, NTMAX))) return rc;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  auto launch = [&](auto kern, int na, int nstage, bool raw, const CUtensorMap& ma0, const CUtensorMap& ma1, const CUtensorMap& mb,
                    const GemmArgs& ga) {
    const size_t sm = smem_bytes(na, nstage, ga.k_codes / 32, raw);
    smem_optin_once(kern, (int)SMEM_LIMIT);
    kern<<<sms, NTHREADS, sm, stream>>>(ma0, ma1, mb, ga);
  };
  GemmArgs a = {};
  a.bank = v.base;
  a.record_bytes = v.record_bytes;
  a.units = s.units;
  a.n_units = s.n_units;
  a.total_rows = (int)Q;
  a.row_w = s.row_w;
  a.limit = limit;
  a.h_codes = s.h_codes;
  a.h_scales = s.h_scales;
  a.y = nullptr;
  a.y32 = s.y32;
  a.round_bf16 = round_bf16 ? 1 : 0;
  a.status = status;
  a.off_sc[0] = v.off[1];
  a.off_sc[1] = v.off[5];
  a.act_scales = s.x_scales;
  a.n_rows = I;
  a.k_codes = H;
  if (smem_bytes(2, STAGES_GU, H / 32, true) <= SMEM_LIMIT)
    launch(grouped_mxf4_kernel<2, STAGES_GU, KSUB, true, DTERMS>, 2, STAGES_GU, true, m_w1, m_w3, m_x, a);
  else
    launch(grouped_mxf4_kernel<2, STAGES_GU, KSUB, false, DTERMS>, 2, STAGES_GU, false, m_w1, m_w3, m_x, a);
  if ((rc = check_launch("moe (grouped, exact activations) gate/up"))) return rc;
  a.off_sc[0] = v.off[3];
  a.off_sc[1] = v.off[3];
  a.act_scales = s.h_scales;
  a.n_rows = H;
  a.k_codes = I;
  if (smem_bytes(1, STAGES_DN, I / 32, true) <= SMEM_LIMIT)
    launch(grouped_mxf4_kernel<1, STAGES_DN, KSUB, true, DTERMS>, 1, STAGES_DN, true, m_w2, m_w2, m_h, a);
  else
    launch(grouped_mxf4_kernel<1, STAGES_DN, KSUB, false, DTERMS>, 1, STAGES_DN, false, m_w2, m_w2, m_h, a);
  return check_launch("moe (grouped, exact activations) down");
}

static void residual_quant(const void* x_bf16, const DecodeScratch& s, long long R, int H, cudaStream_t stream) {
  const long long threads = R * (H / 8);
  mxfp4_residual_quant_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)x_bf16, s.src_token, (int)R, H,
                                                                                    s.x_codes, s.x_scales);
}

// Routed experts of a decode batch with every distinct expert streamed once: rows grouped by bank slot, activations as
// DTERMS residual MXFP4 rows, the two grouped block-scaled GEMMs, slot-ordered fp32 sum.  round_bf16 = false: fp32
// numerics (the FP4 decode op); true: the reference's per-expert prefill rounding points.
int launch_decode_tc(const BankView& v, const void* x_bf16, const int32_t* slots, const float* gate_w, int rows, int k, float limit,
                     void* workspace, void* out, int out_dtype, int* status, cudaStream_t stream, bool round_bf16) {
  if (!decode_tc_supported(v, rows, k)) return CACHALOT_EUNSUPPORTED;
  const int H = v.hidden, R = rows * k;
  const DecodeScratch s = carve_decode(static_cast<uint8_t*>(workspace), H, v.inter, (size_t)R);
  const int threads = R < 1024 ? ((R + 31) / 32) * 32 : 1024;
  decode_plan_kernel<<<1, threads, 2 * R * sizeof(int32_t), stream>>>(slots, gate_w, R, k, v.n_slots, s.seg_off, s.seg_slot, s.inv, s.src_token,
                                                                    s.row_w, status);
  residual_quant(x_bf16, s, R, H, stream);
  int rc = run_terms4(v, s, s.seg_off, s.seg_slot, R, (long long)R * DTERMS, limit, round_bf16, status, stream);
  if (rc) return rc;
  if (out_dtype == CACHALOT_BF16)
    decode_combine_kernel<<<rows, 256, 0, stream>>>(s.y32, s.inv, k, H, static_cast<__nv_bfloat16*>(out));
  else
    decode_combine_kernel<<<rows, 256, 0, stream>>>(s.y32, s.inv, k, H, static_cast<float*>(out));
  return check_launch("moe_decode (grouped) combine");
}

__global__ void scale_offsets_kernel(const int32_t* __restrict__ in, int n, int mul, int32_t* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = in[i] * mul;
}

// Expert-major prefill with bf16 activations taken as they are (the reference's per-expert prefill numerics,
// model/moe_prefill_batched.py:31-61): the grouping's permutation and offsets as in launch_prefill_tc, activations
// as DTERMS residual MXFP4 rows (their sum reproduces the bf16 value to 2.4e-4), g, u, h and y rounded to bf16.
size_t prefill_exact_workspace_bytes(int hidden, int inter, int tokens, int k, int n_experts) {
  return carve_decode(nullptr, hidden, inter, (size_t)tokens * k, (size_t)n_experts).total;
}
int launch_prefill_exact(const BankView& v, const void* x_bf16, const int32_t* perm, const int32_t* offsets, const int32_t* slot_of_expert,
                         const float* gate_w, int tokens, int k, int n_experts, float limit, void* workspace, float* out, int* status,
                         cudaStream_t stream) {
  if (!prefill_tc_supported(v)) return CACHALOT_EUNSUPPORTED;
  const int H = v.hidden;
  const size_t R = (size_t)tokens * k;
  if (R * DTERMS > 0x7fffffffULL) return CACHALOT_EUNSUPPORTED;
  const DecodeScratch s = carve_decode(static_cast<uint8_t*>(workspace), H, v.inter, R, (size_t)n_experts);
  cudaError_t e = cudaMemsetAsync(s.inv, 0xFF, R * 4, stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(s.src_token, 0, R * 4, stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(s.row_w, 0, R * 4, stream);
  if (e != cudaSuccess) return fail(CACHALOT_ECUDA, "moe_prefill: %s", cudaGetErrorString(e));
  plan_rows_kernel<<<n_experts, 128, 0, stream>>>(perm, offsets, slot_of_expert, v.n_slots, k, gate_w, s.inv, s.src_token, s.row_w, status);
  scale_offsets_kernel<<<(n_experts + 256) / 256, 256, 0, stream>>>(offsets, n_experts + 1, DTERMS, s.seg_off);
  int rc;
  if ((rc = check_launch("moe_prefill plan rows"))) return rc;
  residual_quant(x_bf16, s, (long long)R, H, stream);
  if ((rc = run_terms4(v, s, s.seg_off, slot_of_expert, n_experts, (long long)R * DTERMS, limit, true, status, stream))) return rc;
  decode_combine_kernel<<<tokens, 256, 0, stream>>>(s.y32, s.inv, k, H, out);
  return check_launch("moe_prefill combine");
}

bool prefill_tc_supported(const BankView& v) {
  // inter a multiple of 64: rows of scale bytes start on even addresses (the loaders read them in 2-byte units)
  return v.format == CACHALOT_BANK_FP4 && v.hidden % 128 == 0 && v.inter % 64 == 0 && (v.hidden / 2) % 16 == 0 &&
         (v.inter / 2) % 16 == 0 && v.record_bytes % 16 == 0;
}

size_t prefill_tc_workspace_bytes(int hidden, int inter, int tokens, int k, int n_experts) {
  return carve(nullptr, hidden, inter, (size_t)tokens * k, n_experts).total;
}
size_t prefill_rows_workspace_bytes(int inter, long long rows, int n_seg) { return carve_rows(nullptr, inter, (size_t)rows, n_seg).total; }

// Grouped rows in, per-row expert outputs out: x_codes/x_scales = MXFP4 rows [rows, H/2] / [rows, H/32] laid out in
// segments (seg_offsets i32 [n_seg+1], device), segment g belongs to bank slot seg_slot[g] (null: g; out of range or
// negative: absent -> zero rows when zero_absent), row_w f32 [rows]; y bf16 [rows, H].
int launch_prefill_rows(const BankView& v, const uint8_t* x_codes, const uint8_t* x_scales, const float* row_w,
                        const int32_t* seg_offsets, const int32_t* seg_slot, int n_seg, long long rows, float limit, bool zero_absent,
                        void* workspace, __nv_bfloat16* y, int* status, cudaStream_t stream) {
  if (!prefill_tc_supported(v)) return CACHALOT_EUNSUPPORTED;
  if (rows <= 0 || n_seg <= 0) return CACHALOT_OK;
  const int H = v.hidden, I = v.inter;
  const RowScratch s = carve_rows(static_cast<uint8_t*>(workspace), I, (size_t)rows, n_seg);
  CUtensorMap m_w1, m_w3, m_w2, m_x, m_h;
  int rc;
  if ((rc = make_map(&m_w1, v.base + v.off[0], H / 2, H / 2, I, v.record_bytes, v.n_slots, BM))) return rc;
  if ((rc = make_map(&m_w3, v.base + v.off[4], H / 2, H / 2, I, v.record_bytes, v.n_slots, BM))) return rc;
  if ((rc = make_map(&m_w2, v.base + v.off[2], I / 2, I / 2, H, v.record_bytes, v.n_slots, BM))) return rc;
  if ((rc = make_map(&m_x, x_codes, H / 2, H / 2, (int)rows, 0, 0, NTMAX))) return rc;
  if ((rc = make_map(&m_h, s.h_codes, I / 2, I / 2, (int)rows, 0, 0, NTMAX))) return rc;
  plan_units_kernel<<<1, 256, 256 * sizeof(int32_t), stream>>>(seg_offsets, seg_slot, n_seg, v.n_slots, s.units, s.n_units);
  if (zero_absent) zero_absent_rows_kernel<<<n_seg, 256, 0, stream>>>(seg_offsets, seg_slot, v.n_slots, H, y);
  if ((rc = check_launch("moe_prefill plan"))) return rc;

  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  auto launch = [&](auto kern, int na, int nstage, bool raw, const CUtensorMap& ma0, const CUtensorMap& ma1, const CUtensorMap& mb,
                    const GemmArgs& ga) {
    const size_t sm = smem_bytes(na, nstage, ga.k_codes / 32, raw);
    smem_optin_once(kern, (int)SMEM_LIMIT);
    kern<<<sms, NTHREADS, sm, stream>>>(ma0, ma1, mb, ga);
  };
  GemmArgs a;
  a.bank = v.base;
  a.record_bytes = v.record_bytes;
  a.units = s.units;
  a.n_units = s.n_units;
  a.total_rows = (int)rows;
  a.row_w = row_w;
  a.limit = limit;
  a.h_codes = s.h_codes;
  a.h_scales = s.h_scales;
  a.y = y;
  a.status = status;
  // gate/up: K = hidden, N = inter
  a.off_sc[0] = v.off[1];
  a.off_sc[1] = v.off[5];
  a.act_scales = x_scales;
  a.n_rows = I;
  a.k_codes = H;
  if (smem_bytes(2, STAGES_GU, H / 32, true) <= SMEM_LIMIT)
    launch(grouped_mxf4_kernel<2, STAGES_GU, KSUB, true>, 2, STAGES_GU, true, m_w1, m_w3, m_x, a);
  else
    launch(grouped_mxf4_kernel<2, STAGES_GU, KSUB, false>, 2, STAGES_GU, false, m_w1, m_w3, m_x, a);
  if ((rc = check_launch("moe_prefill gate/up (tcgen05)"))) return rc;
  // down: K = inter, N = hidden
  a.off_sc[0] = v.off[3];
  a.off_sc[1] = v.off[3];
  a.act_scales = s.h_scales;
  a.n_rows = H;
  a.k_codes = I;
  if (smem_bytes(1, STAGES_DN, I / 32, true) <= SMEM_LIMIT)
    launch(grouped_mxf4_kernel<1, STAGES_DN, KSUB, true>, 1, STAGES_DN, true, m_w2, m_w2, m_h, a);
  else
    launch(grouped_mxf4_kernel<1, STAGES_DN, KSUB, false>, 1, STAGES_DN, false, m_w2, m_w2, m_h, a);
  return check_launch("moe_prefill down (tcgen05)");
}

int launch_combine_rows(const __nv_bfloat16* y, const int32_t* inv, int tokens, int k, int hidden, float* out, cudaStream_t stream) {
  if (tokens <= 0) return CACHALOT_OK;
  combine_kernel<<<tokens, 256, 0, stream>>>(y, inv, k, hidden, out);
  return check_launch("moe_prefill combine");
}

int launch_prefill_tc(const BankView& v, const void* x_bf16, const int32_t* perm, const int32_t* offsets,
                      const int32_t* slot_of_expert, const float* gate_w, int tokens, int k, int n_experts, float limit,
                      void* workspace, float* out, int* status, cudaStream_t stream) {
  if (!prefill_tc_supported(v)) return CACHALOT_EUNSUPPORTED;
  const int H = v.hidden, I = v.inter;
  const size_t rows = (size_t)tokens * k;
  const Scratch s = carve(static_cast<uint8_t*>(workspace), H, I, rows, n_experts);
  cudaError_t e = cudaMemsetAsync(s.inv, 0xFF, rows * 4, stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(s.src_token, 0, rows * 4, stream);
  if (e == cudaSuccess) e = cudaMemsetAsync(s.row_w, 0, rows * 4, stream);
  if (e != cudaSuccess) return fail(CACHALOT_ECUDA, "moe_prefill: memset: %s", cudaGetErrorString(e));
  plan_rows_kernel<<<n_experts, 128, 0, stream>>>(perm, offsets, slot_of_expert, v.n_slots, k, gate_w, s.inv, s.src_token, s.row_w,
                                                 status);
  int rc;
  if ((rc = check_launch("moe_prefill plan rows"))) return rc;
  if ((rc = cachalot_mxfp4_act_quant(x_bf16, s.src_token, (int)rows, H, s.x_codes, s.x_scales, stream))) return rc;
  // rows of absent experts are skipped by the combine (inv = -1), so they need no zeroing
  if ((rc = launch_prefill_rows(v, s.x_codes, s.x_scales, s.row_w, offsets, slot_of_expert, n_experts, (long long)rows, limit, false,
                                s.rows_ws, s.y, status, stream)))
    return rc;
  return launch_combine_rows(s.y, s.inv, tokens, k, H, out, stream);
}

}  // namespace cachalot

