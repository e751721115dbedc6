// Decode-time routed experts over bank slots: two launches per call for all (token, route slot)
// rows, as the reference's fused pair does for one token:
//   gate_up : hidden[r, i] = silu(min(g,L)) * clip(u,+-L) * gate_w[r]      r = token*k + route slot
//   down    : out[t, n]    = sum_j  W2_{slot(t,j)}[n, :] . hidden[t*k+j, :]  (j = 0..k-1 in order)
// Weights are read as 16-byte chunks straight from the slot record (FP4: 32 codes + one E8M0
// byte; 2-bit affine: 64 codes, scale/bias per group), activations sit in shared memory in a
// chunk-transposed order so that a warp's lanes hit distinct banks.
#include <cstdlib>
#include <mutex>

#include "kernels.cuh"

namespace cachalot {

__device__ __forceinline__ float scale_at(const void* p, long long i, int dt) {
  return dt == CACHALOT_F16 ? __half2float(reinterpret_cast<const __half*>(p)[i])
                            : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// Lane-partial dot product of one weight row with the activation in shared memory.
//   xs    : activation, element (c*CH + i) stored at xs[i*nch + c]
//   xsum  : per-chunk sums of the activation (affine only)
template <int FMT>
__device__ __forceinline__ float row_dot(const uint8_t* __restrict__ w, const uint8_t* __restrict__ sc,
                                         const uint8_t* __restrict__ bi, long long row, int K, int group, int sdt,
                                         const float* __restrict__ xs, const float* __restrict__ xsum,
                                         const float* __restrict__ lut, int lane) {
  constexpr int CH = Fmt<FMT>::CH;
  const int nch = K / CH;
  const uint8_t* wrow = w + row * (long long)(nch * 16);
  float acc = 0.f;
  for (int c = lane; c < nch; c += 32) {
    uint4 v = ld_stream_u4(wrow + (size_t)c * 16);
    uint32_t words[4] = {v.x, v.y, v.z, v.w};
    float part = 0.f;
    if constexpr (FMT == CACHALOT_BANK_FP4) {
      float s = e8m0_to_f32(sc[row * nch + c]);
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          uint32_t code = (words[wi] >> (4 * n)) & 15u;
          part = fmaf(lut[code], xs[(wi * 8 + n) * nch + c], part);
        }
      }
      acc = fmaf(part, s, acc);
    } else {
      // groups run over the flattened [N*K] element index, which is the reference's [N, K/group]
      // layout whenever K is a multiple of the group
      long long g = (row * (long long)K + (long long)c * CH) / group;
      float s = scale_at(sc, g, sdt), b = scale_at(bi, g, sdt);
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
        for (int n = 0; n < 16; ++n) {
          uint32_t code = (words[wi] >> (2 * n)) & 3u;
          part = fmaf(lut[code], xs[(wi * 16 + n) * nch + c], part);
        }
      }
      acc = fmaf(s, part, acc);
      acc = fmaf(b, xsum[c], acc);
    }
  }
  return acc;
}

__device__ __forceinline__ void fill_lut(float* lut, int fmt) {
  if (threadIdx.x < 16) lut[threadIdx.x] = fmt == CACHALOT_BANK_FP4 ? e2m1_to_f32(threadIdx.x) : (float)threadIdx.x;
}

// stage `K` activations (read through `get(k)`) chunk-transposed, plus per-chunk sums
template <int CH, typename F>
__device__ __forceinline__ void stage(float* xs, float* xsum, int K, F get) {
  const int nch = K / CH;
  for (int e = threadIdx.x; e < K; e += blockDim.x) {
    int c = e / CH, i = e - c * CH;
    xs[i * nch + c] = get(e);
  }
  __syncthreads();
  if (xsum) {
    for (int c = threadIdx.x; c < nch; c += blockDim.x) {
      float s = 0.f;
      for (int i = 0; i < CH; ++i) s += xs[i * nch + c];
      xsum[c] = s;
    }
    __syncthreads();
  }
}

constexpr int WARPS = 8;

// grid = (ceil(I / WARPS), rows*k): one warp per (row r, intermediate index i)
template <int FMT>
__global__ void __launch_bounds__(WARPS * 32)
gate_up_kernel(BankView bank, const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ slots,
               const float* __restrict__ gate_w, int k, float limit, int numerics, float* __restrict__ hidden,
               int* __restrict__ status) {
  extern __shared__ float smem[];
  constexpr int CH = Fmt<FMT>::CH;
  const int H = bank.hidden, I = bank.inter;
  float* xs = smem;
  float* xsum = FMT == CACHALOT_BANK_AFFINE ? smem + H : nullptr;
  __shared__ float lut[16];
  const int r = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i = blockIdx.x * WARPS + warp;
  const int slot = slots[r];
  if (slot < 0 || slot >= bank.n_slots) {  // absent expert: zero rows, never an out-of-range read
    if (slot >= bank.n_slots && status && threadIdx.x == 0) atomicOr(status, CACHALOT_STATUS_SLOT_RANGE);
    if (i < I && lane == 0) hidden[(size_t)r * I + i] = 0.f;
    return;
  }
  fill_lut(lut, FMT);
  const __nv_bfloat16* xr = x + (size_t)(r / k) * H;
  stage<CH>(xs, xsum, H, [&](int e) { return __bfloat162float(xr[e]); });
  __syncthreads();
  if (i >= I) return;
  const uint8_t* rec = bank.base + (size_t)slot * bank.record_bytes;
  float g, u;
  if constexpr (FMT == CACHALOT_BANK_FP4) {
    g = row_dot<FMT>(rec + bank.off[0], rec + bank.off[1], nullptr, i, H, 32, 0, xs, xsum, lut, lane);
    u = row_dot<FMT>(rec + bank.off[4], rec + bank.off[5], nullptr, i, H, 32, 0, xs, xsum, lut, lane);
  } else {
    g = row_dot<FMT>(rec + bank.off[0], rec + bank.off[1], rec + bank.off[2], i, H, bank.group, bank.scale_dtype, xs, xsum, lut, lane);
    u = row_dot<FMT>(rec + bank.off[6], rec + bank.off[7], rec + bank.off[8], i, H, bank.group, bank.scale_dtype, xs, xsum, lut, lane);
  }
  g = warp_sum(g);
  u = warp_sum(u);
  if (lane == 0) {
    if (numerics != CACHALOT_NUMERICS_F32) {
      g = bf16_round(g);
      u = bf16_round(u);
    }
    float h = swiglu(g, u, limit) * gate_w[r];
    if (numerics == CACHALOT_NUMERICS_BF16) h = bf16_round(h);
    hidden[(size_t)r * I + i] = h;
  }
}

// grid = (ceil(H / WARPS), rows): one warp per (token t, output index n), experts summed j = 0..k-1
template <int FMT, typename OutT>
__global__ void __launch_bounds__(WARPS * 32)
down_kernel(BankView bank, const float* __restrict__ hidden, const int32_t* __restrict__ slots, int k, int numerics,
            OutT* __restrict__ out) {
  extern __shared__ float smem[];
  constexpr int CH = Fmt<FMT>::CH;
  const int H = bank.hidden, I = bank.inter;
  float* hs = smem;
  float* hsum = FMT == CACHALOT_BANK_AFFINE ? smem + I : nullptr;
  __shared__ float lut[16];
  const int t = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * WARPS + warp;
  fill_lut(lut, FMT);
  float total = 0.f;
  for (int j = 0; j < k; ++j) {
    const int r = t * k + j;
    const int slot = slots[r];
    if (slot < 0 || slot >= bank.n_slots) continue;  // uniform across the CTA
    __syncthreads();
    const float* hr = hidden + (size_t)r * I;
    stage<CH>(hs, hsum, I, [&](int e) { return hr[e]; });
    __syncthreads();
    if (n < H) {
      const uint8_t* rec = bank.base + (size_t)slot * bank.record_bytes;
      float y;
      if constexpr (FMT == CACHALOT_BANK_FP4)
        y = row_dot<FMT>(rec + bank.off[2], rec + bank.off[3], nullptr, n, I, 32, 0, hs, hsum, lut, lane);
      else
        y = row_dot<FMT>(rec + bank.off[3], rec + bank.off[4], rec + bank.off[5], n, I, bank.group, bank.scale_dtype, hs, hsum, lut, lane);
      y = warp_sum(y);
      if (numerics != CACHALOT_NUMERICS_F32) y = bf16_round(y);
      total += y;
    }
  }
  if (n < H && lane == 0) {
    if constexpr (sizeof(OutT) == 2)
      out[(size_t)t * H + n] = __float2bfloat16_rn(total);
    else
      out[(size_t)t * H + n] = total;
  }
}

static int make_view(const void* bank, const cachalot_bank_desc* d, BankView* v, const char* who) {
  if (!bank || !d) return fail(CACHALOT_EINVAL, "%s: null bank", who);
  if (d->hidden <= 0 || d->inter <= 0 || d->n_slots <= 0) return fail(CACHALOT_EINVAL, "%s: bad bank shape", who);
  int n_t;
  if (d->format == CACHALOT_BANK_FP4) {
    n_t = 6;
    if (d->hidden % 32 || d->inter % 32)
      return fail(CACHALOT_EINVAL, "%s: FP4 bank needs hidden and inter to be multiples of 32 (got %d, %d)", who, d->hidden, d->inter);
  } else if (d->format == CACHALOT_BANK_AFFINE) {
    n_t = 9;
    if (d->bits != 2) return fail(CACHALOT_EUNSUPPORTED, "%s: affine bank with bits=%d (only 2-bit is built)", who, d->bits);
    if (d->group != 64 && d->group != 128) return fail(CACHALOT_EUNSUPPORTED, "%s: affine group %d (64 or 128)", who, d->group);
    if (d->hidden % 64 || d->inter % 64)
      return fail(CACHALOT_EINVAL, "%s: 2-bit bank needs hidden and inter to be multiples of 64 (got %d, %d)", who, d->hidden, d->inter);
    if (((long long)d->hidden * d->inter) % d->group) return fail(CACHALOT_EINVAL, "%s: matrix size is not a whole number of groups", who);
    if (d->scale_dtype != CACHALOT_F16 && d->scale_dtype != CACHALOT_BF16) return fail(CACHALOT_EINVAL, "%s: scale dtype must be f16 or bf16", who);
  } else {
    return fail(CACHALOT_EINVAL, "%s: unknown bank format %d", who, d->format);
  }
  if (!aligned(bank, 16) || d->record_bytes % 16) return fail(CACHALOT_EALIGN, "%s: bank base and record_bytes must be multiples of 16", who);
  for (int i = 0; i < n_t; ++i) {
    if (d->off[i] < 0 || d->off[i] % 16 || d->off[i] >= d->record_bytes)
      return fail(CACHALOT_EALIGN, "%s: tensor offset %d (%lld) must be a multiple of 16 inside the record", who, i, (long long)d->off[i]);
    v->off[i] = d->off[i];
  }
  v->base = static_cast<const uint8_t*>(bank);
  v->record_bytes = d->record_bytes;
  v->n_slots = d->n_slots;
  v->hidden = d->hidden;
  v->inter = d->inter;
  v->bits = d->bits;
  v->group = d->group;
  v->scale_dtype = d->scale_dtype;
  v->format = d->format;
  v->scale_centre = d->fp4_scale_centre > 0 ? d->fp4_scale_centre : 121;
  if (v->scale_centre > 254) return fail(CACHALOT_EINVAL, "%s: fp4_scale_centre %d out of range", who, d->fp4_scale_centre);
  return CACHALOT_OK;
}

template <int FMT>
static int launch_decode(const BankView& v, const void* x, const int32_t* slots, const float* gate_w, int rows, int k,
                         float limit, int numerics_flags, float* hidden, void* out, int out_dtype, int* status,
                         cudaStream_t stream, bool mx_hidden = false) {
  const int numerics = numerics_flags & 0xff;
  const bool do_gate_up = !(numerics_flags & CACHALOT_DECODE_ONLY_DOWN);
  const bool do_down = !(numerics_flags & CACHALOT_DECODE_ONLY_GATE_UP);
  constexpr int CH = Fmt<FMT>::CH;
  const int H = v.hidden, I = v.inter;
  size_t smem_gu = (size_t)H * 4 + (FMT == CACHALOT_BANK_AFFINE ? (size_t)(H / CH) * 4 : 0);
  size_t smem_dn = (size_t)I * 4 + (FMT == CACHALOT_BANK_AFFINE ? (size_t)(I / CH) * 4 : 0);
  if (smem_gu > 200 * 1024 || smem_dn > 200 * 1024) return fail(CACHALOT_EINVAL, "moe_decode: hidden/inter too large for shared memory");
  // the shared-memory opt-in is a per-device attribute of a kernel: once per device and format
  static bool attr_done[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(CACHALOT_ECUDA, "moe_decode: no current device");
  if (!attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gate_up_kernel<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(down_kernel<FMT, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(down_kernel<FMT, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return fail(CACHALOT_ECUDA, "moe_decode: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done[dev] = true;
  }
  int rc = CACHALOT_OK;
  if (do_gate_up) {
    dim3 g1((I + WARPS - 1) / WARPS, rows * k);
    gate_up_kernel<FMT><<<g1, WARPS * 32, smem_gu, stream>>>(v, (const __nv_bfloat16*)x, slots, gate_w, k, limit, numerics, hidden, status);
    rc = check_launch("moe_decode gate_up");
    if (rc) return rc;
  }
  if (mx_hidden) {
    rc = launch_mxfp4_roundtrip_f32(hidden, (long long)rows * k, I, stream);
    if (rc) return rc;
  }
  if (!do_down) return rc;
  dim3 g2((H + WARPS - 1) / WARPS, rows);
  if (out_dtype == CACHALOT_BF16)
    down_kernel<FMT, __nv_bfloat16><<<g2, WARPS * 32, smem_dn, stream>>>(v, hidden, slots, k, numerics, (__nv_bfloat16*)out);
  else
    down_kernel<FMT, float><<<g2, WARPS * 32, smem_dn, stream>>>(v, hidden, slots, k, numerics, (float*)out);
  return check_launch("moe_decode down");
}

}  // namespace cachalot

using namespace cachalot;

#ifndef CB_FUSED_PER_TOKEN_MAX_ROWS
#define CB_FUSED_PER_TOKEN_MAX_ROWS 64
#endif
static constexpr int FUSED_PER_TOKEN_MAX_ROWS = CB_FUSED_PER_TOKEN_MAX_ROWS;

// FP4 bank, fp32 numerics, from this many tokens: rows grouped by expert on the block-scaled tensor cores, every distinct
// expert streamed once (below it, one single-launch kernel per token is faster)
#ifndef CB_GROUPED_TC_MIN_ROWS
#define CB_GROUPED_TC_MIN_ROWS 8
#endif
static int grouped_tc_min_rows() {  // CACHALOT_GROUPED_MIN_ROWS overrides the built-in threshold (for measurements)
  static const int v = [] {
    const char* e = std::getenv("CACHALOT_GROUPED_MIN_ROWS");
    const int n = e ? std::atoi(e) : 0;
    return n > 0 ? n : CB_GROUPED_TC_MIN_ROWS;
  }();
  return v;
}
#define GROUPED_TC_MIN_ROWS grouped_tc_min_rows()

extern "C" size_t cachalot_moe_decode_workspace_bytes(const cachalot_bank_desc* desc, int rows, int k) {
  if (!desc || rows <= 0 || k <= 0) return 0;
  const size_t a = decode_mma_workspace_bytes(desc->hidden, desc->inter, rows, k);  // >= the simple kernels' rows*k*inter floats
  const size_t b = decode_fused_workspace_bytes(desc->hidden, desc->inter, rows, k);
  size_t c = 0;
  if (desc->format == CACHALOT_BANK_FP4 && rows >= GROUPED_TC_MIN_ROWS && (long long)rows * k <= 1024)
    c = decode_tc_workspace_bytes(desc->hidden, desc->inter, rows, k);
  const size_t m = a > b ? a : b;
  return m > c ? m : c;
}

extern "C" int cachalot_moe_decode(const void* bank, const cachalot_bank_desc* desc, const void* x_bf16,
                                   const int32_t* slots, const float* gate_w, int rows, int k, float swiglu_limit,
                                   int numerics, void* workspace, size_t workspace_bytes, void* out, int out_dtype,
                                   int* status, cachalot_stream_t stream) {
  BankView v;
  int rc = make_view(bank, desc, &v, "moe_decode");
  if (rc) return rc;
  if (!x_bf16 || !slots || !gate_w || !out) return fail(CACHALOT_EINVAL, "moe_decode: null pointer");
  if (rows < 0 || k <= 0 || k > 64) return fail(CACHALOT_EINVAL, "moe_decode: rows=%d k=%d out of range", rows, k);
  if ((long long)rows * k > 65535) return fail(CACHALOT_EINVAL, "moe_decode: rows*k=%lld exceeds 65535", (long long)rows * k);
  if ((numerics & 0xff) > CACHALOT_NUMERICS_BF16_H32 || (numerics & ~0xfff))
    return fail(CACHALOT_EINVAL, "moe_decode: unknown numerics %d", numerics);
  if (out_dtype != CACHALOT_F32 && out_dtype != CACHALOT_BF16) return fail(CACHALOT_EINVAL, "moe_decode: out dtype must be f32 or bf16");
  if (rows == 0) return CACHALOT_OK;
  size_t need = cachalot_moe_decode_workspace_bytes(desc, rows, k);
  if (!workspace || workspace_bytes < need) return fail(CACHALOT_ESCRATCH, "moe_decode: workspace %zu < %zu bytes", workspace_bytes, need);
  if (!aligned(workspace, 256) || !aligned(x_bf16, 16) || !aligned(out, 4)) return fail(CACHALOT_EALIGN, "moe_decode: workspace needs 256-byte, x 16-byte alignment");
  const bool fused_ok = !(numerics & (CACHALOT_DECODE_SIMPLE | CACHALOT_DECODE_UNFUSED | CACHALOT_DECODE_ONLY_GATE_UP | CACHALOT_DECODE_ONLY_DOWN));
  if (fused_ok && decode_fused_supported(v, rows, k))
    return launch_decode_fused(v, x_bf16, slots, gate_w, rows, k, swiglu_limit, numerics, workspace, out, out_dtype, status, (cudaStream_t)stream);
  if (fused_ok && rows >= GROUPED_TC_MIN_ROWS && v.format == CACHALOT_BANK_FP4 && decode_tc_supported(v, rows, k) &&
      ((numerics & 0xff) == CACHALOT_NUMERICS_F32 || (numerics & 0xff) == CACHALOT_NUMERICS_BF16))
    return launch_decode_tc(v, x_bf16, slots, gate_w, rows, k, swiglu_limit, workspace, out, out_dtype, status, (cudaStream_t)stream,
                            (numerics & 0xff) == CACHALOT_NUMERICS_BF16);
  // Up to 64 tokens: one single-launch kernel per token, back to back.  Tokens share few experts at these sizes (384
  // routed rows touch about 244 of 384 experts), so grouping rows by expert saves less than the per-token kernel
  // gains by streaming its experts about twice as fast as the grouped kernels (measured: FP4 bank, 8 tokens 0.29 ms
  // per layer against 0.64 ms, 64 tokens 2.24 ms against 2.98 ms).
  // The 2-bit bank has no grouped kernel that beats the per-token one at any row count (measured up to 4096 tokens:
  // 21-25 us per token against ~100 us per token on the grouped and the one-warp-per-output kernels).
  if (fused_ok && (rows <= FUSED_PER_TOKEN_MAX_ROWS || v.format == CACHALOT_BANK_AFFINE) && decode_fused_supported(v, 1, k)) {
    const size_t out_row = (size_t)v.hidden * (out_dtype == CACHALOT_BF16 ? 2 : 4);
    for (int r = 0; r < rows; ++r) {
      rc = launch_decode_fused(v, static_cast<const __nv_bfloat16*>(x_bf16) + (size_t)r * v.hidden, slots + (size_t)r * k,
                               gate_w + (size_t)r * k, 1, k, swiglu_limit, numerics, workspace, static_cast<uint8_t*>(out) + r * out_row,
                               out_dtype, status, (cudaStream_t)stream);
      if (rc) return rc;
    }
    return CACHALOT_OK;
  }
  if (!(numerics & CACHALOT_DECODE_SIMPLE) && decode_mma_supported(v, rows, k))
    return launch_decode_mma(v, x_bf16, slots, gate_w, rows, k, swiglu_limit, numerics, workspace, out, out_dtype, status, (cudaStream_t)stream);
  if (desc->format == CACHALOT_BANK_FP4)
    return launch_decode<CACHALOT_BANK_FP4>(v, x_bf16, slots, gate_w, rows, k, swiglu_limit, numerics, (float*)workspace, out, out_dtype, status, (cudaStream_t)stream);
  return launch_decode<CACHALOT_BANK_AFFINE>(v, x_bf16, slots, gate_w, rows, k, swiglu_limit, numerics, (float*)workspace, out, out_dtype, status, (cudaStream_t)stream);
}

// ---- decode layer: routing tail + routed experts in one call --------------------------------------

extern "C" size_t cachalot_moe_layer_decode_workspace_bytes(const cachalot_bank_desc* desc, int k) {
  if (!desc || k <= 0) return 0;
  return cachalot_moe_decode_workspace_bytes(desc, 1, k) + 1024;  // + indices, weights, slots of the two-call path
}

extern "C" int cachalot_moe_layer_decode(const void* bank, const cachalot_bank_desc* desc, const void* x_bf16,
                                         const float* logits, const float* bias, const int32_t* slot_table, int layer,
                                         int n_experts, int k, int mode, float gate_temp, float route_scale,
                                         int norm_topk_prob, int weights_bf16, float swiglu_limit, int numerics,
                                         void* workspace, size_t workspace_bytes, void* out, int out_dtype,
                                         int32_t* indices_out, float* weights_out, int* status, cachalot_stream_t stream) {
  BankView v;
  int rc = make_view(bank, desc, &v, "moe_layer_decode");
  if (rc) return rc;
  if (!x_bf16 || !logits || !out) return fail(CACHALOT_EINVAL, "moe_layer_decode: null pointer");
  if (n_experts <= 0 || n_experts > 1024) return fail(CACHALOT_EINVAL, "moe_layer_decode: E=%d must be in 1..1024", n_experts);
  if (k < 1 || k > n_experts || k > 32) return fail(CACHALOT_EINVAL, "Invalid topk=%d for %d experts", k, n_experts);
  if (mode != CACHALOT_ROUTER_SQRT_SOFTPLUS && mode != CACHALOT_ROUTER_SIGMOID)
    return fail(CACHALOT_EINVAL, "moe_layer_decode: unknown router mode %d", mode);
  if (layer < 0) return fail(CACHALOT_EINVAL, "moe_layer_decode: bad layer");
  if ((numerics & 0xff) > CACHALOT_NUMERICS_BF16_H32 || (numerics & ~0xfff)) return fail(CACHALOT_EINVAL, "moe_layer_decode: unknown numerics %d", numerics);
  if (out_dtype != CACHALOT_F32 && out_dtype != CACHALOT_BF16) return fail(CACHALOT_EINVAL, "moe_layer_decode: out dtype must be f32 or bf16");
  const size_t need = cachalot_moe_layer_decode_workspace_bytes(desc, k);
  if (!workspace || workspace_bytes < need) return fail(CACHALOT_ESCRATCH, "moe_layer_decode: workspace %zu < %zu bytes", workspace_bytes, need);
  if (!aligned(workspace, 256) || !aligned(x_bf16, 16) || !aligned(out, 4)) return fail(CACHALOT_EALIGN, "moe_layer_decode: workspace needs 256-byte, x 16-byte alignment");
  cudaStream_t s = (cudaStream_t)stream;
  if (!(numerics & (CACHALOT_DECODE_SIMPLE | CACHALOT_DECODE_UNFUSED)) && layer_fused_supported(v, n_experts, k))
    return launch_layer_fused(v, x_bf16, logits, bias, slot_table, layer, n_experts, k, mode, gate_temp, route_scale, norm_topk_prob,
                              weights_bf16, swiglu_limit, numerics, workspace, out, out_dtype, indices_out, weights_out, status, s);
  // two calls: the routing kernel, then the experts
  uint8_t* tail = static_cast<uint8_t*>(workspace) + (need - 1024);
  int32_t* idx = indices_out ? indices_out : reinterpret_cast<int32_t*>(tail);
  float* w = weights_out ? weights_out : reinterpret_cast<float*>(tail + 256);
  int32_t* slots = reinterpret_cast<int32_t*>(tail + 512);
  rc = cachalot_route_topk(logits, bias, slot_table, layer, 1, n_experts, k, mode, gate_temp, route_scale, norm_topk_prob,
                           weights_bf16, idx, w, slots, nullptr, stream);
  if (rc) return rc;
  return cachalot_moe_decode(bank, desc, x_bf16, slots, w, 1, k, swiglu_limit, numerics, workspace, need - 1024, out, out_dtype,
                             status, stream);
}

extern "C" size_t cachalot_peer_layer_inbox_bytes(int world, int hidden) { return (size_t)2 * world * hidden * sizeof(unsigned long long); }

extern "C" int cachalot_moe_layer_decode_peer(const void* bank, const cachalot_bank_desc* desc, const void* x_bf16,
                                              const float* logits, const float* bias, const int32_t* slot_table, int layer,
                                              int n_experts, int k, int mode, float gate_temp, float route_scale,
                                              int norm_topk_prob, int weights_bf16, float swiglu_limit, int numerics,
                                              void* workspace, size_t workspace_bytes, void* out, int out_dtype,
                                              int32_t* indices_out, float* weights_out, const cachalot_peer_ctx* peer,
                                              int* status, cachalot_stream_t stream) {
  BankView v;
  int rc = make_view(bank, desc, &v, "moe_layer_decode_peer");
  if (rc) return rc;
  if (!x_bf16 || !logits || !out || !peer) return fail(CACHALOT_EINVAL, "moe_layer_decode_peer: null pointer");
  if (peer->world < 1 || peer->world > PEER_LINK_MAX || peer->rank < 0 || peer->rank >= peer->world || !peer->epoch)
    return fail(CACHALOT_EINVAL, "moe_layer_decode_peer: world %d (1..%d), rank %d", peer->world, PEER_LINK_MAX, peer->rank);
  if (n_experts <= 0 || n_experts > 1024) return fail(CACHALOT_EINVAL, "moe_layer_decode_peer: E=%d must be in 1..1024", n_experts);
  if (k < 1 || k > n_experts) return fail(CACHALOT_EINVAL, "Invalid topk=%d for %d experts", k, n_experts);
  if (mode != CACHALOT_ROUTER_SQRT_SOFTPLUS && mode != CACHALOT_ROUTER_SIGMOID) return fail(CACHALOT_EINVAL, "moe_layer_decode_peer: unknown router mode %d", mode);
  if (layer < 0) return fail(CACHALOT_EINVAL, "moe_layer_decode_peer: bad layer");
  if ((numerics & 0xff) > CACHALOT_NUMERICS_BF16_H32 || (numerics & ~0xff)) return fail(CACHALOT_EINVAL, "moe_layer_decode_peer: unknown numerics %d", numerics);
  if (out_dtype != CACHALOT_F32 && out_dtype != CACHALOT_BF16) return fail(CACHALOT_EINVAL, "moe_layer_decode_peer: out dtype must be f32 or bf16");
  const size_t need = cachalot_moe_layer_decode_workspace_bytes(desc, k);
  if (!workspace || workspace_bytes < need) return fail(CACHALOT_ESCRATCH, "moe_layer_decode_peer: workspace %zu < %zu bytes", workspace_bytes, need);
  if (!aligned(workspace, 256) || !aligned(x_bf16, 16) || !aligned(out, 4)) return fail(CACHALOT_EALIGN, "moe_layer_decode_peer: workspace needs 256-byte, x 16-byte alignment");
  if (!layer_fused_supported(v, n_experts, k))
    return fail(CACHALOT_EUNSUPPORTED, "moe_layer_decode_peer: the single-launch kernel does not cover this bank shape or top-k; use cachalot_moe_layer_decode and cachalot_peer_sum");
  PeerLink P = {};
  for (int r = 0; r < peer->world; ++r) {
    P.inbox[r] = static_cast<unsigned long long*>(peer->inbox[r]);
    if (!P.inbox[r] || !aligned(P.inbox[r], 16)) return fail(CACHALOT_EINVAL, "moe_layer_decode_peer: rank %d's inbox pointer is null or misaligned", r);
  }
  P.epoch = peer->epoch, P.world = peer->world, P.rank = peer->rank;
  return launch_layer_fused(v, x_bf16, logits, bias, slot_table, layer, n_experts, k, mode, gate_temp, route_scale, norm_topk_prob,
                            weights_bf16, swiglu_limit, numerics, workspace, out, out_dtype, indices_out, weights_out, status,
                            (cudaStream_t)stream, &P);
}

// ---- prefill -------------------------------------------------------------------------------

namespace cachalot {

// slots[t*k+j] = slot_of_expert[ids-by-row]; the row's expert id is recovered from the grouping:
// row perm[p] belongs to expert e for offsets[e] <= p < offsets[e+1]
__global__ void rows_to_slots_kernel(const int32_t* __restrict__ perm, const int32_t* __restrict__ offsets,
                                     const int32_t* __restrict__ slot_of_expert, int n_experts,
                                     int32_t* __restrict__ slots) {
  const int e = blockIdx.x;
  const int s = slot_of_expert ? slot_of_expert[e] : e;
  for (int p = offsets[e] + threadIdx.x; p < offsets[e + 1]; p += blockDim.x) slots[perm[p]] = s;
}

__global__ void fill_i32_kernel(int32_t* p, int n, int32_t v) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] = v;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

}  // namespace cachalot

extern "C" size_t cachalot_moe_prefill_workspace_bytes(const cachalot_bank_desc* desc, int tokens, int k,
                                                       int mxfp4_act) {
  if (!desc || tokens <= 0 || k <= 0) return 0;
  size_t rows = (size_t)tokens * k;
  // the tensor-core path (what prefill_tc_supported() accepts, stated on the descriptor) needs its own scratch only
  const bool tc_shape = desc->format == CACHALOT_BANK_FP4 && desc->hidden % 128 == 0 && desc->inter % 64 == 0 && desc->record_bytes % 16 == 0;
  if (mxfp4_act == 1 && tc_shape) return prefill_tc_workspace_bytes(desc->hidden, desc->inter, tokens, k, tokens * k);
  // bf16 activations on the same kernels (residual MXFP4 rows); the caller's expert count is not known here, and a
  // segment list never has more entries than routed rows plus the 8192 experts the grouping accepts
  if (mxfp4_act == 0 && tc_shape) return prefill_exact_workspace_bytes(desc->hidden, desc->inter, tokens, k, 8192);
  size_t b = align_up(rows * desc->inter * sizeof(float), 256);   // hidden
  b += align_up(rows * sizeof(int32_t), 256);                     // slot per routed row
  if (mxfp4_act) b += align_up((size_t)tokens * desc->hidden * 2, 256);  // MXFP4-rounded x as bf16
  if (mxfp4_act == 1 && desc->format == CACHALOT_BANK_FP4) {
    // experts without rows get no unit, so the unit list is bounded by the rows whatever the number of experts is
    const size_t tc = prefill_tc_workspace_bytes(desc->hidden, desc->inter, tokens, k, tokens * k);
    if (tc > b) b = tc;
  }
  return b;
}

extern "C" int cachalot_moe_prefill(const void* bank, const cachalot_bank_desc* desc, const void* x_bf16,
                                    const int32_t* perm, const int32_t* offsets, const int32_t* slot_of_expert,
                                    const float* gate_w, int tokens, int k, int n_experts, float swiglu_limit,
                                    int mxfp4_act, void* workspace, size_t workspace_bytes, float* out, int* status,
                                    cachalot_stream_t stream) {
  BankView v;
  int rc = make_view(bank, desc, &v, "moe_prefill");
  if (rc) return rc;
  if (tokens < 0 || k <= 0 || n_experts <= 0) return fail(CACHALOT_EINVAL, "moe_prefill: bad shape");
  if (tokens == 0) return CACHALOT_OK;  // an empty chunk: nothing to read or write
  if (!x_bf16 || !perm || !offsets || !gate_w || !out) return fail(CACHALOT_EINVAL, "moe_prefill: null pointer");
  const bool tc = (mxfp4_act == 1 || mxfp4_act == 0) && prefill_tc_supported(v);
  if (tc && mxfp4_act == 0 && n_experts > 8192) return fail(CACHALOT_EUNSUPPORTED, "moe_prefill: more than 8192 experts");
  if ((long long)tokens * k > 0x7fffffffLL) return fail(CACHALOT_EINVAL, "moe_prefill: tokens*k=%lld is too large", (long long)tokens * k);
  // the per-row kernels index routed rows in a grid dimension; the tensor-core path has no such limit
  if (!tc && (long long)tokens * k > 65535) return fail(CACHALOT_EINVAL, "moe_prefill: tokens*k=%lld exceeds 65535 (chunk the prompt)", (long long)tokens * k);
  size_t need = cachalot_moe_prefill_workspace_bytes(desc, tokens, k, mxfp4_act);
  if (!workspace || workspace_bytes < need) return fail(CACHALOT_ESCRATCH, "moe_prefill: workspace %zu < %zu bytes", workspace_bytes, need);
  if (!aligned(workspace, 256)) return fail(CACHALOT_EALIGN, "moe_prefill: workspace must be 256-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const size_t rows = (size_t)tokens * k;
  if (tc && mxfp4_act == 0)
    return launch_prefill_exact(v, x_bf16, perm, offsets, slot_of_expert, gate_w, tokens, k, n_experts, swiglu_limit, workspace, out, status, s);
  if (tc)
    return launch_prefill_tc(v, x_bf16, perm, offsets, slot_of_expert, gate_w, tokens, k, n_experts, swiglu_limit, workspace, out,
                             status, s);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  float* hidden = reinterpret_cast<float*>(ws);
  ws += align_up(rows * desc->inter * sizeof(float), 256);
  int32_t* slots = reinterpret_cast<int32_t*>(ws);
  ws += align_up(rows * sizeof(int32_t), 256);
  const void* x_in = x_bf16;
  if (mxfp4_act) {
    __nv_bfloat16* xq = reinterpret_cast<__nv_bfloat16*>(ws);
    rc = launch_mxfp4_roundtrip_bf16((const __nv_bfloat16*)x_bf16, xq, tokens, desc->hidden, s);
    if (rc) return rc;
    x_in = xq;
  }
  // rows whose expert id was dropped by the grouping stay at -1 and contribute zeros
  fill_i32_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, s>>>(slots, (int)rows, -1);
  rows_to_slots_kernel<<<n_experts, 128, 0, s>>>(perm, offsets, slot_of_expert, n_experts, slots);
  rc = check_launch("moe_prefill slots");
  if (rc) return rc;
  const int num = mxfp4_act ? CACHALOT_NUMERICS_BF16_H32 : CACHALOT_NUMERICS_BF16;
  // bf16 activations where no tensor-core path exists (the 2-bit bank): the single-launch kernel, token by token - a
  // quarter of the time of the one-warp-per-output kernels (86 ms against 400 ms for 4096 tokens at 4096 x 2880)
  if (!mxfp4_act && decode_fused_supported(v, 1, k)) {
    for (int r = 0; r < tokens; ++r) {
      rc = launch_decode_fused(v, static_cast<const __nv_bfloat16*>(x_in) + (size_t)r * v.hidden, slots + (size_t)r * k, gate_w + (size_t)r * k, 1,
                               k, swiglu_limit, num, hidden, out + (size_t)r * v.hidden, CACHALOT_F32, status, s);
      if (rc) return rc;
    }
    return CACHALOT_OK;
  }
  if (desc->format == CACHALOT_BANK_FP4)
    return launch_decode<CACHALOT_BANK_FP4>(v, x_in, slots, gate_w, tokens, k, swiglu_limit, num, hidden, out, CACHALOT_F32, status, s, mxfp4_act != 0);
  return launch_decode<CACHALOT_BANK_AFFINE>(v, x_in, slots, gate_w, tokens, k, swiglu_limit, num, hidden, out, CACHALOT_F32, status, s, mxfp4_act != 0);
}

extern "C" size_t cachalot_moe_prefill_rows_workspace_bytes(const cachalot_bank_desc* desc, long long rows, int n_segments) {
  if (!desc || rows <= 0 || n_segments <= 0) return 0;
  return prefill_rows_workspace_bytes(desc->inter, rows, n_segments);
}

extern "C" int cachalot_moe_prefill_rows(const void* bank, const cachalot_bank_desc* desc, const uint8_t* x_codes,
                                         const uint8_t* x_scales, const float* row_weights, const int32_t* seg_offsets,
                                         const int32_t* seg_slot, int n_segments, long long rows, float swiglu_limit,
                                         void* workspace, size_t workspace_bytes, void* y_bf16, int* status,
                                         cachalot_stream_t stream) {
  BankView v;
  int rc = make_view(bank, desc, &v, "moe_prefill_rows");
  if (rc) return rc;
  if (rows < 0 || n_segments < 0 || rows > 0x7fffffff) return fail(CACHALOT_EINVAL, "moe_prefill_rows: bad shape");
  if (rows == 0 || n_segments == 0) return CACHALOT_OK;
  if (!x_codes || !x_scales || !row_weights || !seg_offsets || !y_bf16) return fail(CACHALOT_EINVAL, "moe_prefill_rows: null pointer");
  if (!prefill_tc_supported(v))
    return fail(CACHALOT_EUNSUPPORTED, "moe_prefill_rows: needs an FP4 bank with hidden a multiple of 128 and inter a multiple of 64");
  if (!aligned(x_codes, 16)) return fail(CACHALOT_EALIGN, "moe_prefill_rows: x_codes must be 16-byte aligned");
  const size_t need = prefill_rows_workspace_bytes(v.inter, rows, n_segments);
  if (!workspace || workspace_bytes < need) return fail(CACHALOT_ESCRATCH, "moe_prefill_rows: workspace %zu < %zu bytes", workspace_bytes, need);
  if (!aligned(workspace, 256)) return fail(CACHALOT_EALIGN, "moe_prefill_rows: workspace must be 256-byte aligned");
  return launch_prefill_rows(v, x_codes, x_scales, row_weights, seg_offsets, seg_slot, n_segments, rows, swiglu_limit, true, workspace,
                             static_cast<__nv_bfloat16*>(y_bf16), status, (cudaStream_t)stream);
}

extern "C" int cachalot_moe_combine_rows(const void* y_bf16, const int32_t* inv, int tokens, int k, int hidden, float* out,
                                         cachalot_stream_t stream) {
  if (!y_bf16 || !inv || !out) return fail(CACHALOT_EINVAL, "moe_combine_rows: null pointer");
  if (tokens < 0 || k <= 0 || hidden <= 0 || hidden % 2) return fail(CACHALOT_EINVAL, "moe_combine_rows: bad shape");
  return launch_combine_rows(static_cast<const __nv_bfloat16*>(y_bf16), inv, tokens, k, hidden, out, (cudaStream_t)stream);
}

// ---- decode with built-in scratch (no allocation anywhere) ------------------------------------

namespace cachalot {
namespace {

constexpr size_t STATIC_SCRATCH_BYTES = (size_t)4 << 20;
// Scratch of cachalot_moe_decode_static.  Every GPU that loads the library carries these 4 MiB
// until the process exits.  In host code this name is only a handle for the runtime's symbol
// table; the device address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char static_scratch[STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
void* static_scratch_addr[MAX_DEVICES];  // per device ordinal; null until that device's first call
std::mutex static_scratch_mu;

}  // namespace
}  // namespace cachalot

extern "C" size_t cachalot_moe_decode_static_scratch_bytes(void) { return STATIC_SCRATCH_BYTES; }

extern "C" int cachalot_moe_decode_static(const void* bank, const cachalot_bank_desc* desc, const void* x_bf16,
                                          const int32_t* slots, const float* gate_w, int rows, int k,
                                          float swiglu_limit, int numerics, void* out, int out_dtype, int* status,
                                          cachalot_stream_t stream) {
  if (!desc) return fail(CACHALOT_EINVAL, "moe_decode_static: null bank descriptor");
  if (rows > 0 && k > 0) {
    const size_t need = cachalot_moe_decode_workspace_bytes(desc, rows, k);
    if (need > STATIC_SCRATCH_BYTES)
      return fail(CACHALOT_ESCRATCH,
                  "moe_decode_static: rows=%d k=%d needs %zu bytes of scratch but the built-in scratch holds %zu; "
                  "call cachalot_moe_decode with a workspace of your own",
                  rows, k, need, STATIC_SCRATCH_BYTES);
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(CACHALOT_ECUDA, "moe_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= MAX_DEVICES) return fail(CACHALOT_EUNSUPPORTED, "moe_decode_static: device ordinal %d", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(static_scratch_mu);
    scratch = static_scratch_addr[dev];
    if (!scratch) {  // set-up, once per device, with that device current
      e = cudaGetSymbolAddress(&scratch, static_scratch);
      if (e != cudaSuccess || !scratch)
        return fail(CACHALOT_ECUDA, "moe_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      static_scratch_addr[dev] = scratch;
    }
  }
  // Nothing in the scratch has to start at zero: the kernels reset their own arrival counters at
  // the start of every call and overwrite every intermediate they later read.
  return cachalot_moe_decode(bank, desc, x_bf16, slots, gate_w, rows, k, swiglu_limit, numerics, scratch,
                             STATIC_SCRATCH_BYTES, out, out_dtype, status, stream);
}
