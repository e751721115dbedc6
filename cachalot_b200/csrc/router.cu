// Router kernels: fp32 gate logits and the top-k selection tail (both score functions).
#include "common.cuh"

namespace cachalot {

// one warp per (token row, expert): logits[r,e] = dot(x[r], W[e]) in fp32, lane-strided in k
// then a butterfly sum (the reduction shape of the reference's router_scores kernel).
template <typename W>
__global__ void router_logits_kernel(const __nv_bfloat16* __restrict__ x, const W* __restrict__ w, int rows,
                                     int n_experts, int hidden, float* __restrict__ logits) {
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  if (warp >= rows * n_experts) return;
  int r = warp / n_experts, e = warp - r * n_experts;
  const __nv_bfloat16* xr = x + (size_t)r * hidden;
  const W* wr = w + (size_t)e * hidden;
  float acc = 0.f;
  for (int k = lane; k < hidden; k += 32) {
    float wv;
    if constexpr (sizeof(W) == 2)
      wv = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(wr)[k]);
    else
      wv = reinterpret_cast<const float*>(wr)[k];
    acc = fmaf(__bfloat162float(xr[k]), wv, acc);
  }
  acc = warp_sum(acc);
  if (lane == 0) logits[warp] = acc;
}

// One CTA per token row, one thread per expert (E <= 1024).  Every expert counts how many
// others beat it under a strict total order, which gives its rank; the first k ranks are the
// selection.  The order encodes the reference's tie rules:
//   SQRT_SOFTPLUS: higher score+bias first, ties to the LARGER index; written weakest-first
//   SIGMOID:       lower -(s+bias) first,   ties to the LOWER index;  written strongest-first
__global__ void route_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                  const int32_t* __restrict__ slot_table, int layer, int n_experts, int k, int mode,
                                  float gate_temp, float route_scale, int norm, int weights_bf16,
                                  int32_t* __restrict__ indices, float* __restrict__ weights,
                                  int32_t* __restrict__ slots, float* __restrict__ scores_out) {
  extern __shared__ float sm[];
  float* key = sm;                  // selection key per expert
  float* score = sm + n_experts;    // score per expert
  __shared__ int top[32];
  const int row = blockIdx.x;
  const int t = threadIdx.x;
  float my_key = 0.f, my_score = 0.f;
  if (t < n_experts) {
    float raw = logits[(size_t)row * n_experts + t];
    float b = bias ? bias[t] : 0.f;
    router_score_key(mode, raw, b, gate_temp, my_score, my_key);
    key[t] = my_key;
    score[t] = my_score;
    if (scores_out) scores_out[(size_t)row * n_experts + t] = my_score;
  }
  __syncthreads();
  if (t < n_experts) {
    int rank = 0;
    if (mode == CACHALOT_ROUTER_SQRT_SOFTPLUS) {
      for (int j = 0; j < n_experts; ++j) {
        float o = key[j];
        rank += (o > my_key || (o == my_key && j > t)) ? 1 : 0;
      }
    } else {
      for (int j = 0; j < n_experts; ++j) {
        float o = key[j];
        rank += (o < my_key || (o == my_key && j < t)) ? 1 : 0;
      }
    }
    if (rank < k) top[mode == CACHALOT_ROUTER_SQRT_SOFTPLUS ? k - 1 - rank : rank] = t;
  }
  __syncthreads();
  if (t < k) {
    // one thread per selected expert (the slot lookups are independent loads); every thread adds the
    // scores up in output order, as both reference kernels do, so all of them hold the same total
    float total = 0.f;
    for (int r = 0; r < k; ++r) total += score[top[r]];
    const float den = total + 1e-20f;
    const int e = top[t];
    float w = score[e];
    if (mode == CACHALOT_ROUTER_SIGMOID) {
      w = (w / den) * route_scale;
    } else {
      if (norm && k > 1) w = w / den;
      w = w * route_scale;
    }
    if (weights_bf16) w = bf16_round(w);
    indices[(size_t)row * k + t] = e;
    weights[(size_t)row * k + t] = w;
    if (slots) slots[(size_t)row * k + t] = slot_table ? slot_table[(size_t)layer * n_experts + e] : e;
  }
}

}  // namespace cachalot

using namespace cachalot;

extern "C" int cachalot_router_logits(const void* x_bf16, const void* gate_w, int w_dtype, int rows, int n_experts,
                                      int hidden, float* logits, cachalot_stream_t stream) {
  if (!x_bf16 || !gate_w || !logits) return fail(CACHALOT_EINVAL, "router_logits: null pointer");
  if (rows < 0 || n_experts <= 0 || hidden <= 0) return fail(CACHALOT_EINVAL, "router_logits: bad shape");
  if (rows == 0) return CACHALOT_OK;
  long long warps = (long long)rows * n_experts;
  int threads = 256;
  unsigned blocks = (unsigned)((warps * 32 + threads - 1) / threads);
  if (w_dtype == CACHALOT_BF16)
    router_logits_kernel<__nv_bfloat16><<<blocks, threads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x_bf16, (const __nv_bfloat16*)gate_w, rows, n_experts, hidden, logits);
  else if (w_dtype == CACHALOT_F32)
    router_logits_kernel<float><<<blocks, threads, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x_bf16, (const float*)gate_w, rows, n_experts, hidden, logits);
  else
    return fail(CACHALOT_EINVAL, "router_logits: gate weight dtype must be bf16 or f32");
  return check_launch("router_logits");
}

extern "C" int cachalot_route_topk(const float* logits, const float* bias, const int32_t* slot_table, int layer,
                                   int rows, int n_experts, int k, int mode, float gate_temp, float route_scale,
                                   int norm_topk_prob, int weights_bf16, int32_t* indices, float* weights,
                                   int32_t* slots, float* scores, cachalot_stream_t stream) {
  if (!logits || !indices || !weights) return fail(CACHALOT_EINVAL, "route_topk: null pointer");
  if (n_experts <= 0 || n_experts > 1024) return fail(CACHALOT_EINVAL, "route_topk: E=%d must be in 1..1024", n_experts);
  if (k < 1 || k > n_experts || k > 32) return fail(CACHALOT_EINVAL, "Invalid topk=%d for %d experts", k, n_experts);
  if (mode != CACHALOT_ROUTER_SQRT_SOFTPLUS && mode != CACHALOT_ROUTER_SIGMOID)
    return fail(CACHALOT_EINVAL, "route_topk: unknown mode %d", mode);
  if (rows < 0 || layer < 0) return fail(CACHALOT_EINVAL, "route_topk: bad rows/layer");
  if (rows == 0) return CACHALOT_OK;
  int threads = ((n_experts + 31) / 32) * 32;
  size_t smem = 2 * (size_t)n_experts * sizeof(float);
  route_topk_kernel<<<rows, threads, smem, (cudaStream_t)stream>>>(logits, bias, slot_table, layer, n_experts, k, mode,
                                                                  gate_temp, route_scale, norm_topk_prob, weights_bf16,
                                                                  indices, weights, slots, scores);
  return check_launch("route_topk");
}
