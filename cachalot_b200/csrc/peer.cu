// Sum of the ranks' partial outputs over NVLink peer memory (expert-parallel decode): one launch per rank,
// no library collective.  Every rank owns an inbox in memory that its peers can write (the host maps it,
// e.g. through CUDA IPC or a symmetric allocation, and passes every rank's base pointer):
//
//   inbox  f32 [2 slots][world][n]      rank r's partial lands in row r of every peer's inbox
//   flags  u32 [2 slots][world][CTAS]   flag (r, cta) = number of the exchange whose row-r chunk `cta` is complete
//   epoch  u32                          number of exchanges this rank has done (kept on the device so that a
//                                       captured CUDA graph can be replayed)
//
// A CTA stores its chunk of the local partial into every inbox (plain peer stores), fences, raises its flag
// on every peer, waits (bounded) for the peers' flags for the same chunk, and adds the rows in rank order.
// Two slots are enough: a rank cannot start exchange e+2 before every peer has finished reading exchange e.
#include "kernels.cuh"

namespace cachalot {
namespace {

constexpr int PEER_MAX = 8;
constexpr int PEER_CTAS = 8;
constexpr int PEER_THREADS = 256;
constexpr uint32_t PEER_WAIT_LIMIT = 1u << 22;

struct PeerArgs {
  float* inbox[PEER_MAX];
  uint32_t* flags[PEER_MAX];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(PEER_THREADS)
peer_sum_kernel(PeerArgs P, int world, int rank, const float* __restrict__ partial, float* __restrict__ out, int n,
                uint32_t* __restrict__ epoch, int* __restrict__ status) {
  __shared__ int expired;
  const uint32_t e = *epoch + 1u;  // every CTA reads it before anyone can write it (see the end)
  const int slot = (int)(e & 1u);
  const int cta = blockIdx.x;
  const int per = ((n / 4 + PEER_CTAS - 1) / PEER_CTAS) * 4;  // floats per CTA, whole float4s
  const int lo = min(cta * per, n), hi = min(lo + per, n);
  if (threadIdx.x == 0) expired = 0;
  // 1. my chunk into row `rank` of every inbox
  for (int p = 0; p < world; ++p) {
    float* dst = P.inbox[p] + ((size_t)slot * world + rank) * n;
    for (int i = lo + threadIdx.x * 4; i < hi; i += PEER_THREADS * 4)
      *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(partial + i);
  }
  __threadfence_system();
  __syncthreads();
  // 2. tell every rank that chunk `cta` of row `rank` is there
  if ((int)threadIdx.x < world) st_release_sys(P.flags[threadIdx.x] + ((size_t)slot * world + rank) * PEER_CTAS + cta, e);
  // 3. wait for the same chunk of every row of my inbox
  if ((int)threadIdx.x < world) {
    const uint32_t* f = P.flags[rank] + ((size_t)slot * world + threadIdx.x) * PEER_CTAS + cta;
    uint32_t i = 0;
    while (ld_acquire_sys(f) != e) {
      if (++i >= PEER_WAIT_LIMIT) {
        expired = 1;
        break;
      }
      if (i > 64) __nanosleep(64);
    }
  }
  __syncthreads();
  if (expired && threadIdx.x == 0 && status) atomicOr(status, CACHALOT_STATUS_WAIT_EXPIRED);
  // 4. rows in rank order
  const float* mine = P.inbox[rank] + (size_t)slot * world * n;
  for (int i = lo + threadIdx.x * 4; i < hi; i += PEER_THREADS * 4) {
    // the rows were written by other GPUs: read them past L1, which may still hold this slot's lines of two exchanges ago
    float4 acc = __ldcg(reinterpret_cast<const float4*>(mine + i));
    for (int r = 1; r < world; ++r) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(mine + (size_t)r * n + i));
      acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
    }
    *reinterpret_cast<float4*>(out + i) = acc;
  }
  // the exchange counter moves on once: by the CTA that arrives last at a device-scope ticket
  __shared__ unsigned ticket;
  __syncthreads();
  if (threadIdx.x == 0) ticket = atomicAdd(epoch + 1, 1u);
  __syncthreads();
  if (ticket == (unsigned)(gridDim.x - 1) && threadIdx.x == 0) {
    epoch[1] = 0;
    __threadfence();
    epoch[0] = e;
  }
}

}  // namespace
}  // namespace cachalot

using namespace cachalot;

extern "C" size_t cachalot_peer_sum_inbox_bytes(int world, int n) { return (size_t)2 * world * n * sizeof(float); }
extern "C" size_t cachalot_peer_sum_flag_bytes(int world) { return (size_t)2 * world * PEER_CTAS * sizeof(uint32_t); }

extern "C" int cachalot_peer_sum(void* const* inbox_ptrs, void* const* flag_ptrs, int world, int rank, const float* partial,
                                 float* out, int n, uint32_t* epoch, int* status, cachalot_stream_t stream) {
  if (!inbox_ptrs || !flag_ptrs || !partial || !out || !epoch) return fail(CACHALOT_EINVAL, "peer_sum: null pointer");
  if (world < 1 || world > PEER_MAX || rank < 0 || rank >= world) return fail(CACHALOT_EINVAL, "peer_sum: world %d (1..%d), rank %d", world, PEER_MAX, rank);
  if (n <= 0 || n % 4) return fail(CACHALOT_EINVAL, "peer_sum: n=%d must be a positive multiple of 4", n);
  if (!aligned(partial, 16) || !aligned(out, 16)) return fail(CACHALOT_EALIGN, "peer_sum: partial and out must be 16-byte aligned");
  PeerArgs P;
  for (int r = 0; r < PEER_MAX; ++r) {
    P.inbox[r] = r < world ? static_cast<float*>(inbox_ptrs[r]) : nullptr;
    P.flags[r] = r < world ? static_cast<uint32_t*>(flag_ptrs[r]) : nullptr;
    if (r < world && (!P.inbox[r] || !P.flags[r] || !aligned(P.inbox[r], 16)))
      return fail(CACHALOT_EINVAL, "peer_sum: rank %d's inbox or flags pointer is null or misaligned", r);
  }
  peer_sum_kernel<<<PEER_CTAS, PEER_THREADS, 0, (cudaStream_t)stream>>>(P, world, rank, partial, out, n, epoch, status);
  return check_launch("peer_sum");
}
