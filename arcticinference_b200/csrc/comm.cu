// Cross-GPU synchronisation and reduction over peer-mapped (symmetric) memory.
//
// Every rank owns one symmetric heap; all ranks map all heaps. Data moves by plain
// peer stores / loads over NVLink issued from inside kernels (the GEMM and
// attention epilogues push their tiles straight into the consumer's heap; see
// gemm_bf16.cu and attention.cu). This file holds what those kernels need around
// them:
//
//   * barrier_kernel     -- flag exchange with release/acquire at system scope.
//     Flags are monotonically increasing epochs kept per source rank; the epoch
//     is a device-side counter, so a captured CUDA graph can replay the barrier.
//     Waits are bounded (2 s): on expiry the kernel records kErrPeerFlagTimeout
//     in the status word and returns.
//   * allreduce_kernel   -- one-shot sum of W peers' partial buffers (bf16 in,
//     fp32 accumulate in rank order 0..W-1 so that every rank produces the same
//     bits), optional residual add fused.
//   * gather_rows_peers  -- copies selected rows of a token-sliced tensor from
//     the ranks that own them (last-token gather of sequence-parallel mode).
//
// The reference reaches the same points with NCCL calls
// (arctic_inference/vllm/ulysses.py:436-455, vLLM row-parallel all-reduce).

#include "api.h"
#include "common/ptx.cuh"

namespace ab200 {

constexpr int kMaxPeers = 16;

struct PeerTable {
  void* ptr[kMaxPeers];
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// 16-byte load at system scope: data written by another GPU's kernel must not be served
// from a stale non-coherent cache line left by an earlier read of the same address.
__device__ __forceinline__ uint4 ld_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// flags: per rank an array unsigned[kMaxPeers] in its heap; flags.ptr[r] is rank r's array.
// Thread j publishes this rank's epoch into rank j's slot [my_rank] and then waits for
// rank j's epoch in the local slot [j].
__global__ void barrier_kernel(PeerTable flags, int my_rank, int world, unsigned int* epoch_ctr,
                               int* status, unsigned long long limit_ns) {
  __shared__ unsigned int epoch;
  if (threadIdx.x == 0) epoch = *epoch_ctr + 1;
  __syncthreads();
  const unsigned int e = epoch;
  const int j = threadIdx.x;
  if (j < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<unsigned int*>(flags.ptr[j]) + my_rank, e);
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(flags.ptr[my_rank]) + j;
    const unsigned long long t0 = globaltimer_ns();
    unsigned int spins = 0;
    while ((int)(ld_acquire_sys(mine) - e) < 0) {
      if ((++spins & 255u) == 0u && globaltimer_ns() - t0 > limit_ns) {
        report_error(status, kErrPeerFlagTimeout, j, (int)e);
        break;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *epoch_ctr = e;
}

// out[i] = sum_r part_r[i] (+ residual[i]); 8 bf16 per thread per iteration.
__global__ void __launch_bounds__(512)
allreduce_kernel(PeerTable parts, int world, __nv_bfloat16* __restrict__ out,
                 const __nv_bfloat16* __restrict__ residual, long long n_vec) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_vec;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    uint4 v[kMaxPeers];
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r)
      if (r < world) v[r] = ld_sys_v4(reinterpret_cast<const uint4*>(parts.ptr[r]) + i);
#pragma unroll
    for (int r = 0; r < kMaxPeers; ++r) {
      if (r < world) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[r]);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(h[k]);
          acc[2 * k] += f.x;
          acc[2 * k + 1] += f.y;
        }
      }
    }
    if (residual != nullptr) {
      const uint4 q = reinterpret_cast<const uint4*>(residual)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        acc[2 * k] += f.x;
        acc[2 * k + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// dst[r] = src_{owner(idx[r])}[idx[r] - owner*rows_per_rank], rows of `hidden` bf16.
__global__ void gather_rows_peers_kernel(PeerTable src, long long rows_per_rank,
                                         const long long* __restrict__ idx,
                                         __nv_bfloat16* __restrict__ dst, int hidden) {
  const long long r = blockIdx.x;
  const long long g = idx[r];
  const int owner = (int)(g / rows_per_rank);
  const long long local = g - owner * rows_per_rank;
  const uint4* s = reinterpret_cast<const uint4*>(
      reinterpret_cast<const __nv_bfloat16*>(src.ptr[owner]) + local * hidden);
  uint4* d = reinterpret_cast<uint4*>(dst + r * (long long)hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) d[i] = ld_sys_v4(s + i);
}

}  // namespace ab200

using namespace ab200;

extern "C" {

// peer_ptrs: host array of `world` device pointers.
int ab200_barrier(const void* const* flag_ptrs, int my_rank, int world, void* epoch_ctr,
                  int* status, cudaStream_t stream) {
  if (world < 1 || world > kMaxPeers) return -2;
  PeerTable t;
  for (int i = 0; i < kMaxPeers; ++i) t.ptr[i] = i < world ? const_cast<void*>(flag_ptrs[i]) : nullptr;
  barrier_kernel<<<1, 32, 0, stream>>>(t, my_rank, world,
                                       reinterpret_cast<unsigned int*>(epoch_ctr), status,
                                       kWaitLimitNs);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Same barrier with a caller-chosen wait limit (milliseconds). A rank whose peers never
// arrive leaves the kernel after the limit with kErrPeerFlagTimeout in the status word and a
// usable context: the host decides what to do about the missing peer.
int ab200_barrier_timed(const void* const* flag_ptrs, int my_rank, int world, void* epoch_ctr,
                        int limit_ms, int* status, cudaStream_t stream) {
  if (world < 1 || world > kMaxPeers || limit_ms < 1 || limit_ms > 60000) return -2;
  PeerTable t;
  for (int i = 0; i < kMaxPeers; ++i) t.ptr[i] = i < world ? const_cast<void*>(flag_ptrs[i]) : nullptr;
  barrier_kernel<<<1, 32, 0, stream>>>(t, my_rank, world,
                                       reinterpret_cast<unsigned int*>(epoch_ctr), status,
                                       (unsigned long long)limit_ms * 1000000ull);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_allreduce(const void* const* part_ptrs, int world, void* out, const void* residual,
                    long long n_elems, cudaStream_t stream) {
  if (world < 1 || world > kMaxPeers || (n_elems % 8)) return -2;
  if (n_elems == 0) return 0;
  PeerTable t;
  for (int i = 0; i < kMaxPeers; ++i) t.ptr[i] = i < world ? const_cast<void*>(part_ptrs[i]) : nullptr;
  const long long n_vec = n_elems / 8;
  long long blocks = (n_vec + 511) / 512;
  if (blocks > 148 * 2) blocks = 148 * 2;
  allreduce_kernel<<<(unsigned)blocks, 512, 0, stream>>>(
      t, world, reinterpret_cast<__nv_bfloat16*>(out),
      reinterpret_cast<const __nv_bfloat16*>(residual), n_vec);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_gather_rows_peers(const void* const* src_ptrs, int world, long long rows_per_rank,
                            const void* idx, void* dst, long long R, int hidden,
                            cudaStream_t stream) {
  if (world < 1 || world > kMaxPeers || (hidden % 8)) return -2;
  if (R <= 0) return 0;
  PeerTable t;
  for (int i = 0; i < kMaxPeers; ++i) t.ptr[i] = i < world ? const_cast<void*>(src_ptrs[i]) : nullptr;
  gather_rows_peers_kernel<<<(unsigned)R, 128, 0, stream>>>(
      t, rows_per_rank, reinterpret_cast<const long long*>(idx),
      reinterpret_cast<__nv_bfloat16*>(dst), hidden);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // extern "C"
