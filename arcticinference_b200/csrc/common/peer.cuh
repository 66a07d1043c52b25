// Peer-memory helpers shared by the kernels that talk to other GPUs: the table of the
// ranks' mapped pointers, system-scope loads / stores, and the flag barrier.
#pragma once

#include "ptx.cuh"

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

__device__ __forceinline__ void st_v4_global(void* p, const uint4& v) {
  asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// Flag barrier among `world` ranks, run by the first `world` threads of a block (the whole
// block must call it; it ends with __syncthreads, after which data the peers wrote before
// their own call is visible to every thread of the block).
// flags: per rank an array unsigned[kMaxPeers] in its heap; flags.ptr[r] is rank r's array.
// Thread j publishes this rank's epoch into rank j's slot [my_rank] and then waits for rank
// j's epoch in the local slot [j]. The epoch is a device-side counter, so a captured CUDA
// graph replays the barrier. The wait is bounded: on expiry kErrPeerFlagTimeout is recorded
// in the status word and the block carries on (returns false).
__device__ __forceinline__ bool flag_barrier(const PeerTable& flags, int my_rank, int world,
                                             unsigned int* epoch_ctr, int* status,
                                             unsigned long long limit_ns) {
  __shared__ unsigned int fb_epoch;
  __shared__ int fb_failed;
  __syncthreads();
  if (threadIdx.x == 0) {
    fb_epoch = *epoch_ctr + 1;
    fb_failed = 0;
  }
  __syncthreads();
  const unsigned int e = fb_epoch;
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
        fb_failed = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) *epoch_ctr = e;
  return fb_failed == 0;
}

}  // namespace ab200
