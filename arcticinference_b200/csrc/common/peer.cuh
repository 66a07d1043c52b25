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

// ---------------------------------------------------------------------------------------------
// One-way completion signal between a producer kernel and the consumer kernels of other ranks.
//
// A producer kernel whose blocks store into peers' memory (a scatter epilogue) or whose output
// the peers will read ends with tail_signal(): each block counts itself done after a
// system-scope fence, and the block that finds itself last bumps this rank's epoch counter
// and stores the new epoch into its slot [my_rank] of every rank's arrival words. A consumer
// kernel that follows the rank's own producer in the stream calls wait_peers(): the epoch to
// wait for is the value the local producer left in the epoch counter (all ranks issue the
// same sequence of kernels, so the producers' epochs agree), and every rank's slot must have
// reached it. The wait is bounded like every other wait in this library. Compared with a
// barrier kernel between the two there is no launch of its own, no second direction, and a
// consumer block that starts after the signals arrived pays W loads.
//
// Arrival words and counters live in the symmetric heap, one set per kind of exchange
// ("channel"), so that two exchanges in flight do not share epochs.
struct TailSignal {
  unsigned int* flags[kMaxPeers];  // flags[r]: rank r's arrival words of this channel
  unsigned int* done_ctr;          // this rank: blocks that have finished (returns to 0)
  unsigned int* epoch_ctr;         // this rank: number of signals sent
  int my_rank;
  int world;                       // 0: no signal
};

// Every thread of every block calls this after the block's last global store.
__device__ __forceinline__ void tail_signal(const TailSignal& s, unsigned int total_blocks) {
  if (s.world <= 0) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();   // this block's stores, local and remote, before its count
    const unsigned int prev = atomicAdd(s.done_ctr, 1u);
    if (prev + 1u == total_blocks) {
      *s.done_ctr = 0u;
      const unsigned int e = *s.epoch_ctr + 1u;
      *s.epoch_ctr = e;
      __threadfence_system();
      for (int w = 0; w < s.world; ++w) {
        int peer = s.my_rank + w;
        if (peer >= s.world) peer -= s.world;
        st_release_sys(s.flags[peer] + s.my_rank, e);
      }
    }
  }
}

struct PeerWait {
  const unsigned int* flags;      // this rank's arrival words of the channel
  const unsigned int* epoch_ctr;  // this rank's epoch counter of the channel
  int world;                      // 0: nothing to wait for
};

// Called by (at least) the first `world` threads of a warp, all lanes converged. Returns false
// when a peer did not arrive in time (the status word then holds kErrPeerFlagTimeout).
__device__ __forceinline__ bool wait_peers(const PeerWait& w, int* status,
                                           unsigned long long limit_ns) {
  bool ok = true;
  const int j = threadIdx.x & 31;
  if (w.world > 0 && j < w.world) {
    const unsigned int e = *reinterpret_cast<const volatile unsigned int*>(w.epoch_ctr);
    const unsigned long long t0 = globaltimer_ns();
    unsigned int spins = 0;
    while ((int)(ld_acquire_sys(w.flags + j) - e) < 0) {
      if ((++spins & 255u) == 0u && globaltimer_ns() - t0 > limit_ns) {
        report_error(status, kErrPeerFlagTimeout, j, (int)e);
        ok = false;
        break;
      }
    }
  }
  return __all_sync(0xffffffffu, ok);
}

// Orders the asynchronous proxy (TMA) after this thread's generic-proxy acquire: data that
// peers stored with ordinary stores is then safe to fetch with bulk tensor copies.
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

}  // namespace ab200
