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
//
// The reference reaches the same points with NCCL calls
// (arctic_inference/vllm/ulysses.py:436-455, vLLM row-parallel all-reduce).

#include "api.h"
#include "common/peer.cuh"
#include "common/ptx.cuh"

namespace ab200 {

// flags: per rank an array unsigned[kMaxPeers] in its heap; flags.ptr[r] is rank r's array.
// Thread j publishes this rank's epoch into rank j's slot [my_rank] and then waits for
// rank j's epoch in the local slot [j].
__global__ void barrier_kernel(PeerTable flags, int my_rank, int world, unsigned int* epoch_ctr,
                               int* status, unsigned long long limit_ns) {
  flag_barrier(flags, my_rank, world, epoch_ctr, status, limit_ns);
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

// Two-shot all-reduce in one launch: reduce-scatter by peer loads, all-gather by peer stores.
//
// Rank r owns slice r of the vector (n_vec / world 16-byte pieces, rounded up). Block b of
// every rank works on the same positions of its rank's slice, so blocks pair up across ranks
// and synchronise among themselves only:
//   A. block b tells every peer that this rank's partial product is complete (it is: the
//      producing GEMM precedes this kernel in the stream) and waits for the same word from
//      every peer's block b;
//   B. it sums its pieces of the slice over all ranks' partials (fp32, rank order 0..W-1, so
//      every element is reduced by exactly one rank and all ranks hold the same bits) and
//      stores the bf16 result into every rank's result buffer;
//   C. it publishes a second flag and waits for every peer's block b: after that the pieces
//      the peers' blocks b own have landed in this rank's result buffer.
// Per rank (W-1)/W of the vector crosses NVLink in each direction, against (W-1) times the
// vector for the one-shot kernel. Flags are epochs from a per-block device-side counter (a
// captured graph replays them); waits are bounded and record kErrPeerFlagTimeout.
//
// flags layout per rank: unsigned[2][kMaxPeers][kMaxArBlocks], slot [phase][source rank][block].
constexpr int kMaxArBlocks = 128;

__device__ __forceinline__ bool exchange_flags(const PeerTable& flags, int phase, int my_rank,
                                               int world, int b, unsigned int e, int* status,
                                               unsigned long long limit_ns) {
  const int j = threadIdx.x;
  bool ok = true;
  if (j < world) {
    st_release_sys(reinterpret_cast<unsigned int*>(flags.ptr[j]) +
                       (phase * kMaxPeers + my_rank) * kMaxArBlocks + b, e);
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(flags.ptr[my_rank]) +
                               (phase * kMaxPeers + j) * kMaxArBlocks + b;
    const unsigned long long t0 = globaltimer_ns();
    unsigned int spins = 0;
    while ((int)(ld_acquire_sys(mine) - e) < 0) {
      if ((++spins & 255u) == 0u && globaltimer_ns() - t0 > limit_ns) {
        report_error(status, kErrPeerFlagTimeout, j, (int)e);
        ok = false;
        break;
      }
    }
  }
  return ok;
}

__global__ void __launch_bounds__(512)
allreduce2_kernel(PeerTable parts, PeerTable res, PeerTable flags, unsigned int* epochs,
                  int my_rank, int world, long long n_vec, int* status,
                  unsigned long long limit_ns) {
  __shared__ unsigned int epoch;
  __shared__ int failed;
  const int b = blockIdx.x;
  if (threadIdx.x == 0) {
    epoch = epochs[b] + 1;
    failed = 0;
  }
  __syncthreads();
  const unsigned int e = epoch;
  __threadfence_system();
  if (!exchange_flags(flags, 0, my_rank, world, b, e, status, limit_ns)) failed = 1;
  __syncthreads();
  if (!failed) {
    const long long slice = (n_vec + world - 1) / world;
    const long long lo = (long long)my_rank * slice;
    const long long hi = lo + slice < n_vec ? lo + slice : n_vec;
    for (long long i = lo + (long long)b * blockDim.x + threadIdx.x; i < hi;
         i += (long long)gridDim.x * blockDim.x) {
      uint4 v[kMaxPeers];
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)
        if (r < world) v[r] = ld_sys_v4(reinterpret_cast<const uint4*>(parts.ptr[r]) + i);
      float acc[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
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
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)
        if (r < world) st_v4_global(reinterpret_cast<uint4*>(res.ptr[r]) + i, o);
    }
    __threadfence_system();
  }
  __syncthreads();
  if (!failed) exchange_flags(flags, 1, my_rank, world, b, e, status, limit_ns);
  __syncthreads();
  if (threadIdx.x == 0) epochs[b] = e;
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

// Two-shot all-reduce (see allreduce2_kernel). part_ptrs / res_ptrs / flag_ptrs: host arrays
// of `world` device pointers into the ranks' symmetric heaps; the flag area of every rank is
// ab200_allreduce2_flag_bytes() bytes, zero at start; `epochs` is this rank's own
// unsigned[128], zero at start. Every rank must call with the same n_elems. The result is
// complete in this rank's result buffer when the kernel ends.
long long ab200_allreduce2_flag_bytes() {
  return 2ll * kMaxPeers * kMaxArBlocks * (long long)sizeof(unsigned int);
}

int ab200_allreduce2(const void* const* part_ptrs, const void* const* res_ptrs,
                     const void* const* flag_ptrs, void* epochs, int my_rank, int world,
                     long long n_elems, int* status, cudaStream_t stream) {
  if (world < 1 || world > kMaxPeers || (n_elems % 8) || my_rank < 0 || my_rank >= world) return -2;
  if (n_elems == 0) return 0;
  PeerTable p, r, f;
  for (int i = 0; i < kMaxPeers; ++i) {
    p.ptr[i] = i < world ? const_cast<void*>(part_ptrs[i]) : nullptr;
    r.ptr[i] = i < world ? const_cast<void*>(res_ptrs[i]) : nullptr;
    f.ptr[i] = i < world ? const_cast<void*>(flag_ptrs[i]) : nullptr;
  }
  const long long n_vec = n_elems / 8;
  const long long slice = (n_vec + world - 1) / world;
  long long blocks = (slice + 511) / 512;   // the same on every rank: blocks pair up by index
  if (blocks > kMaxArBlocks) blocks = kMaxArBlocks;
  if (blocks < 1) blocks = 1;
  allreduce2_kernel<<<(unsigned)blocks, 512, 0, stream>>>(
      p, r, f, reinterpret_cast<unsigned int*>(epochs), my_rank, world, n_vec, status,
      kWaitLimitNs);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // extern "C"
