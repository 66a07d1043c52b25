// The small exchanges of a sequence- / tensor-parallel step, done by this library's own kernels
// over peer-mapped memory instead of library collectives:
//
//   * push_rows           -- the rows that feed the sampler (hidden state and residual of each
//     request's last token) go from the rank that owns the token to every rank: the owner
//     stores them into all ranks' staging buffers (the final all-gather of sequence-parallel
//     mode, arctic_inference/vllm/model_runner.py:397-403, of which only these rows are used).
//   * rmsnorm_allgather   -- the SwiftKV boundary: every rank normalises its own token slice
//     and stores the result rows into all ranks' full-length buffers in the same pass
//     (arctic_inference/vllm/swiftkv/llama_swiftkv.py:236-241 gathers hidden states, residual
//     and positions with three collectives; here the residual is needed for the sampled rows
//     only, which push_rows delivers).
//   * argmax_exchange     -- global arg-max over vocabulary shards: every rank stores its
//     (best value, best token) pair, 16 bytes per row, into all ranks' slots, the ranks meet
//     at a flag barrier inside the same kernel, and each reduces the W candidates locally
//     (arctic_inference/vllm/fp32_lm_head.py:179-185 and arctic_speculator.py:328-342 use an
//     all-gather of packed fp64 pairs).
//
//   * reduce_rmsnorm      -- the tensor-parallel reduction after a row-parallel linear layer,
//     folded into the RMSNorm that follows it: every rank's GEMM leaves its partial product in
//     its own heap and signals completion from its last block (tail_signal); this kernel waits
//     for the W signals, sums the W partial rows with peer loads in rank order (so every rank
//     gets the same bits), adds the residual, normalises and, for fp8 linears, quantises the
//     row, all in one pass. GEMM -> barrier -> all-reduce -> norm becomes GEMM -> this kernel
//     (the reference: NCCL all-reduce after vLLM's RowParallelLinear, then a norm kernel).
//
// All remote traffic is plain peer loads / stores; waits on peers are bounded (common/peer.cuh).

#include <cuda_fp8.h>

#include "api.h"
#include "common/peer.cuh"
#include "common/ptx.cuh"

namespace ab200 {

typedef __nv_bfloat16 bf16;

// Row r of the selection is global token idx[r], owned by rank idx[r] / rows_per_rank. The
// owner copies the token's row of src_a (and src_b) into row r of every rank's dst_a (dst_b).
// Destinations are visited starting at the owner itself, so that the W ranks' stores spread
// over the W destinations instead of all arriving at rank 0 first.
__global__ void __launch_bounds__(128)
push_rows_kernel(const bf16* __restrict__ src_a, long long ld_a, const bf16* __restrict__ src_b,
                 long long ld_b, long long rows_per_rank, int my_rank, int world,
                 const long long* __restrict__ idx, PeerTable dst_a, PeerTable dst_b,
                 int hidden) {
  const long long r = blockIdx.x;
  const long long g = idx[r];
  if (g < 0 || g / rows_per_rank != my_rank) return;
  const long long local = g - (long long)my_rank * rows_per_rank;
  const int nvec = hidden / 8;
  const uint4* sa = reinterpret_cast<const uint4*>(src_a + local * ld_a);
  const uint4* sb = src_b ? reinterpret_cast<const uint4*>(src_b + local * ld_b) : nullptr;
  for (int i = threadIdx.x; i < nvec; i += blockDim.x) {
    const uint4 va = sa[i];
    uint4 vb = make_uint4(0, 0, 0, 0);
    if (sb) vb = sb[i];
    for (int w = 0; w < world; ++w) {
      int peer = my_rank + w;
      if (peer >= world) peer -= world;
      st_v4_global(reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dst_a.ptr[peer]) +
                                            r * (long long)hidden) + i, va);
      if (sb)
        st_v4_global(reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dst_b.ptr[peer]) +
                                              r * (long long)hidden) + i, vb);
    }
  }
}

__device__ __forceinline__ void cf_unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 cf_pack8(const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]);
  q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]);
  q.w = pack_bf16x2(f[6], f[7]);
  return q;
}

// residual += x (written back, local); y = RMSNorm(residual) * weight goes to row
// (row_off + row) of every rank's destination. Up to 8 vectors of 8 per thread (hidden <= 16384).
constexpr int kCfThreads = 256;
constexpr int kCfMaxVec = 8;

__global__ void __launch_bounds__(kCfThreads)
rmsnorm_allgather_kernel(const bf16* __restrict__ x, long long ldx, bf16* __restrict__ residual,
                         const bf16* __restrict__ weight, PeerTable dst, long long row_off,
                         int my_rank, int world, int hidden, float eps) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int nvec = hidden / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + row * (long long)hidden) : nullptr;
  float vals[kCfMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kCfMaxVec; ++j) {
    const int i = threadIdx.x + j * kCfThreads;
    if (i < nvec) {
      cf_unpack8(xr[i], vals[j]);
      if (rr) {
        float r[8];
        cf_unpack8(rr[i], r);
#pragma unroll
        for (int k = 0; k < 8; ++k) vals[j][k] += r[k];
        const uint4 q = cf_pack8(vals[j]);
        rr[i] = q;
        cf_unpack8(q, vals[j]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += vals[j][k] * vals[j][k];
    }
  }
  ss = warp_sum(ss);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float t = (lane < kCfThreads / 32) ? red[lane] : 0.f;
  t = warp_sum(t);
  const float inv = rsqrtf(t / (float)hidden + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(weight);
#pragma unroll
  for (int j = 0; j < kCfMaxVec; ++j) {
    const int i = threadIdx.x + j * kCfThreads;
    if (i < nvec) {
      float w[8];
      cf_unpack8(wr[i], w);
#pragma unroll
      for (int k = 0; k < 8; ++k) vals[j][k] = vals[j][k] * inv * w[k];
      const uint4 q = cf_pack8(vals[j]);
      for (int p = 0; p < world; ++p) {
        int peer = my_rank + p;
        if (peer >= world) peer -= world;
        st_v4_global(reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dst.ptr[peer]) +
                                              (row_off + row) * (long long)hidden) + i, q);
      }
    }
  }
}

// out row = sum over ranks r = 0..W-1 of parts[r][row] (fp32 accumulation in rank order, rounded
// to bf16 as a stand-alone all-reduce would store it). With a weight: residual (+)= sum, then
// y = RMSNorm(residual) * weight as bf16 and / or as e4m3 with one scale per row. Without a
// weight only the reduced row is written (h_out). One CTA per row, the row stays in registers.
constexpr int kRnThreads = 256;
constexpr float kRnE4m3Max = 448.f;

template <int VPT>
__global__ void __launch_bounds__(kRnThreads)
reduce_rmsnorm_kernel(PeerTable parts, int world, long long ld_part, bf16* __restrict__ residual,
                      const bf16* __restrict__ weight, bf16* __restrict__ y, long long ldy,
                      uint8_t* __restrict__ yq, long long ldq, float* __restrict__ sy,
                      bf16* __restrict__ h_out, long long ldh, int hidden, float eps,
                      const PeerWait wait, int* status) {
  __shared__ float red[32];
  __shared__ int peers_ok;
  if (threadIdx.x < 32) {
    const bool ok = wait_peers(wait, status, kWaitLimitNs);
    if (threadIdx.x == 0) peers_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!peers_ok) return;
  const long long row = blockIdx.x;
  const int nvec = hidden / 8;
  float vals[VPT][8];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * kRnThreads;
#pragma unroll
    for (int k = 0; k < 8; ++k) vals[j][k] = 0.f;
    if (i < nvec) {
      uint4 v[kMaxPeers];
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r)
        if (r < world)
          v[r] = ld_sys_v4(reinterpret_cast<const uint4*>(
                               reinterpret_cast<const bf16*>(parts.ptr[r]) + row * ld_part) + i);
#pragma unroll
      for (int r = 0; r < kMaxPeers; ++r) {
        if (r < world) {
          float f[8];
          cf_unpack8(v[r], f);
#pragma unroll
          for (int k = 0; k < 8; ++k) vals[j][k] += f[k];
        }
      }
      const uint4 q = cf_pack8(vals[j]);   // the bf16 value an all-reduce would have stored
      cf_unpack8(q, vals[j]);
      if (h_out) reinterpret_cast<uint4*>(h_out + row * ldh)[i] = q;
    }
  }
  if (weight == nullptr) return;
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + row * (long long)hidden) : nullptr;
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * kRnThreads;
    if (i < nvec) {
      if (rr) {
        float r[8];
        cf_unpack8(rr[i], r);
#pragma unroll
        for (int k = 0; k < 8; ++k) vals[j][k] += r[k];
        const uint4 q = cf_pack8(vals[j]);
        rr[i] = q;
        cf_unpack8(q, vals[j]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += vals[j][k] * vals[j][k];
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float t = (lane < kRnThreads / 32) ? red[lane] : 0.f;
  t = warp_sum(t);
  const float inv_rms = rsqrtf(t / (float)hidden + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(weight);
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * kRnThreads;
    if (i < nvec) {
      float w[8];
      cf_unpack8(wr[i], w);
#pragma unroll
      for (int k = 0; k < 8; ++k) vals[j][k] = vals[j][k] * inv_rms * w[k];
      const uint4 q = cf_pack8(vals[j]);
      cf_unpack8(q, vals[j]);
      if (y) reinterpret_cast<uint4*>(y + row * ldy)[i] = q;
#pragma unroll
      for (int k = 0; k < 8; ++k) amax = fmaxf(amax, fabsf(vals[j][k]));
    }
  }
  if (yq == nullptr) return;
  amax = warp_max(amax);
  __syncthreads();
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  float m = (lane < kRnThreads / 32) ? red[lane] : 0.f;
  m = warp_max(m);
  const float scale = fmaxf(m, 1e-10f) / kRnE4m3Max;
  const float inv = 1.f / scale;
  uint2* qr = reinterpret_cast<uint2*>(yq + row * ldq);
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * kRnThreads;
    if (i < nvec) {
      uint32_t w2[2];
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2) {
        const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
            make_float2(vals[j][4 * h2] * inv, vals[j][4 * h2 + 1] * inv), __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
            make_float2(vals[j][4 * h2 + 2] * inv, vals[j][4 * h2 + 3] * inv), __NV_SATFINITE,
            __NV_E4M3);
        w2[h2] = (uint32_t)lo | ((uint32_t)hi << 16);
      }
      qr[i] = make_uint2(w2[0], w2[1]);
    }
  }
  if (threadIdx.x == 0) sy[row] = scale;
}

// One block. slots.ptr[r] is rank r's candidate array: [2 (parity)][world][max_rows] entries of
// {float value, int32 unused, int64 token}. Phase 1: store this rank's B candidates into every
// rank's array at [parity][my_rank]. Phase 2: flag barrier. Phase 3: per row, the best of the
// W candidates (ties go to the lowest token id, as a single arg-max over the whole vocabulary
// would break them).
struct Candidate {
  float val;
  int pad;
  long long tok;
};

__global__ void __launch_bounds__(1024)
argmax_exchange_kernel(const long long* __restrict__ ids, const float* __restrict__ vals, int B,
                       int max_rows, PeerTable slots, PeerTable flags, int my_rank, int world,
                       unsigned int* epoch_ctr, int* status, unsigned long long limit_ns,
                       long long* __restrict__ out_ids, float* __restrict__ out_vals) {
  const int parity = (int)((*epoch_ctr) & 1u);
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    uint4 q;
    q.x = __float_as_uint(vals[b]);
    q.y = 0;
    const long long t = ids[b];
    q.z = (unsigned int)(t & 0xffffffffll);
    q.w = (unsigned int)((unsigned long long)t >> 32);
    for (int w = 0; w < world; ++w) {
      int peer = my_rank + w;
      if (peer >= world) peer -= world;
      Candidate* base = reinterpret_cast<Candidate*>(slots.ptr[peer]);
      st_v4_global(base + ((long long)parity * world + my_rank) * max_rows + b, q);
    }
  }
  flag_barrier(flags, my_rank, world, epoch_ctr, status, limit_ns);
  const Candidate* mine = reinterpret_cast<const Candidate*>(slots.ptr[my_rank]);
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    float best = 0.f;
    long long tok = -1;
    for (int r = 0; r < world; ++r) {
      const uint4 q = ld_sys_v4(mine + ((long long)parity * world + r) * max_rows + b);
      const float v = __uint_as_float(q.x);
      const long long t = (long long)(((unsigned long long)q.w << 32) | q.z);
      if (tok < 0 || v > best || (v == best && t < tok)) {
        best = v;
        tok = t;
      }
    }
    out_ids[b] = tok;
    if (out_vals) out_vals[b] = best;
  }
}

}  // namespace ab200

using namespace ab200;

static void fill_table(PeerTable& t, const void* const* ptrs, int world) {
  for (int i = 0; i < kMaxPeers; ++i)
    t.ptr[i] = (ptrs != nullptr && i < world) ? const_cast<void*>(ptrs[i]) : nullptr;
}

extern "C" {

// Rows idx[0..R) (global token indices, int64; owner = idx / rows_per_rank) of the local
// token slices src_a / src_b (row strides in elements; src_b and dst_b may be null) land in
// rows 0..R of every rank's dst_a / dst_b ([R, hidden] bf16, contiguous). The caller runs a
// barrier before the destinations are read.
int ab200_push_rows(const void* src_a, long long ld_a, const void* src_b, long long ld_b,
                    long long rows_per_rank, int my_rank, int world, const void* idx,
                    const void* const* dst_a, const void* const* dst_b, long long R, int hidden,
                    cudaStream_t stream) {
  if (world < 1 || world > kMaxPeers || (hidden % 8) || (ld_a % 8) || (ld_b % 8) ||
      rows_per_rank <= 0 || my_rank < 0 || my_rank >= world)
    return -2;
  if (R <= 0) return 0;
  PeerTable ta, tb;
  fill_table(ta, dst_a, world);
  fill_table(tb, src_b != nullptr ? dst_b : nullptr, world);
  push_rows_kernel<<<(unsigned)R, 128, 0, stream>>>(
      reinterpret_cast<const bf16*>(src_a), ld_a, reinterpret_cast<const bf16*>(src_b), ld_b,
      rows_per_rank, my_rank, world, reinterpret_cast<const long long*>(idx), ta, tb, hidden);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// RMSNorm(x (+ residual, updated in place)) of T local rows, written to rows row_off.. of every
// rank's destination ([*, hidden] bf16). hidden <= 16384, multiple of 8.
int ab200_rmsnorm_allgather(const void* x, long long ldx, void* residual, const void* weight,
                            const void* const* dst, long long row_off, int my_rank, int world,
                            long long T, int hidden, float eps, cudaStream_t stream) {
  if (world < 1 || world > kMaxPeers || (hidden % 8) || (ldx % 8) || hidden > 16384 ||
      my_rank < 0 || my_rank >= world)
    return -2;
  if (T <= 0) return 0;
  PeerTable t;
  fill_table(t, dst, world);
  rmsnorm_allgather_kernel<<<(unsigned)T, kCfThreads, 0, stream>>>(
      reinterpret_cast<const bf16*>(x), ldx, reinterpret_cast<bf16*>(residual),
      reinterpret_cast<const bf16*>(weight), t, row_off, my_rank, world, hidden, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Tensor-parallel reduction fused with the norm that follows it. part_ptrs: the ranks' partial
// products ([rows, hidden] bf16 with row stride ld_part, in their symmetric heaps), each
// complete once that rank has signalled on the channel `sync->wait_*` describes. weight == null:
// only the reduced rows are written to h_out. Otherwise residual (may be null; contiguous rows)
// is updated in place and the normalised rows go to y (bf16, may be null) and / or yq + sy (e4m3
// + one fp32 scale per row, may be null). hidden <= 16384, a multiple of 8.
int ab200_reduce_rmsnorm(const void* const* part_ptrs, int world, long long ld_part, void* residual,
                         const void* weight, void* y, long long ldy, void* yq, long long ldq,
                         void* sy, void* h_out, long long ldh, long long rows, int hidden,
                         float eps, const Ab200PeerSync* sync, int* status, cudaStream_t stream) {
  if (world < 1 || world > kMaxPeers || (hidden % 8) || hidden > 16384 || (ld_part % 8) ||
      (y != nullptr && (ldy % 8)) || (yq != nullptr && ((ldq % 8) || sy == nullptr)) ||
      (h_out != nullptr && (ldh % 8)))
    return -2;
  if (weight == nullptr && h_out == nullptr) return -2;
  if (rows <= 0) return 0;
  PeerTable t;
  fill_table(t, part_ptrs, world);
  PeerWait w;
  w.flags = nullptr;
  w.epoch_ctr = nullptr;
  w.world = 0;
  if (sync != nullptr && sync->wait_world > 0) {
    if (sync->wait_world > kMaxPeers) return -2;
    w.flags = reinterpret_cast<const unsigned int*>(sync->wait_flags);
    w.epoch_ctr = reinterpret_cast<const unsigned int*>(sync->wait_epoch_ctr);
    w.world = sync->wait_world;
  }
  const int nvec = hidden / 8;
#define AB200_LAUNCH_RN(V)                                                                      \
  reduce_rmsnorm_kernel<V><<<(unsigned)rows, kRnThreads, 0, stream>>>(                          \
      t, world, ld_part, reinterpret_cast<bf16*>(residual), reinterpret_cast<const bf16*>(weight), \
      reinterpret_cast<bf16*>(y), ldy, reinterpret_cast<uint8_t*>(yq), ldq,                     \
      reinterpret_cast<float*>(sy), reinterpret_cast<bf16*>(h_out), ldh, hidden, eps, w, status)
  if (nvec <= 256) AB200_LAUNCH_RN(1);
  else if (nvec <= 512) AB200_LAUNCH_RN(2);
  else if (nvec <= 1024) AB200_LAUNCH_RN(4);
  else AB200_LAUNCH_RN(8);
#undef AB200_LAUNCH_RN
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

size_t ab200_argmax_exchange_slot_bytes(int world, int max_rows) {
  return (size_t)2 * world * max_rows * sizeof(Candidate);
}

// ids int64 [B], vals fp32 [B]: this rank's best token (already offset into the global
// vocabulary) and its score per row. out_ids int64 [B] (and out_vals, may be null) receive the
// best over all ranks. slot_ptrs: the ranks' candidate arrays (ab200_argmax_exchange_slot_bytes
// each); flag_ptrs / epoch_ctr as for ab200_barrier (the same flags and counter may be shared
// with it: every rank issues the same sequence of exchanges).
int ab200_argmax_exchange(const void* ids, const void* vals, int B, int max_rows,
                          const void* const* slot_ptrs, const void* const* flag_ptrs, int my_rank,
                          int world, void* epoch_ctr, void* out_ids, void* out_vals, int* status,
                          cudaStream_t stream) {
  if (world < 1 || world > kMaxPeers || B < 0 || B > max_rows || my_rank < 0 || my_rank >= world)
    return -2;
  if (B == 0) return 0;
  PeerTable s, f;
  fill_table(s, slot_ptrs, world);
  fill_table(f, flag_ptrs, world);
  int threads = 32;
  while (threads < B && threads < 1024) threads <<= 1;
  if (threads < world) threads = 32;
  argmax_exchange_kernel<<<1, threads, 0, stream>>>(
      reinterpret_cast<const long long*>(ids), reinterpret_cast<const float*>(vals), B, max_rows,
      s, f, my_rank, world, reinterpret_cast<unsigned int*>(epoch_ctr), status, kWaitLimitNs,
      reinterpret_cast<long long*>(out_ids), reinterpret_cast<float*>(out_vals));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // extern "C"
