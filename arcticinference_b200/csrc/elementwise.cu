// Memory-bound building blocks of the decoder / encoder stacks, written for
// sm_100a: every kernel makes a single pass over HBM with 16-byte accesses and
// keeps the row it normalises in registers.
//
//   embedding gather, RMSNorm (+ fused residual add), LayerNorm (+ residual),
//   SiLU*mul, neox RoPE fused with the paged KV-cache write, row gather,
//   arg-max / Gumbel-max sampling over the vocabulary.
//
// The reference takes these from vLLM (arctic_inference/vllm/swiftkv/
// llama_swiftkv.py:129,165-202,254-259); here they are part of the engine.

#include <float.h>
#include <math.h>

#include "api.h"
#include "common/pdl.cuh"
#include "common/peer.cuh"
#include "common/ptx.cuh"

namespace ab200 {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]);
  q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]);
  q.w = pack_bf16x2(f[6], f[7]);
  return q;
}

// Block-wide sum of one value; `red` is 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}

// ------------------------------- embedding ---------------------------------
__global__ void embedding_kernel(const long long* __restrict__ ids, const bf16* __restrict__ table,
                                 bf16* __restrict__ out, int hidden, long long vocab,
                                 long long vocab_start) {
  pdl_wait();
  pdl_trigger();
  const long long t = blockIdx.x;
  long long id = ids[t] - vocab_start;
  const bool valid = id >= 0 && id < vocab;
  const uint4* src = reinterpret_cast<const uint4*>(table + (valid ? id : 0) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + t * hidden);
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) dst[i] = valid ? src[i] : zero;
}

// -------------------------------- RMSNorm ----------------------------------
// If `residual` is non-null: residual += x (written back), y = norm(residual).
// Up to kMaxVec 16-byte vectors per thread are kept in registers (hidden <= 16384 at 256 threads).
constexpr int kNormThreads = 256;
constexpr int kMaxVec = 8;

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(const bf16* __restrict__ x, long long ldx, bf16* __restrict__ residual,
               const bf16* __restrict__ weight, bf16* __restrict__ y, long long ldy, int hidden,
               float eps) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int nvec = hidden / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + row * (long long)hidden) : nullptr;
  float vals[kMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    if (i < nvec) {
      unpack8(xr[i], vals[j]);
      if (rr) {
        float r[8];
        unpack8(rr[i], r);
#pragma unroll
        for (int k = 0; k < 8; ++k) vals[j][k] += r[k];
        const uint4 q = pack8(vals[j]);
        rr[i] = q;
        unpack8(q, vals[j]);  // normalise the value that was stored (bf16-rounded)
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += vals[j][k] * vals[j][k];
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(weight);
  uint4* yr = reinterpret_cast<uint4*>(y + row * ldy);
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    if (i < nvec) {
      float w[8];
      unpack8(wr[i], w);
#pragma unroll
      for (int k = 0; k < 8; ++k) vals[j][k] = vals[j][k] * inv * w[k];
      yr[i] = pack8(vals[j]);
    }
  }
}

// Same operation for hidden == VPT * 8 * kNormThreads exactly (2048, 4096, 8192 for VPT = 1, 2,
// 4): the trip counts are compile-time constants, so every load of the row (x and residual)
// is issued before the first value is used and the row takes VPT * 8 live floats per thread.
template <int VPT>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fixed_kernel(const bf16* __restrict__ x, long long ldx, bf16* __restrict__ residual,
                     const bf16* __restrict__ weight, bf16* __restrict__ y, long long ldy,
                     float eps) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[32];
  constexpr int hidden = VPT * 8 * kNormThreads;
  const long long row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + row * (long long)hidden) : nullptr;
  uint4 xq[VPT], rq[VPT], wq[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) xq[j] = xr[threadIdx.x + j * kNormThreads];
  if (rr) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) rq[j] = rr[threadIdx.x + j * kNormThreads];
  }
#pragma unroll
  for (int j = 0; j < VPT; ++j)
    wq[j] = reinterpret_cast<const uint4*>(weight)[threadIdx.x + j * kNormThreads];
  float vals[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    unpack8(xq[j], vals[j]);
    if (rr) {
      float r[8];
      unpack8(rq[j], r);
#pragma unroll
      for (int k = 0; k < 8; ++k) vals[j][k] += r[k];
      const uint4 q = pack8(vals[j]);
      rr[threadIdx.x + j * kNormThreads] = q;
      unpack8(q, vals[j]);  // normalise the value that was stored (bf16-rounded)
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += vals[j][k] * vals[j][k];
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + row * ldy);
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    float w[8];
    unpack8(wq[j], w);
#pragma unroll
    for (int k = 0; k < 8; ++k) vals[j][k] = vals[j][k] * inv * w[k];
    yr[threadIdx.x + j * kNormThreads] = pack8(vals[j]);
  }
}

// ------------------------------- LayerNorm ---------------------------------
// y = LN(x (+ residual)) * gamma + beta, mean/variance in fp32.
__global__ void __launch_bounds__(kNormThreads)
layernorm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ residual,
                 const bf16* __restrict__ gamma, const bf16* __restrict__ beta,
                 bf16* __restrict__ y, int hidden, float eps) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int nvec = hidden / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * (long long)hidden);
  const uint4* rr =
      residual ? reinterpret_cast<const uint4*>(residual + row * (long long)hidden) : nullptr;
  float vals[kMaxVec][8];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    if (i < nvec) {
      unpack8(xr[i], vals[j]);
      if (rr) {
        float r[8];
        unpack8(rr[i], r);
#pragma unroll
        for (int k = 0; k < 8; ++k) vals[j][k] += r[k];
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) s += vals[j][k];
    }
  }
  const float mean = block_sum(s, red) / (float)hidden;
  float v = 0.f;
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    if (i < nvec) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float d = vals[j][k] - mean;
        v += d * d;
      }
    }
  }
  const float inv = rsqrtf(block_sum(v, red) / (float)hidden + eps);
  const uint4* gr = reinterpret_cast<const uint4*>(gamma);
  const uint4* br = reinterpret_cast<const uint4*>(beta);
  uint4* yr = reinterpret_cast<uint4*>(y + row * (long long)hidden);
#pragma unroll
  for (int j = 0; j < kMaxVec; ++j) {
    const int i = threadIdx.x + j * kNormThreads;
    if (i < nvec) {
      float g[8], b[8];
      unpack8(gr[i], g);
      unpack8(br[i], b);
#pragma unroll
      for (int k = 0; k < 8; ++k) vals[j][k] = (vals[j][k] - mean) * inv * g[k] + b[k];
      yr[i] = pack8(vals[j]);
    }
  }
}

// -------------------------------- SiLU * mul --------------------------------
// x: [T, nblk * 2 * inter] laid out as nblk blocks of (gate | up); out: [T, nblk * inter].
// nblk = 1 is the usual fused gate/up layout; nblk > 1 is the rank-major layout whose
// blocks are the tensor-parallel shards.
// Each thread keeps four (gate, up) vector pairs in flight per iteration: the loads of all
// four are issued before the first is used.
constexpr int kSiluUnroll = 4;

__global__ void __launch_bounds__(256, 4)
silu_mul_kernel(const bf16* __restrict__ x, bf16* __restrict__ out, long long T, int inter,
                int nblk) {
  pdl_wait();
  pdl_trigger();
  const int nvec = inter / 8;
  const long long per_row = (long long)nblk * nvec;
  const long long total = T * per_row;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < total;
       i0 += stride * kSiluUnroll) {
    uint4 gq[kSiluUnroll], uq[kSiluUnroll];
    long long dst[kSiluUnroll];
#pragma unroll
    for (int j = 0; j < kSiluUnroll; ++j) {
      const long long i = i0 + j * stride;
      dst[j] = -1;
      if (i < total) {
        const long long t = i / per_row;
        const int r = (int)(i - t * per_row);
        const int b = r / nvec;
        const int c = r - b * nvec;
        const uint4* row = reinterpret_cast<const uint4*>(x + (t * nblk + b) * 2ll * inter);
        gq[j] = row[c];
        uq[j] = row[nvec + c];
        dst[j] = (t * nblk + b) * (long long)nvec + c;
      }
    }
#pragma unroll
    for (int j = 0; j < kSiluUnroll; ++j) {
      if (dst[j] >= 0) {
        float g[8], u[8];
        unpack8(gq[j], g);
        unpack8(uq[j], u);
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] = __fdividef(g[k], 1.f + __expf(-g[k])) * u[k];
        reinterpret_cast<uint4*>(out)[dst[j]] = pack8(g);
      }
    }
  }
}

// ------------------------ RoPE + paged KV-cache write -----------------------
// qkv: [T, (Hq + 2*Hkv) * D] with row stride ld. Rotates q in place (neox
// pairing: element i with i + D/2), rotates k and writes k, v into the paged
// caches laid out [num_blocks, Hkv, block_size, D]. slot < 0 skips the cache
// write (padding tokens). inv_freq: [D/2] fp32 (any frequency scaling baked in).
__global__ void __launch_bounds__(256)
rope_cache_kernel(bf16* __restrict__ qkv, long long ld, const long long* __restrict__ positions,
                  const long long* __restrict__ slots, const float* __restrict__ inv_freq,
                  bf16* __restrict__ k_cache, bf16* __restrict__ v_cache, int Hq, int Hkv, int D,
                  int block_size, long long num_slots, int rotate_q, int* status,
                  const PeerWait wait) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float cs[];  // cos[D/2] | sin[D/2]
  // rows scattered here by the other ranks' QKV projections: wait for their completion signal
  if (wait.world > 0) {
    __shared__ int peers_ok;
    if (threadIdx.x < 32) {
      const bool ok = wait_peers(wait, status, kWaitLimitNs);
      if (threadIdx.x == 0) peers_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (!peers_ok) return;
  }
  const long long t = blockIdx.x;
  const int half = D / 2;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf(pos * inv_freq[i], &s, &c);
    cs[i] = c;
    cs[half + i] = s;
  }
  __syncthreads();
  bf16* row = qkv + t * ld;
  const long long slot = slots ? slots[t] : -1;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) report_error(status, kErrBounds, 1, (int)t);
    return;
  }
  const long long blk = slot >= 0 ? slot / block_size : 0;
  const int off = slot >= 0 ? (int)(slot % block_size) : 0;
  const int vec_per_half = half / 8;
  const int rot_heads = Hq + Hkv;
  // rotated heads: each work item handles 8 elements of the first half and their partners
  for (int i = threadIdx.x; i < rot_heads * vec_per_half; i += blockDim.x) {
    const int h = i / vec_per_half;
    const int c = i % vec_per_half;
    if (h < Hq && !rotate_q) continue;
    bf16* base = row + (long long)h * D;
    float a[8], b[8], oa[8], ob[8];
    unpack8(reinterpret_cast<uint4*>(base)[c], a);
    unpack8(reinterpret_cast<uint4*>(base + half)[c], b);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float co = cs[c * 8 + k], si = cs[half + c * 8 + k];
      oa[k] = a[k] * co - b[k] * si;
      ob[k] = b[k] * co + a[k] * si;
    }
    const uint4 qa = pack8(oa), qb = pack8(ob);
    if (h < Hq) {
      reinterpret_cast<uint4*>(base)[c] = qa;
      reinterpret_cast<uint4*>(base + half)[c] = qb;
    } else if (slot >= 0) {
      const int kh = h - Hq;
      bf16* dst = k_cache + ((blk * Hkv + kh) * block_size + off) * (long long)D;
      reinterpret_cast<uint4*>(dst)[c] = qa;
      reinterpret_cast<uint4*>(dst + half)[c] = qb;
    }
  }
  if (slot >= 0) {
    const int vec_per_head = D / 8;
    for (int i = threadIdx.x; i < Hkv * vec_per_head; i += blockDim.x) {
      const int kh = i / vec_per_head;
      const int c = i % vec_per_head;
      const uint4 q = reinterpret_cast<const uint4*>(row + (long long)(Hq + Hkv + kh) * D)[c];
      bf16* dst = v_cache + ((blk * Hkv + kh) * block_size + off) * (long long)D;
      reinterpret_cast<uint4*>(dst)[c] = q;
    }
  }
}

// -------------------------------- row gather --------------------------------
__global__ void gather_rows_kernel(const bf16* __restrict__ src, long long ld,
                                   const long long* __restrict__ idx, bf16* __restrict__ dst,
                                   int hidden) {
  pdl_wait();
  pdl_trigger();
  const long long r = blockIdx.x;
  const uint4* s = reinterpret_cast<const uint4*>(src + idx[r] * ld);
  uint4* d = reinterpret_cast<uint4*>(dst + r * (long long)hidden);
  for (int i = threadIdx.x; i < hidden / 8; i += blockDim.x) d[i] = s[i];
}

// ------------------------- arg-max / Gumbel-max sample -----------------------
// One block per row of logits [B, V] (bf16 or fp32). temperature <= 0: arg-max.
// Otherwise token = argmax(logit / T + Gumbel noise), an exact softmax sample;
// the noise comes from a counter-based hash of (the row's seed, the token's global index).
__device__ __forceinline__ float hash_uniform(unsigned long long seed, unsigned long long a,
                                              unsigned long long b) {
  unsigned long long z = seed + a * 0x9E3779B97F4A7C15ull + b * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z = z ^ (z >> 31);
  return ((float)(z >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

template <typename T>
__device__ __forceinline__ float load_logit(const T* p, long long i);
template <>
__device__ __forceinline__ float load_logit<bf16>(const bf16* p, long long i) {
  return __bfloat162float(p[i]);
}
template <>
__device__ __forceinline__ float load_logit<float>(const float* p, long long i) {
  return p[i];
}

template <typename T>
__global__ void __launch_bounds__(1024)
argmax_sample_kernel(const T* __restrict__ logits, long long ld, int V,
                     const float* __restrict__ temperature,
                     const unsigned long long* __restrict__ seeds, long long* __restrict__ out_ids,
                     float* __restrict__ out_vals, long long index_offset) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sv[32];
  __shared__ int si[32];
  const long long row = blockIdx.x;
  const T* lr = logits + row * ld;
  const float temp = temperature ? temperature[row] : 0.f;
  const unsigned long long seed = seeds ? seeds[row] : 0ull;
  float best = -FLT_MAX;
  int best_i = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = load_logit<T>(lr, i);
    if (temp > 0.f) {
      // keyed by the row's seed and the token's index in the whole vocabulary only: a
      // request draws the same token wherever its row sits in the batch, and the shards of
      // a split vocabulary draw independent noise for their columns
      const float u = hash_uniform(seed, 0ull, (unsigned long long)(index_offset + i));
      v = v / temp - __logf(-__logf(u));
    }
    if (v > best) {
      best = v;
      best_i = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ov > best || (ov == best && oi < best_i)) {
      best = ov;
      best_i = oi;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    best = lane < nw ? sv[lane] : -FLT_MAX;
    best_i = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ov > best || (ov == best && oi < best_i)) {
        best = ov;
        best_i = oi;
      }
    }
    if (lane == 0) {
      out_ids[row] = (long long)best_i + index_offset;
      if (out_vals) out_vals[row] = best;
    }
  }
}

// Run-ahead scheduling: rows whose input token is the previous step's sampled token (not yet
// known on the host) take it from that step's device result.
__global__ void patch_ids_kernel(long long* __restrict__ ids, const long long* __restrict__ src_rows,
                                 const long long* __restrict__ prev_ids, long long n,
                                 long long n_prev) {
  pdl_wait();
  pdl_trigger();
  const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  const long long j = src_rows[i];
  if (j >= 0 && j < n_prev) ids[i] = prev_ids[j];
}

}  // namespace ab200

using namespace ab200;

extern "C" {

int ab200_embedding(const void* ids, const void* table, void* out, long long T, int hidden,
                    long long vocab, long long vocab_start, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (hidden % 8) return -2;
  (void)launch_pdl(embedding_kernel, dim3((unsigned)T), dim3(128), 0, stream, 
      reinterpret_cast<const long long*>(ids), reinterpret_cast<const bf16*>(table),
      reinterpret_cast<bf16*>(out), hidden, vocab, vocab_start);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_rmsnorm(const void* x, long long ldx, void* residual, const void* weight, void* y,
                  long long ldy, long long T, int hidden, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((hidden % 8) || hidden > kNormThreads * kMaxVec * 8 || (ldx % 8) || (ldy % 8)) return -2;
  const bf16* xp = reinterpret_cast<const bf16*>(x);
  bf16* rp = reinterpret_cast<bf16*>(residual);
  const bf16* wp = reinterpret_cast<const bf16*>(weight);
  bf16* yp = reinterpret_cast<bf16*>(y);
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(residual) |
                         reinterpret_cast<uintptr_t>(weight) | reinterpret_cast<uintptr_t>(y)) & 15) == 0;
  if (aligned && hidden == 8 * kNormThreads)
    (void)launch_pdl(rmsnorm_fixed_kernel<1>, dim3((unsigned)T), dim3(kNormThreads), 0, stream,
                     xp, ldx, rp, wp, yp, ldy, eps);
  else if (aligned && hidden == 16 * kNormThreads)
    (void)launch_pdl(rmsnorm_fixed_kernel<2>, dim3((unsigned)T), dim3(kNormThreads), 0, stream,
                     xp, ldx, rp, wp, yp, ldy, eps);
  else if (aligned && hidden == 32 * kNormThreads)
    (void)launch_pdl(rmsnorm_fixed_kernel<4>, dim3((unsigned)T), dim3(kNormThreads), 0, stream,
                     xp, ldx, rp, wp, yp, ldy, eps);
  else
    (void)launch_pdl(rmsnorm_kernel, dim3((unsigned)T), dim3(kNormThreads), 0, stream,
                     xp, ldx, rp, wp, yp, ldy, hidden, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_layernorm(const void* x, const void* residual, const void* gamma, const void* beta,
                    void* y, long long T, int hidden, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((hidden % 8) || hidden > kNormThreads * kMaxVec * 8) return -2;
  (void)launch_pdl(layernorm_kernel, dim3((unsigned)T), dim3(kNormThreads), 0, stream, 
      reinterpret_cast<const bf16*>(x), reinterpret_cast<const bf16*>(residual),
      reinterpret_cast<const bf16*>(gamma), reinterpret_cast<const bf16*>(beta),
      reinterpret_cast<bf16*>(y), hidden, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_silu_mul(const void* x, void* out, long long T, int inter, int nblk,
                   cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((inter % 8) || nblk < 1) return -2;
  const long long total = T * nblk * (inter / 8);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  (void)launch_pdl(silu_mul_kernel, dim3((unsigned)blocks), dim3(256), 0, stream,
                   reinterpret_cast<const bf16*>(x),
                                                        reinterpret_cast<bf16*>(out), T, inter, nblk);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_rope_cache(void* qkv, long long ld, const void* positions, const void* slots,
                     const void* inv_freq, void* k_cache, void* v_cache, long long T, int Hq,
                     int Hkv, int D, int block_size, long long num_slots, int rotate_q, int* status,
                     cudaStream_t stream) {
  return ab200_rope_cache_wait(qkv, ld, positions, slots, inv_freq, k_cache, v_cache, T, Hq, Hkv, D,
                               block_size, num_slots, rotate_q, nullptr, status, stream);
}

// The same, first waiting (sync->wait_*) until every rank's producer of `qkv` has signalled.
int ab200_rope_cache_wait(void* qkv, long long ld, const void* positions, const void* slots,
                          const void* inv_freq, void* k_cache, void* v_cache, long long T, int Hq,
                          int Hkv, int D, int block_size, long long num_slots, int rotate_q,
                          const Ab200PeerSync* sync, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((D % 16) || (ld % 8)) return -2;
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
  (void)launch_pdl(rope_cache_kernel, dim3((unsigned)T), dim3(256), D * sizeof(float), stream, 
      reinterpret_cast<bf16*>(qkv), ld, reinterpret_cast<const long long*>(positions),
      reinterpret_cast<const long long*>(slots), reinterpret_cast<const float*>(inv_freq),
      reinterpret_cast<bf16*>(k_cache), reinterpret_cast<bf16*>(v_cache), Hq, Hkv, D, block_size,
      num_slots, rotate_q, status, w);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_gather_rows(const void* src, long long ld, const void* idx, void* dst, long long R,
                      int hidden, cudaStream_t stream) {
  if (R <= 0) return 0;
  if ((hidden % 8) || (ld % 8)) return -2;
  (void)launch_pdl(gather_rows_kernel, dim3((unsigned)R), dim3(128), 0, stream, 
      reinterpret_cast<const bf16*>(src), ld, reinterpret_cast<const long long*>(idx),
      reinterpret_cast<bf16*>(dst), hidden);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_patch_ids(void* ids, const void* src_rows, const void* prev_ids, long long n,
                    long long n_prev, cudaStream_t stream) {
  if (n <= 0) return 0;
  (void)launch_pdl(patch_ids_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, 
      reinterpret_cast<long long*>(ids), reinterpret_cast<const long long*>(src_rows),
      reinterpret_cast<const long long*>(prev_ids), n, n_prev);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// dtype: 0 = bf16 logits, 1 = fp32 logits
int ab200_argmax_sample(const void* logits, int dtype, long long ld, long long B, int V,
                        const void* temperature, const void* seeds, void* out_ids, void* out_vals,
                        long long index_offset, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (dtype == 0)
    (void)launch_pdl(argmax_sample_kernel<bf16>, dim3((unsigned)B), dim3(1024), 0, stream, 
        reinterpret_cast<const bf16*>(logits), ld, V, reinterpret_cast<const float*>(temperature),
        reinterpret_cast<const unsigned long long*>(seeds), reinterpret_cast<long long*>(out_ids),
        reinterpret_cast<float*>(out_vals), index_offset);
  else
    (void)launch_pdl(argmax_sample_kernel<float>, dim3((unsigned)B), dim3(1024), 0, stream, 
        reinterpret_cast<const float*>(logits), ld, V, reinterpret_cast<const float*>(temperature),
        reinterpret_cast<const unsigned long long*>(seeds), reinterpret_cast<long long*>(out_ids),
        reinterpret_cast<float*>(out_vals), index_offset);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // extern "C"
