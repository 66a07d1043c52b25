// Top-k / top-p truncation of a batch of logit rows without sorting them.
//
//   y = x / temperature;  keep the k largest y;  of those keep the smallest set of the most
//   likely tokens whose probability mass reaches top_p;  write y for kept tokens, -inf for
//   the others.
//
// The result feeds the arg-max / Gumbel-max kernel, so sampling from the truncated
// distribution needs no probability vector and no sort. The usual formulation sorts every row
// (vLLM's sampler does; the reference samples through it,
// arctic_inference/vllm/model_runner.py:594-617); a row of 128 256 logits is 0.5 MB, a batch
// of rows stays in the 126 MB L2, and a selection needs only counts and sums over it:
//
//   * top-k: the k-th largest value is found bit by bit on an order-preserving 32-bit key
//     (one counting pass over the row per bit, 32 passes, exact);
//   * top-p: a token is kept iff the mass of the tokens strictly more likely than it is at
//     most top_p * Z, Z being the mass of the top-k set. The kept set is {key >= c} for the
//     smallest key c that satisfies this; c is found by bisection on the key (one summing pass
//     per step, at most 32).
//
// Exactly k tokens survive the top-k step: of the tokens that tie for the k-th place the ones
// with the lowest ids stay (32 more counting passes, only when there is such a tie), so
// top_k = 1 is greedy decoding. At the top-p cut, tokens with equal logits stay or go
// together (a sort would split them arbitrarily). One CTA of 1024 threads per row; every pass is a coalesced read of the row,
// sums are reduced in a fixed order, so the result does not depend on timing.

#include <math.h>

#include "api.h"
#include "common/pdl.cuh"
#include "common/ptx.cuh"

namespace ab200 {
namespace {

constexpr int kThreads = 1024;

// order-preserving map from float to uint32 (larger float -> larger key)
__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ unsigned int block_sum_u32(unsigned int v, unsigned int* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // `red` may still be read by the previous reduction
  if (lane == 0) red[warp] = v;
  __syncthreads();
  unsigned int t = red[lane];   // kThreads / 32 == 32 entries
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;                     // the same value in every thread
}

__device__ __forceinline__ float block_sum_f32(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  return warp_sum(red[lane]);
}

__device__ __forceinline__ float block_max_f32(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  return warp_max(red[lane]);
}

__global__ void __launch_bounds__(kThreads)
topk_topp_mask_kernel(const float* __restrict__ logits, long long ld_in, float* __restrict__ out,
                      long long ld_out, int V, const float* __restrict__ temperature,
                      const long long* __restrict__ top_k, const float* __restrict__ top_p) {
  pdl_wait();
  pdl_trigger();
  __shared__ unsigned int red_u[32];
  __shared__ float red_f[32];
  const float* x = logits + (long long)blockIdx.x * ld_in;
  float* y_out = out + (long long)blockIdx.x * ld_out;
  const float temp = temperature != nullptr ? temperature[blockIdx.x] : 1.0f;
  const float inv_t = 1.0f / fmaxf(temp, 1e-5f);
  long long k = top_k != nullptr ? top_k[blockIdx.x] : 0;
  if (k <= 0 || k > V) k = V;
  const float p = top_p != nullptr ? top_p[blockIdx.x] : 1.0f;

  // the key of the k-th largest scaled logit (0: keep every token); of the tokens that hold
  // exactly this value, those with an index below tie_end belong to the k
  uint32_t k_key = 0u;
  unsigned int tie_end = 0xffffffffu;
  if (k < V) {
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = k_key | (1u << bit);
      unsigned int n = 0;
      for (int i = threadIdx.x; i < V; i += kThreads) n += float_key(x[i] * inv_t) >= cand ? 1u : 0u;
      n = block_sum_u32(n, red_u);
      if ((long long)n >= k) k_key = cand;
    }
    unsigned int above = 0, equal = 0;
    for (int i = threadIdx.x; i < V; i += kThreads) {
      const uint32_t key = float_key(x[i] * inv_t);
      above += key > k_key ? 1u : 0u;
      equal += key == k_key ? 1u : 0u;
    }
    above = block_sum_u32(above, red_u);
    equal = block_sum_u32(equal, red_u);
    const unsigned int need = (unsigned int)k - above;   // 1 <= need <= equal
    if (equal > need) {
      // the largest bound with at most `need` equal-valued tokens below it
      tie_end = 0u;
      for (int bit = 31; bit >= 0; --bit) {
        const unsigned int cand = tie_end | (1u << bit);
        unsigned int n = 0;
        for (int i = threadIdx.x; i < V; i += kThreads)
          n += ((unsigned int)i < cand && float_key(x[i] * inv_t) == k_key) ? 1u : 0u;
        n = block_sum_u32(n, red_u);
        if (n <= need) tie_end = cand;
      }
    }
  }
  // membership of the top-k set
  auto in_k = [&](uint32_t key, int i) {
    return key > k_key || (key == k_key && (unsigned int)i < tie_end);
  };

  uint32_t keep_key = k_key;
  if (p < 1.0f) {
    float m = -INFINITY;
    for (int i = threadIdx.x; i < V; i += kThreads) m = fmaxf(m, x[i] * inv_t);
    m = block_max_f32(m, red_f);
    if (m > -INFINITY) {
      float z = 0.f;
      for (int i = threadIdx.x; i < V; i += kThreads) {
        const float y = x[i] * inv_t;
        if (in_k(float_key(y), i)) z += __expf(y - m);
      }
      z = block_sum_f32(z, red_f);
      const float target = p * z;
      // smallest key c in [k_key, key(m)] with  sum_{key > c} exp(y - m) <= target
      uint32_t lo = k_key, hi = float_key(m);
      while (lo < hi) {
        const uint32_t mid = lo + ((hi - lo) >> 1);
        float s = 0.f;
        for (int i = threadIdx.x; i < V; i += kThreads) {
          const float y = x[i] * inv_t;
          if (float_key(y) > mid) s += __expf(y - m);
        }
        s = block_sum_f32(s, red_f);
        if (s <= target) hi = mid; else lo = mid + 1u;
      }
      keep_key = hi;
    }
  }

  for (int i = threadIdx.x; i < V; i += kThreads) {
    const float y = x[i] * inv_t;
    const uint32_t key = float_key(y);
    y_out[i] = (key >= keep_key && in_k(key, i)) ? y : -INFINITY;
  }
}

}  // namespace
}  // namespace ab200

using namespace ab200;

// logits, out: fp32 [B, V] with row strides ld_in / ld_out, not overlapping. temperature fp32
// [B] (null: 1), top_k int64 [B] (null or <= 0: off), top_p fp32 [B] (null or >= 1: off).
extern "C" int ab200_topk_topp_mask(const void* logits, long long ld_in, void* out, long long ld_out,
                                    int B, int V, const void* temperature, const void* top_k,
                                    const void* top_p, cudaStream_t stream) {
  if (B <= 0 || V <= 0) return 0;
  if (ld_in < V || ld_out < V || logits == out) return -2;
  (void)launch_pdl(topk_topp_mask_kernel, dim3((unsigned)B), dim3(kThreads), 0, stream,
                   reinterpret_cast<const float*>(logits), ld_in, reinterpret_cast<float*>(out),
                   ld_out, V, reinterpret_cast<const float*>(temperature),
                   reinterpret_cast<const long long*>(top_k),
                   reinterpret_cast<const float*>(top_p));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
