// Encoder-only (BERT family) pieces that the decoder stack does not have:
//
//  * embedding: word + position + token-type rows summed and layer-normalised in one pass
//    (the three gathers never touch HBM as separate tensors);
//  * pooling: CLS row or mean over each sequence's rows, then optional L2 normalisation,
//    written as fp32 (what the embedding service returns).
//
// The reference obtains these from the vLLM pooling model that its embedding replica wraps
// (arctic_inference/embedding/replica.py:83-128).

#include "api.h"
#include "common/ptx.cuh"

namespace ab200 {

typedef __nv_bfloat16 bf16;

constexpr int kEncThreads = 128;
constexpr int kEncMaxVec = 8;  // hidden <= 128 * 8 * 8 = 8192

__device__ __forceinline__ void enc_unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ float enc_block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (kEncThreads >> 5)) ? red[lane] : 0.f;
  return warp_sum(t);
}

__global__ void __launch_bounds__(kEncThreads)
bert_embed_ln_kernel(const long long* __restrict__ ids, const long long* __restrict__ positions,
                     const long long* __restrict__ type_ids, const bf16* __restrict__ word,
                     const bf16* __restrict__ pos, const bf16* __restrict__ type,
                     const bf16* __restrict__ gamma, const bf16* __restrict__ beta,
                     bf16* __restrict__ out, int hidden, long long vocab, long long max_pos,
                     long long n_types, float eps, int* status) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  long long id = ids[t], p = positions[t], ty = type_ids ? type_ids[t] : 0;
  if (id < 0 || id >= vocab || p < 0 || p >= max_pos || ty < 0 || ty >= n_types) {
    if (threadIdx.x == 0) report_error(status, kErrBounds, 4, (int)t);
    id = 0;
    p = 0;
    ty = 0;
  }
  const int nvec = hidden / 8;
  const uint4* wr = reinterpret_cast<const uint4*>(word + id * hidden);
  const uint4* pr = reinterpret_cast<const uint4*>(pos + p * hidden);
  const uint4* tr = reinterpret_cast<const uint4*>(type + ty * hidden);
  float vals[kEncMaxVec][8];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < kEncMaxVec; ++j) {
    const int i = threadIdx.x + j * kEncThreads;
    if (i < nvec) {
      float a[8], b[8], c[8];
      enc_unpack8(wr[i], a);
      enc_unpack8(pr[i], b);
      enc_unpack8(tr[i], c);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        vals[j][k] = a[k] + b[k] + c[k];
        s += vals[j][k];
      }
    }
  }
  const float mean = enc_block_sum(s, red) / (float)hidden;
  float v = 0.f;
#pragma unroll
  for (int j = 0; j < kEncMaxVec; ++j) {
    const int i = threadIdx.x + j * kEncThreads;
    if (i < nvec) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float d = vals[j][k] - mean;
        v += d * d;
      }
    }
  }
  const float inv = rsqrtf(enc_block_sum(v, red) / (float)hidden + eps);
  const uint4* gr = reinterpret_cast<const uint4*>(gamma);
  const uint4* br = reinterpret_cast<const uint4*>(beta);
  uint4* yr = reinterpret_cast<uint4*>(out + t * hidden);
#pragma unroll
  for (int j = 0; j < kEncMaxVec; ++j) {
    const int i = threadIdx.x + j * kEncThreads;
    if (i < nvec) {
      float g[8], b[8];
      enc_unpack8(gr[i], g);
      enc_unpack8(br[i], b);
      uint4 q;
      uint32_t* qw = reinterpret_cast<uint32_t*>(&q);
#pragma unroll
      for (int k = 0; k < 4; ++k)
        qw[k] = pack_bf16x2((vals[j][2 * k] - mean) * inv * g[2 * k] + b[2 * k],
                            (vals[j][2 * k + 1] - mean) * inv * g[2 * k + 1] + b[2 * k + 1]);
      yr[i] = q;
    }
  }
}

// One block per sequence. mode 0: first row (CLS); 1: mean over the rows; 2: last row.
__global__ void __launch_bounds__(kEncThreads)
pool_normalize_kernel(const bf16* __restrict__ h, long long ld, const long long* __restrict__ starts,
                      float* __restrict__ out, int hidden, int mode, int normalize) {
  __shared__ float red[32];
  const int sidx = blockIdx.x;
  const long long r0 = starts[sidx], r1 = starts[sidx + 1];
  const int nvec = hidden / 8;
  float acc[kEncMaxVec][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kEncMaxVec; ++j) {
    const int i = threadIdx.x + j * kEncThreads;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[j][k] = 0.f;
    if (i < nvec && r1 > r0) {
      if (mode == 1) {
        for (long long r = r0; r < r1; ++r) {
          float f[8];
          enc_unpack8(reinterpret_cast<const uint4*>(h + r * ld)[i], f);
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[j][k] += f[k];
        }
        const float invn = 1.f / (float)(r1 - r0);
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[j][k] *= invn;
      } else {
        const long long r = mode == 0 ? r0 : r1 - 1;
        enc_unpack8(reinterpret_cast<const uint4*>(h + r * ld)[i], acc[j]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) ss += acc[j][k] * acc[j][k];
    }
  }
  float scale = 1.f;
  if (normalize) {
    const float tot = enc_block_sum(ss, red);
    scale = rsqrtf(fmaxf(tot, 1e-24f));
  }
#pragma unroll
  for (int j = 0; j < kEncMaxVec; ++j) {
    const int i = threadIdx.x + j * kEncThreads;
    if (i < nvec) {
      float4* o = reinterpret_cast<float4*>(out + (long long)sidx * hidden + i * 8);
      o[0] = make_float4(acc[j][0] * scale, acc[j][1] * scale, acc[j][2] * scale, acc[j][3] * scale);
      o[1] = make_float4(acc[j][4] * scale, acc[j][5] * scale, acc[j][6] * scale, acc[j][7] * scale);
    }
  }
}

}  // namespace ab200

using namespace ab200;

extern "C" {

int ab200_bert_embed_ln(const void* ids, const void* positions, const void* type_ids,
                        const void* word, const void* pos, const void* type, const void* gamma,
                        const void* beta, void* out, long long T, int hidden, long long vocab,
                        long long max_pos, long long n_types, float eps, int* status,
                        cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((hidden % 8) || hidden > kEncThreads * kEncMaxVec * 8) return -2;
  bert_embed_ln_kernel<<<(unsigned)T, kEncThreads, 0, stream>>>(
      reinterpret_cast<const long long*>(ids), reinterpret_cast<const long long*>(positions),
      reinterpret_cast<const long long*>(type_ids), reinterpret_cast<const bf16*>(word),
      reinterpret_cast<const bf16*>(pos), reinterpret_cast<const bf16*>(type),
      reinterpret_cast<const bf16*>(gamma), reinterpret_cast<const bf16*>(beta),
      reinterpret_cast<bf16*>(out), hidden, vocab, max_pos, n_types, eps, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_pool_normalize(const void* h, long long ld, const void* starts, void* out, int n_seqs,
                         int hidden, int mode, int normalize, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if ((hidden % 8) || (ld % 8) || hidden > kEncThreads * kEncMaxVec * 8 || mode < 0 || mode > 2)
    return -2;
  pool_normalize_kernel<<<(unsigned)n_seqs, kEncThreads, 0, stream>>>(
      reinterpret_cast<const bf16*>(h), ld, reinterpret_cast<const long long*>(starts),
      reinterpret_cast<float*>(out), hidden, mode, normalize);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // extern "C"
