// Per-token dynamic fp8 (e4m3) quantisation of activations, stand-alone and fused into the
// kernels that produce the activations of the decoder's linear layers:
//
//   quant_fp8_row        x bf16 [M, K]                   -> xq e4m3 [M, K], sx fp32 [M]
//   rmsnorm_quant        RMSNorm(x (+ residual))         -> same pair (residual updated in place)
//   silu_mul_quant       SiLU(gate) * up of fused blocks -> same pair
//
// sx[m] = max_k |y[m, k]| / 448 and xq = round_e4m3(y / sx), where y is the bf16-rounded value
// the unfused kernel would have stored, so fused and unfused paths agree bit for bit. One CTA
// owns one row and keeps it in registers between the reduction and the conversion: one pass
// over HBM, 16-byte loads, 8-byte stores. Together with per-output-feature weight scales this
// is the format ab200_linear_fp8_row multiplies (the reference: dynamic per-token activation
// scales of arctic_inference/vllm/spec_dec/fp8.py:34-309 and ops.scaled_fp8_quant).

#include <cuda_fp8.h>
#include <math.h>

#include "api.h"
#include "common/pdl.cuh"
#include "common/peer.cuh"
#include "common/ptx.cuh"

namespace ab200 {

typedef __nv_bfloat16 bf16;

constexpr int kQThreads = 256;
constexpr float kE4m3Max = 448.f;

__device__ __forceinline__ void q_unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 q_pack8(const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]);
  q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]);
  q.w = pack_bf16x2(f[6], f[7]);
  return q;
}
// eight floats, already divided by the scale, to eight e4m3 bytes
__device__ __forceinline__ uint2 to_e4m3x8(const float (&v)[8], float inv) {
  uint32_t w[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
        make_float2(v[4 * i] * inv, v[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
        make_float2(v[4 * i + 2] * inv, v[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
    w[i] = (uint32_t)lo | ((uint32_t)hi << 16);
  }
  return make_uint2(w[0], w[1]);
}
__device__ __forceinline__ float amax8(const float (&v)[8]) {
  float m = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) m = fmaxf(m, fabsf(v[k]));
  return m;
}
// round to bf16 and back: the value a bf16 store would have kept
__device__ __forceinline__ void round_bf16x8(float (&v)[8]) {
  const uint4 q = q_pack8(v);
  q_unpack8(q, v);
}

__device__ __forceinline__ float q_block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float q_block_max(float v, float* red) {
  v = warp_max(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? red[lane] : 0.f;
  return warp_max(t);
}

// ----------------------------------------------------------------- stand-alone
// MAXV vectors of 8 elements per thread stay in registers (K <= MAXV * 8 * blockDim.x).
template <int MAXV>
__global__ void __launch_bounds__(512)
quant_fp8_row_kernel(const bf16* __restrict__ x, long long ldx, uint8_t* __restrict__ xq,
                     long long ldq, float* __restrict__ sx, int K, const PeerWait wait,
                     int* status) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[32];
  // x may be rows that other ranks' attention kernels scattered here: wait for their signal
  if (wait.world > 0) {
    __shared__ int peers_ok;
    if (threadIdx.x < 32) {
      const bool ok = wait_peers(wait, status, kWaitLimitNs);
      if (threadIdx.x == 0) peers_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (!peers_ok) return;
  }
  const long long row = blockIdx.x;
  const int nvec = K / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  uint4 raw[MAXV];
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    raw[j] = (i < nvec) ? xr[i] : make_uint4(0, 0, 0, 0);
  }
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    float v[8];
    q_unpack8(raw[j], v);
    amax = fmaxf(amax, amax8(v));
  }
  amax = q_block_max(amax, red);
  const float scale = fmaxf(amax, 1e-10f) / kE4m3Max;
  const float inv = 1.f / scale;
  uint2* qr = reinterpret_cast<uint2*>(xq + row * ldq);
#pragma unroll
  for (int j = 0; j < MAXV; ++j) {
    const int i = threadIdx.x + j * blockDim.x;
    if (i < nvec) {
      float v[8];
      q_unpack8(raw[j], v);
      qr[i] = to_e4m3x8(v, inv);
    }
  }
  if (threadIdx.x == 0) sx[row] = scale;
}

// ------------------------------------------------------------- RMSNorm + quant
// residual (if given, contiguous rows of `hidden`) += x and is written back; the normalised
// row goes out as e4m3 with its scale, and also as bf16 when y != nullptr.
template <int VPT>
__global__ void __launch_bounds__(kQThreads)
rmsnorm_quant_kernel(const bf16* __restrict__ x, long long ldx, bf16* __restrict__ residual,
                     const bf16* __restrict__ weight, uint8_t* __restrict__ yq, long long ldq,
                     float* __restrict__ sy, bf16* __restrict__ y, long long ldy, int hidden,
                     float eps) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int nvec = hidden / 8;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * ldx);
  uint4* rr = residual ? reinterpret_cast<uint4*>(residual + row * (long long)hidden) : nullptr;
  const uint4* wr = reinterpret_cast<const uint4*>(weight);
  uint4 xraw[VPT], rraw[VPT], wraw[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * kQThreads;
    xraw[j] = (i < nvec) ? xr[i] : make_uint4(0, 0, 0, 0);
  }
  if (rr) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = threadIdx.x + j * kQThreads;
      rraw[j] = (i < nvec) ? rr[i] : make_uint4(0, 0, 0, 0);
    }
  }
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * kQThreads;
    wraw[j] = (i < nvec) ? wr[i] : make_uint4(0, 0, 0, 0);
  }
  float vals[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * kQThreads;
    q_unpack8(xraw[j], vals[j]);
    if (rr) {
      float r[8];
      q_unpack8(rraw[j], r);
#pragma unroll
      for (int k = 0; k < 8; ++k) vals[j][k] += r[k];
      const uint4 q = q_pack8(vals[j]);
      if (i < nvec) rr[i] = q;
      q_unpack8(q, vals[j]);  // normalise the value that was stored (bf16-rounded)
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) ss += vals[j][k] * vals[j][k];
  }
  ss = q_block_sum(ss, red);
  const float inv_rms = rsqrtf(ss / (float)hidden + eps);
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    float w[8];
    q_unpack8(wraw[j], w);
#pragma unroll
    for (int k = 0; k < 8; ++k) vals[j][k] = vals[j][k] * inv_rms * w[k];
    round_bf16x8(vals[j]);
    amax = fmaxf(amax, amax8(vals[j]));
  }
  amax = q_block_max(amax, red);
  const float scale = fmaxf(amax, 1e-10f) / kE4m3Max;
  const float inv = 1.f / scale;
  uint2* qr = reinterpret_cast<uint2*>(yq + row * ldq);
  uint4* yr = y ? reinterpret_cast<uint4*>(y + row * ldy) : nullptr;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int i = threadIdx.x + j * kQThreads;
    if (i < nvec) {
      qr[i] = to_e4m3x8(vals[j], inv);
      if (yr) yr[i] = q_pack8(vals[j]);
    }
  }
  if (threadIdx.x == 0) sy[row] = scale;
}

// ----------------------------------------------------------- SiLU * mul + quant
// x: [T, nblk * 2 * inter] as nblk blocks of (gate | up) -> outq [T, nblk * inter] e4m3 with one
// scale per token over the whole output row. One CTA per row: the products are computed once,
// parked as bf16 in shared memory (2 bytes per output element) while the row's largest
// magnitude is reduced, then converted to e4m3 from there. Few registers, several rows in
// flight per SM, one pass over HBM.
constexpr int kSiluQThreads = 256;
constexpr int kSiluQUnroll = 4;

__device__ __forceinline__ uint4 silu_mul8(const uint4& gq, const uint4& uq) {
  float g[8], u[8];
  q_unpack8(gq, g);
  q_unpack8(uq, u);
#pragma unroll
  for (int k = 0; k < 8; ++k) g[k] = __fdividef(g[k], 1.f + __expf(-g[k])) * u[k];
  return q_pack8(g);
}

__global__ void __launch_bounds__(kSiluQThreads)
silu_mul_quant_kernel(const bf16* __restrict__ x, uint8_t* __restrict__ outq, long long ldq,
                      float* __restrict__ so, int inter, int nblk) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ uint4 prod[];   // nblk * inter / 8 vectors of 8 bf16
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const int nvec = inter / 8;
  const int total = nblk * nvec;
  const bf16* xrow = x + row * (long long)nblk * 2 * inter;
  float amax = 0.f;
  for (int i0 = threadIdx.x; i0 < total; i0 += kSiluQThreads * kSiluQUnroll) {
    uint4 gq[kSiluQUnroll], uq[kSiluQUnroll];
#pragma unroll
    for (int j = 0; j < kSiluQUnroll; ++j) {
      const int i = i0 + j * kSiluQThreads;
      gq[j] = make_uint4(0, 0, 0, 0);
      uq[j] = make_uint4(0, 0, 0, 0);
      if (i < total) {
        const int b = nblk == 1 ? 0 : i / nvec;
        const int c = i - b * nvec;
        const uint4* blk = reinterpret_cast<const uint4*>(xrow + (long long)b * 2 * inter);
        gq[j] = blk[c];
        uq[j] = blk[nvec + c];
      }
    }
#pragma unroll
    for (int j = 0; j < kSiluQUnroll; ++j) {
      const int i = i0 + j * kSiluQThreads;
      if (i < total) {
        const uint4 p = silu_mul8(gq[j], uq[j]);
        prod[i] = p;
        float o[8];
        q_unpack8(p, o);
        amax = fmaxf(amax, amax8(o));
      }
    }
  }
  amax = q_block_max(amax, red);   // its barriers also publish `prod`
  const float scale = fmaxf(amax, 1e-10f) / kE4m3Max;
  const float inv = 1.f / scale;
  uint2* qr = reinterpret_cast<uint2*>(outq + row * ldq);
  for (int i = threadIdx.x; i < total; i += kSiluQThreads) {
    float o[8];
    q_unpack8(prod[i], o);
    qr[i] = to_e4m3x8(o, inv);
  }
  if (threadIdx.x == 0) so[row] = scale;
}

}  // namespace ab200

using namespace ab200;

extern "C" {

// x bf16 [M, K] (row stride ldx elements) -> xq e4m3 [M, K] (row stride ldq bytes), sx fp32 [M].
// K must be a multiple of 8 and at most 32768.
int ab200_quant_fp8_row(const void* x, long long ldx, void* xq, long long ldq, void* sx,
                        long long M, int K, cudaStream_t stream) {
  return ab200_quant_fp8_row_wait(x, ldx, xq, ldq, sx, M, K, nullptr, nullptr, stream);
}

// The same, first waiting (sync->wait_*) until every rank's producer of `x` has signalled.
int ab200_quant_fp8_row_wait(const void* x, long long ldx, void* xq, long long ldq, void* sx,
                             long long M, int K, const Ab200PeerSync* sync, int* status,
                             cudaStream_t stream) {
  if (M <= 0) return 0;
  if ((K % 8) || (ldx % 8) || (ldq % 8) || K > 32768) return -2;
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
  const bf16* xp = reinterpret_cast<const bf16*>(x);
  uint8_t* qp = reinterpret_cast<uint8_t*>(xq);
  float* sp = reinterpret_cast<float*>(sx);
  const int nvec = K / 8;
  if (nvec <= 256)
    (void)launch_pdl(quant_fp8_row_kernel<1>, dim3((unsigned)M), dim3(256), 0, stream,
                     xp, ldx, qp, ldq, sp, K, w, status);
  else if (nvec <= 512)
    (void)launch_pdl(quant_fp8_row_kernel<2>, dim3((unsigned)M), dim3(256), 0, stream,
                     xp, ldx, qp, ldq, sp, K, w, status);
  else if (nvec <= 1024)
    (void)launch_pdl(quant_fp8_row_kernel<4>, dim3((unsigned)M), dim3(256), 0, stream,
                     xp, ldx, qp, ldq, sp, K, w, status);
  else if (nvec <= 2048)
    (void)launch_pdl(quant_fp8_row_kernel<8>, dim3((unsigned)M), dim3(256), 0, stream,
                     xp, ldx, qp, ldq, sp, K, w, status);
  else
    (void)launch_pdl(quant_fp8_row_kernel<8>, dim3((unsigned)M), dim3(512), 0, stream,
                     xp, ldx, qp, ldq, sp, K, w, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// RMSNorm(x (+ residual)) -> yq e4m3 [T, hidden] + sy fp32 [T] (and bf16 y when y != null).
// hidden must be a multiple of 8 and at most 16384.
int ab200_rmsnorm_quant(const void* x, long long ldx, void* residual, const void* weight,
                        void* yq, long long ldq, void* sy, void* y, long long ldy, long long T,
                        int hidden, float eps, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((hidden % 8) || (ldx % 8) || (ldq % 8) || (y != nullptr && (ldy % 8)) || hidden > 16384)
    return -2;
  const bf16* xp = reinterpret_cast<const bf16*>(x);
  bf16* rp = reinterpret_cast<bf16*>(residual);
  const bf16* wp = reinterpret_cast<const bf16*>(weight);
  uint8_t* qp = reinterpret_cast<uint8_t*>(yq);
  float* sp = reinterpret_cast<float*>(sy);
  bf16* yp = reinterpret_cast<bf16*>(y);
  const int nvec = hidden / 8;
#define AB200_LAUNCH_NQ(V)                                                                   \
  (void)launch_pdl(rmsnorm_quant_kernel<V>, dim3((unsigned)T), dim3(kQThreads), 0, stream, xp, \
                   ldx, rp, wp, qp, ldq, sp, yp, ldy, hidden, eps)
  if (nvec <= 256) AB200_LAUNCH_NQ(1);
  else if (nvec <= 512) AB200_LAUNCH_NQ(2);
  else if (nvec <= 1024) AB200_LAUNCH_NQ(4);
  else AB200_LAUNCH_NQ(8);
#undef AB200_LAUNCH_NQ
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// SiLU(gate) * up over nblk fused (gate | up) blocks of width inter -> e4m3 [T, nblk * inter]
// + one scale per token.
int ab200_silu_mul_quant(const void* x, void* outq, long long ldq, void* so, long long T,
                         int inter, int nblk, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((inter % 8) || (ldq % 8) || nblk < 1) return -2;
  const bf16* xp = reinterpret_cast<const bf16*>(x);
  uint8_t* qp = reinterpret_cast<uint8_t*>(outq);
  float* sp = reinterpret_cast<float*>(so);
  const size_t smem = (size_t)nblk * inter * 2;
  if (smem > 200 * 1024) return -2;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -3;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(silu_mul_quant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             200 * 1024) != cudaSuccess)
      return -3;
    attr_set[dev] = true;
  }
  (void)launch_pdl(silu_mul_quant_kernel, dim3((unsigned)T), dim3(kSiluQThreads), smem, stream,
                   xp, qp, ldq, sp, inter, nblk);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // extern "C"
