// Per-head RMSNorm of the query and key heads (Qwen3): every head of head_dim D is
// normalised on its own, y = x * rsqrt(mean(x^2) + eps) * w, with one weight vector [D] for
// all query heads and one for all key heads; it runs between the QKV projection and RoPE.
//
// qkv: [T, (Hq + 2*Hkv) * D] bf16 with row stride ld, updated in place (the value heads are
// not touched). One warp owns one (token, head): a head is 128 or 256 contiguous bytes, so a
// warp's load and store are one or two full 128-byte lines, the row stays in registers, and
// the reduction is five shuffles. In Hugging Face's Qwen3 the two norms are
// `self_attn.q_norm` / `self_attn.k_norm`, applied to the projections reshaped to heads.
//
// With a `sync` the kernel first waits (bounded) until every rank's QKV projection has stored
// its rows here, like the RoPE kernel does when it is the first reader.

#include "api.h"
#include "common/pdl.cuh"
#include "common/peer.cuh"
#include "common/ptx.cuh"

namespace ab200 {
namespace {

typedef __nv_bfloat16 bf16;
constexpr int kWarpsPerBlock = 8;

template <int VEC>  // elements per lane: D / 32
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
qk_norm_kernel(bf16* __restrict__ qkv, long long ld, const bf16* __restrict__ wq,
               const bf16* __restrict__ wk, long long T, int Hq, int heads, float eps, int* status,
               const PeerWait wait) {
  pdl_wait();
  pdl_trigger();
  if (wait.world > 0) {
    __shared__ int peers_ok;
    if (threadIdx.x < 32) {
      const bool ok = wait_peers(wait, status, kWaitLimitNs);
      if (threadIdx.x == 0) peers_ok = ok ? 1 : 0;
    }
    __syncthreads();
    if (!peers_ok) return;
  }
  constexpr int D = VEC * 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * kWarpsPerBlock + warp;
  if (item >= T * heads) return;
  const long long t = item / heads;
  const int j = (int)(item % heads);
  bf16* p = qkv + t * ld + (long long)j * D + lane * VEC;
  const bf16* w = (j < Hq ? wq : wk) + lane * VEC;
  float x[VEC], g[VEC];
  if constexpr (VEC == 4) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const uint2 wraw = *reinterpret_cast<const uint2*>(w);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    const float2 wa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wraw.x));
    const float2 wb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wraw.y));
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
    g[0] = wa.x; g[1] = wa.y; g[2] = wb.x; g[3] = wb.y;
  } else {
    const uint32_t raw = *reinterpret_cast<const uint32_t*>(p);
    const uint32_t wraw = *reinterpret_cast<const uint32_t*>(w);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw));
    const float2 wa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wraw));
    x[0] = a.x; x[1] = a.y;
    g[0] = wa.x; g[1] = wa.y;
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) ss += x[i] * x[i];
  ss = warp_sum(ss);
  const float r = rsqrtf(ss * (1.0f / D) + eps);
  if constexpr (VEC == 4) {
    uint2 out;
    out.x = pack_bf16x2(x[0] * r * g[0], x[1] * r * g[1]);
    out.y = pack_bf16x2(x[2] * r * g[2], x[3] * r * g[3]);
    *reinterpret_cast<uint2*>(p) = out;
  } else {
    *reinterpret_cast<uint32_t*>(p) = pack_bf16x2(x[0] * r * g[0], x[1] * r * g[1]);
  }
}

}  // namespace
}  // namespace ab200

using namespace ab200;

extern "C" int ab200_qk_norm(void* qkv, long long ld, const void* wq, const void* wk, long long T,
                             int Hq, int Hkv, int D, float eps, const Ab200PeerSync* sync,
                             int* status, cudaStream_t stream) {
  if (T <= 0 || Hq + Hkv <= 0) return 0;
  if ((D != 64 && D != 128) || (ld % 8) || Hq < 0 || Hkv < 0) return -2;
  if (ld < (long long)(Hq + Hkv) * D) return -2;
  const int heads = Hq + Hkv;
  const long long items = T * heads;
  const long long blocks = (items + kWarpsPerBlock - 1) / kWarpsPerBlock;
  if (blocks > 0x7fffffffll) return -2;
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
  const dim3 grid((unsigned)blocks), block(kWarpsPerBlock * 32);
  if (D == 128) {
    (void)launch_pdl(qk_norm_kernel<4>, grid, block, 0, stream, reinterpret_cast<bf16*>(qkv), ld,
                     reinterpret_cast<const bf16*>(wq), reinterpret_cast<const bf16*>(wk), T, Hq,
                     heads, eps, status, w);
  } else {
    (void)launch_pdl(qk_norm_kernel<2>, grid, block, 0, stream, reinterpret_cast<bf16*>(qkv), ld,
                     reinterpret_cast<const bf16*>(wq), reinterpret_cast<const bf16*>(wk), T, Hq,
                     heads, eps, status, w);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
