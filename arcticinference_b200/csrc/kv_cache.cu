// Paged KV-cache writers beyond the per-layer RoPE+write kernel of elementwise.cu.
//
// 1. Bulk write for SwiftKV. One projection yields K and V of all later layers for every
//    token ([T, L * 2 * Hkv * D], layer j at columns j * 2*Hkv*D, K heads then V heads). One
//    launch rotates every K head and scatters K and V of all L layers into their paged
//    caches [num_blocks, Hkv, block_size, D], as bf16 or as e4m3 with one scale per layer
//    and tensor. The cache base pointers sit in a device table that the engine builds once.
//    (The reference scatters already-rotated rows with one element per thread and uploads the
//    pointer tables on every call: csrc/custom_ops/reshape_and_cache_flash_bulk.cu:12-144.)
//
// 2. NVFP4 cache write. Groups of 16 elements share one e4m3 scale (amax / 6); elements are
//    stored as e2m1 nibbles, even element in the low nibble. Codes [num_blocks, Hkv,
//    block_size, D/2] bytes, scales [num_blocks, Hkv, block_size, D/16] bytes. Two threads per
//    group, 16-byte loads, cvt.rn.satfinite.e2m1x2.f32 for the rounding, 4-byte code stores.
//    (Reference: csrc/custom_ops/reshape_and_cache_flash_fp4.cu:102-254.) A gather kernel
//    expands slots of such a cache back to bf16 rows.

#include <cuda_fp8.h>

#include "api.h"
#include "common/ptx.cuh"

namespace ab200 {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void kv_unpack8(const uint4& q, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ uint4 kv_pack8_bf16(const float (&f)[8]) {
  uint4 q;
  q.x = pack_bf16x2(f[0], f[1]);
  q.y = pack_bf16x2(f[2], f[3]);
  q.z = pack_bf16x2(f[4], f[5]);
  q.w = pack_bf16x2(f[6], f[7]);
  return q;
}

__device__ __forceinline__ uint2 kv_pack8_e4m3(const float (&f)[8], float inv_scale) {
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t b = (uint32_t)__nv_cvt_float_to_fp8(f[i] * inv_scale, __NV_SATFINITE, __NV_E4M3);
    w[i >> 2] |= b << (8 * (i & 3));
  }
  return make_uint2(w[0], w[1]);
}

// grid (T, L); FP8 = 0: bf16 caches, 1: e4m3 caches.
template <int FP8>
__global__ void __launch_bounds__(128)
kv_bulk_write_kernel(const bf16* __restrict__ kv, long long ld,
                     const long long* __restrict__ positions, const long long* __restrict__ slots,
                     const float* __restrict__ inv_freq, const long long* __restrict__ k_ptrs,
                     const long long* __restrict__ v_ptrs, const float* __restrict__ k_scales,
                     const float* __restrict__ v_scales, int Hkv, int D, int block_size,
                     long long num_slots, int* status) {
  extern __shared__ float cs[];  // cos[D/2] | sin[D/2]
  const long long t = blockIdx.x;
  const int layer = blockIdx.y;
  const long long slot = slots[t];
  if (slot < 0) return;  // padding token
  if (slot >= num_slots) {
    if (threadIdx.x == 0) report_error(status, kErrBounds, 2, (int)t);
    return;
  }
  const int half = D / 2;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float s, c;
    sincosf(pos * inv_freq[i], &s, &c);
    cs[i] = c;
    cs[half + i] = s;
  }
  __syncthreads();
  const long long blk = slot / block_size;
  const int off = (int)(slot % block_size);
  const bf16* row = kv + t * ld + (long long)layer * 2 * Hkv * D;
  const float ks = FP8 ? 1.f / k_scales[layer] : 1.f;
  const float vs = FP8 ? 1.f / v_scales[layer] : 1.f;
  const int vec_per_half = half / 8;
  for (int i = threadIdx.x; i < Hkv * vec_per_half; i += blockDim.x) {
    const int h = i / vec_per_half;
    const int c = i % vec_per_half;
    const bf16* base = row + (long long)h * D;
    float a[8], b[8], oa[8], ob[8];
    kv_unpack8(reinterpret_cast<const uint4*>(base)[c], a);
    kv_unpack8(reinterpret_cast<const uint4*>(base + half)[c], b);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float co = cs[c * 8 + k], si = cs[half + c * 8 + k];
      oa[k] = a[k] * co - b[k] * si;
      ob[k] = b[k] * co + a[k] * si;
    }
    const long long e = ((blk * Hkv + h) * block_size + off) * (long long)D;
    if (FP8) {
      uint8_t* dst = reinterpret_cast<uint8_t*>(k_ptrs[layer]) + e;
      // round the rotated value to bf16 first, as the unquantised path stores it
      float ra[8], rb[8];
      const uint4 qa = kv_pack8_bf16(oa), qb = kv_pack8_bf16(ob);
      kv_unpack8(qa, ra);
      kv_unpack8(qb, rb);
      reinterpret_cast<uint2*>(dst)[c] = kv_pack8_e4m3(ra, ks);
      reinterpret_cast<uint2*>(dst + half)[c] = kv_pack8_e4m3(rb, ks);
    } else {
      bf16* dst = reinterpret_cast<bf16*>(k_ptrs[layer]) + e;
      reinterpret_cast<uint4*>(dst)[c] = kv_pack8_bf16(oa);
      reinterpret_cast<uint4*>(dst + half)[c] = kv_pack8_bf16(ob);
    }
  }
  const int vec_per_head = D / 8;
  for (int i = threadIdx.x; i < Hkv * vec_per_head; i += blockDim.x) {
    const int h = i / vec_per_head;
    const int c = i % vec_per_head;
    const uint4 q = reinterpret_cast<const uint4*>(row + (long long)(Hkv + h) * D)[c];
    const long long e = ((blk * Hkv + h) * block_size + off) * (long long)D;
    if (FP8) {
      float f[8];
      kv_unpack8(q, f);
      reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(v_ptrs[layer]) + e)[c] = kv_pack8_e4m3(f, vs);
    } else {
      reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(v_ptrs[layer]) + e)[c] = q;
    }
  }
}

// ---------------------------------------------------------------------------- NVFP4
// Eight floats (already divided by the group scale) -> eight e2m1 nibbles in one word,
// element 0 in the lowest nibble.
__device__ __forceinline__ uint32_t pack8_e2m1(const float (&f)[8]) {
  uint32_t out;
  asm volatile(
      "{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3};\n"
      "}\n"
      : "=r"(out)
      : "f"(f[0]), "f"(f[1]), "f"(f[2]), "f"(f[3]), "f"(f[4]), "f"(f[5]), "f"(f[6]), "f"(f[7]));
  return out;
}

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  const __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&h));
}

// One call writes K and V of one layer. grid (T), 2 threads per 16-element group.
__global__ void __launch_bounds__(256)
kv_write_fp4_kernel(const bf16* __restrict__ k, long long ldk, const bf16* __restrict__ v,
                    long long ldv, const long long* __restrict__ slots,
                    uint8_t* __restrict__ k_codes, uint8_t* __restrict__ v_codes,
                    uint8_t* __restrict__ k_scales, uint8_t* __restrict__ v_scales, int Hkv, int D,
                    int block_size, long long num_slots, int* status) {
  const long long t = blockIdx.x;
  const long long slot = slots[t];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) report_error(status, kErrBounds, 3, (int)t);
    return;
  }
  const long long blk = slot / block_size;
  const int off = (int)(slot % block_size);
  const int vec_per_head = D / 8;          // even: D is a multiple of 16
  const int items = 2 * Hkv * vec_per_head;  // K then V
  // the loop bound is rounded up to a multiple of 2 lanes so that both lanes of a group
  // reach the shuffle together
  for (int i0 = 0; i0 < items; i0 += blockDim.x) {
    const int i = i0 + threadIdx.x;
    const bool live = i < items;
    const int which = live ? i / (Hkv * vec_per_head) : 0;
    const int j = live ? i % (Hkv * vec_per_head) : 0;
    const int h = j / vec_per_head;
    const int c = j % vec_per_head;
    const bf16* src = which ? v + t * ldv : k + t * ldk;
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (live) kv_unpack8(reinterpret_cast<const uint4*>(src + (long long)h * D)[c], f);
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const uint8_t sb = (uint8_t)__nv_cvt_float_to_fp8(amax * (1.f / 6.f), __NV_SATFINITE, __NV_E4M3);
    const float sd = e4m3_to_float(sb);
    const float inv = sd > 0.f ? 1.f / sd : 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] *= inv;
    const uint32_t codes = pack8_e2m1(f);
    if (live) {
      const long long row = (blk * Hkv + h) * block_size + off;
      uint8_t* cdst = (which ? v_codes : k_codes) + row * (D / 2);
      reinterpret_cast<uint32_t*>(cdst)[c] = codes;
      if ((c & 1) == 0) ((which ? v_scales : k_scales) + row * (D / 16))[c >> 1] = sb;
    }
  }
}

__device__ __forceinline__ float e2m1_to_float(uint32_t nib) {
  // 0, 0.5, 1, 1.5, 2, 3, 4, 6 with a sign bit
  const uint32_t m = nib & 7u;
  const float mag = m < 2u ? 0.5f * (float)m
                           : (float)(2u | (m & 1u)) * (float)(1u << ((m >> 1) - 1u)) * 0.5f;
  return (nib & 8u) ? -mag : mag;
}

// rows of one fp4 cache tensor at the given slots -> bf16 [R, Hkv * D]
__global__ void __launch_bounds__(256)
kv_read_fp4_kernel(const uint8_t* __restrict__ codes, const uint8_t* __restrict__ scales,
                   const long long* __restrict__ slots, bf16* __restrict__ out, long long ldo,
                   int Hkv, int D, int block_size) {
  const long long r = blockIdx.x;
  const long long slot = slots[r];
  if (slot < 0) return;
  const long long blk = slot / block_size;
  const int off = (int)(slot % block_size);
  const int vec_per_head = D / 8;
  for (int i = threadIdx.x; i < Hkv * vec_per_head; i += blockDim.x) {
    const int h = i / vec_per_head;
    const int c = i % vec_per_head;
    const long long row = (blk * Hkv + h) * block_size + off;
    const uint32_t w = reinterpret_cast<const uint32_t*>(codes + row * (D / 2))[c];
    const float s = e4m3_to_float(scales[row * (D / 16) + (c >> 1)]);
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = e2m1_to_float((w >> (4 * e)) & 15u) * s;
    reinterpret_cast<uint4*>(out + r * ldo + (long long)h * D)[c] = kv_pack8_bf16(f);
  }
}

}  // namespace ab200

using namespace ab200;

extern "C" {

int ab200_kv_bulk_write(const void* kv, long long ld, const void* positions, const void* slots,
                        const void* inv_freq, const void* k_ptrs, const void* v_ptrs,
                        const void* k_scales, const void* v_scales, long long T, int L, int Hkv,
                        int D, int block_size, long long num_slots, int fp8, int* status,
                        cudaStream_t stream) {
  if (T <= 0 || L <= 0) return 0;
  if ((D % 16) || (ld % 8) || L > 65535) return -2;
  if (fp8 && (k_scales == nullptr || v_scales == nullptr)) return -2;
  const dim3 grid((unsigned)T, (unsigned)L);
  const size_t smem = D * sizeof(float);
  if (fp8)
    kv_bulk_write_kernel<1><<<grid, 128, smem, stream>>>(
        reinterpret_cast<const bf16*>(kv), ld, reinterpret_cast<const long long*>(positions),
        reinterpret_cast<const long long*>(slots), reinterpret_cast<const float*>(inv_freq),
        reinterpret_cast<const long long*>(k_ptrs), reinterpret_cast<const long long*>(v_ptrs),
        reinterpret_cast<const float*>(k_scales), reinterpret_cast<const float*>(v_scales), Hkv, D,
        block_size, num_slots, status);
  else
    kv_bulk_write_kernel<0><<<grid, 128, smem, stream>>>(
        reinterpret_cast<const bf16*>(kv), ld, reinterpret_cast<const long long*>(positions),
        reinterpret_cast<const long long*>(slots), reinterpret_cast<const float*>(inv_freq),
        reinterpret_cast<const long long*>(k_ptrs), reinterpret_cast<const long long*>(v_ptrs),
        nullptr, nullptr, Hkv, D, block_size, num_slots, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_kv_write_fp4(const void* k, long long ldk, const void* v, long long ldv,
                       const void* slots, void* k_codes, void* v_codes, void* k_scales,
                       void* v_scales, long long T, int Hkv, int D, int block_size,
                       long long num_slots, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((D % 16) || (ldk % 8) || (ldv % 8)) return -2;
  kv_write_fp4_kernel<<<(unsigned)T, 256, 0, stream>>>(
      reinterpret_cast<const bf16*>(k), ldk, reinterpret_cast<const bf16*>(v), ldv,
      reinterpret_cast<const long long*>(slots), reinterpret_cast<uint8_t*>(k_codes),
      reinterpret_cast<uint8_t*>(v_codes), reinterpret_cast<uint8_t*>(k_scales),
      reinterpret_cast<uint8_t*>(v_scales), Hkv, D, block_size, num_slots, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_kv_read_fp4(const void* codes, const void* scales, const void* slots, void* out,
                      long long ldo, long long R, int Hkv, int D, int block_size,
                      cudaStream_t stream) {
  if (R <= 0) return 0;
  if ((D % 16) || (ldo % 8)) return -2;
  kv_read_fp4_kernel<<<(unsigned)R, 256, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(codes), reinterpret_cast<const uint8_t*>(scales),
      reinterpret_cast<const long long*>(slots), reinterpret_cast<bf16*>(out), ldo, Hkv, D,
      block_size);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // extern "C"
