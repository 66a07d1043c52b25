// Block-scaled fp8 linear layer for sm_100a:
//   out[M,N] = (xq[M,K] * sx[M, K/128]) . (wq[N,K] * sw[N/128, K/128])^T
// wq: e4m3 weights with one fp32 scale per 128x128 block (the checkpoint format of
// block-quantised fp8 models); xq: e4m3 activations with one scale per token and 128
// consecutive k (produced by quant_fp8_kernel below, or fused into the producer).
//
// Tensor cores cannot apply a scale that changes along K, so the K loop is cut at the
// scale granularity: each 128-wide k-block is one tcgen05.mma group (kind::f8f6f4,
// 4 x K=32) into one of two TMEM buffers, and eight epilogue warps fold finished
// buffers into fp32 registers with the block's scale (acc += s * partial) while the
// tensor core works on the next k-block. Two epilogue warps share each TMEM lane
// quadrant and take half of the columns each, so a thread carries at most 128
// accumulators.
//
// Orientations as in gemm_bf16.cu: token-major (M > 128: 128 tokens x 256 features per
// tile, the scale is one scalar per thread and k-block) and feature-major (M <= 128:
// 128 weight rows x all tokens, with split-K into an fp32 scratch buffer when N/128
// alone cannot fill the GPU).
//
// The reference reaches fp8 linears through vLLM (arctic_inference/vllm/spec_dec/fp8.py:
// 282-309, apply_w8a8_block_fp8_linear) and ops.scaled_fp8_quant.

#include <cuda_fp8.h>
#include <math.h>
#include <string.h>

#include "api.h"
#include "common/ptx.cuh"
#include "common/tensormap.h"

namespace ab200 {

constexpr int kF8Threads = 320;  // TMA warp, MMA warp, 8 epilogue warps
constexpr int kF8BlockK = 128;   // fp8 elements per stage row = one 128-byte swizzle atom
constexpr int kF8MaxStages = 8;
constexpr uint32_t kF8ABytes = 128 * 128;

struct Fp8Args {
  int rows_a, rows_b, K;
  int bn, stages, splits, kblocks_per_split, kblocks_total;
  int tiles_a, tiles_b;
  int transposed;   // feature-major: A = weights, out[b_row*ldo + a_row]
  int out_f32;      // split-K partials
  long long ldo, partial_stride;
  void* out;
  const float* sx_t;  // [K/128][ld_sx] activation scales, token index contiguous
  long long ld_sx;
  const float* sw;    // [N/128][ld_sw] weight block scales
  long long ld_sw;
  int* status;
  int peer_cols;
  long long peer_row_off;
  __nv_bfloat16* peer_out[16];
};

__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a,
                const __grid_constant__ CUtensorMap tmap_b, const Fp8Args p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t b_bytes = (uint32_t)p.bn * kF8BlockK;
  const uint32_t stage_bytes = kF8ABytes + b_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)p.stages * stage_bytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kF8MaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bb = smem_u32(bars);
  auto full_bar = [&](int s) { return bb + 8u * s; };
  auto empty_bar = [&](int s) { return bb + 8u * (kF8MaxStages + s); };
  auto tfull_bar = [&](int a) { return bb + 8u * (2 * kF8MaxStages + a); };
  auto tempty_bar = [&](int a) { return bb + 8u * (2 * kF8MaxStages + 2 + a); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int total_work = p.tiles_a * p.tiles_b * p.splits;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int tile_a = w % p.tiles_a;
        const int rest = w / p.tiles_a;
        const int tile_b = rest % p.tiles_b;
        const int split = rest / p.tiles_b;
        const int kb0 = split * p.kblocks_per_split;
        const int kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 1100 + stage, kb)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full_bar(stage), stage_bytes);
          const uint32_t dst = smem_base + (uint32_t)stage * stage_bytes;
          tma_load_2d(dst, &tmap_a, full_bar(stage), kb * kF8BlockK, tile_a * 128);
          tma_load_2d(dst + kF8ABytes, &tmap_b, full_bar(stage), kb * kF8BlockK, tile_b * p.bn);
          ++issued;
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        const int pending = (int)min((long long)p.stages, issued);
        int s = stage;
        uint32_t ph = phase;
        for (int i = 0; i < pending; ++i) {
          if (--s < 0) {
            s = p.stages - 1;
            ph ^= 1u;
          }
          mbar_drain(full_bar(s), ph);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(128, (uint32_t)p.bn, 0, 0, 0, 0);  // e4m3 x e4m3 -> f32
      int stage = 0;
      uint32_t phase = 0;
      uint32_t it = 0;  // k-blocks issued by this CTA: selects the TMEM buffer
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int split = (w / p.tiles_a) / p.tiles_b;
        const int kb0 = split * p.kblocks_per_split;
        const int kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int buf = it & 1;
          const uint32_t bph = (it >> 1) & 1u;
          if (!mbar_wait(tempty_bar(buf), bph ^ 1u, abort_flag, p.status, 1200 + buf, kb) ||
              !mbar_wait(full_bar(stage), phase, abort_flag, p.status, 1300 + stage, kb)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_base + (uint32_t)stage * stage_bytes;
          const uint64_t a_desc = make_desc_kmajor_sw128(a_addr);
          const uint64_t b_desc = make_desc_kmajor_sw128(a_addr + kF8ABytes);
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 32 fp8 = 32 bytes further inside the swizzle atom
            umma_f8_ss(tmem_base + (uint32_t)buf * 256u, a_desc + (uint64_t)(2 * k),
                       b_desc + (uint64_t)(2 * k), idesc, k > 0 ? 1u : 0u);
          tc_commit(empty_bar(stage));
          tc_commit(tfull_bar(buf));
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else {
    // ---- epilogue: warps 2..9; two warps per TMEM lane quadrant, half of the columns each
    const int e = warp - 2;
    const int quad = warp & 3;
    const int half = e >> 2;
    const int row = quad * 32 + lane;
    const int ncols = p.bn / 2;            // columns this thread accumulates (multiple of 16)
    const int col0 = half * ncols;
    uint32_t it = 0;
    for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
      const int tile_a = w % p.tiles_a;
      const int rest = w / p.tiles_a;
      const int tile_b = rest % p.tiles_b;
      const int split = rest / p.tiles_b;
      const int kb0 = split * p.kblocks_per_split;
      const int kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
      const long long a_row = (long long)tile_a * 128 + row;
      const bool row_ok = a_row < p.rows_a;
      const long long b0 = (long long)tile_b * p.bn + col0;
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      bool ok = true;
      // Scales are fetched one k-block ahead, before the wait on the accumulator, so that
      // their global-memory latency hides behind the tensor core's work on that block.
      const long long nblk = b0 / 128;
      auto load_sw = [&](int kb) -> float {
        if (!p.transposed) return (b0 < p.rows_b) ? p.sw[nblk * p.ld_sw + kb] : 0.f;
        return row_ok ? p.sw[(long long)tile_a * p.ld_sw + kb] : 0.f;
      };
      auto load_sx = [&](int kb) -> float {
        return (!p.transposed && row_ok) ? p.sx_t[(long long)kb * p.ld_sx + a_row] : 0.f;
      };
      float sw_next = load_sw(kb0), sx_next = load_sx(kb0);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int buf = it & 1;
        const uint32_t bph = (it >> 1) & 1u;
        const float sw_s = sw_next;
        const float s_row = sx_next * sw_next;
        if (kb + 1 < kb1) {
          sw_next = load_sw(kb + 1);
          sx_next = load_sx(kb + 1);
        }
        if (!mbar_wait(tfull_bar(buf), bph, abort_flag, p.status, 1400 + buf, kb)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t t_addr =
            tmem_base + (uint32_t)buf * 256u + (uint32_t)col0 + ((uint32_t)(quad * 32) << 16);
        const float* sx_kb = p.sx_t + (long long)kb * p.ld_sx;
#pragma unroll
        for (int c = 0; c < 8; c += 2) {
          if (c * 16 < ncols) {
            // two 16-column loads in flight per wait
            uint32_t r[2][16];
            const bool two = (c + 1) * 16 < ncols;
            __syncwarp();
            tmem_ld_x16(t_addr + (uint32_t)c * 16u, r[0]);
            if (two) tmem_ld_x16(t_addr + (uint32_t)(c + 1) * 16u, r[1]);
            tmem_ld_wait();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              if (h == 1 && !two) break;
              const int cc = c + h;
              if (!p.transposed) {
#pragma unroll
                for (int t = 0; t < 16; ++t)
                  acc[cc * 16 + t] = fmaf(s_row, __uint_as_float(r[h][t]), acc[cc * 16 + t]);
              } else {
#pragma unroll
                for (int t = 0; t < 16; ++t) {
                  const long long tok = b0 + cc * 16 + t;
                  const float s = tok < p.rows_b ? sx_kb[tok] * sw_s : 0.f;
                  acc[cc * 16 + t] = fmaf(s, __uint_as_float(r[h][t]), acc[cc * 16 + t]);
                }
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(buf));
      }
      if (!ok) break;
      if (!row_ok) continue;
      // ---- store
      if (p.out_f32) {
        float* o = reinterpret_cast<float*>(p.out) + (long long)split * p.partial_stride;
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          if (i < ncols) {
            const long long b_row = b0 + i;
            if (b_row < p.rows_b) {
              if (p.transposed) o[b_row * p.ldo + a_row] = acc[i];
              else o[a_row * p.ldo + b_row] = acc[i];
            }
          }
        }
      } else if (!p.transposed) {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + a_row * p.ldo + b0;
        if (p.peer_cols > 0)
          dst = p.peer_out[b0 / p.peer_cols] + (a_row + p.peer_row_off) * p.ldo + b0 % p.peer_cols;
#pragma unroll
        for (int i = 0; i < 128; i += 8) {
          if (i < ncols && b0 + i + 8 <= p.rows_b) {
            uint4 q;
            q.x = pack_bf16x2(acc[i], acc[i + 1]);
            q.y = pack_bf16x2(acc[i + 2], acc[i + 3]);
            q.z = pack_bf16x2(acc[i + 4], acc[i + 5]);
            q.w = pack_bf16x2(acc[i + 6], acc[i + 7]);
            *reinterpret_cast<uint4*>(dst + i) = q;
          }
        }
      } else {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out);
        long long o_col = a_row, o_off = 0;
        if (p.peer_cols > 0) {
          o = p.peer_out[a_row / p.peer_cols];
          o_col = a_row % p.peer_cols;
          o_off = p.peer_row_off;
        }
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          if (i < ncols) {
            const long long b_row = b0 + i;
            if (b_row < p.rows_b) o[(b_row + o_off) * p.ldo + o_col] = __float2bfloat16(acc[i]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------ W8A16 (decode)
// Few tokens (M <= 128): the GEMM is bound by streaming the weights, so only their size
// matters. Weight tiles arrive as fp8 (TMA), eight converter warps expand them to bf16 with
// the block scale applied (read the swizzled fp8 tile, write a swizzled bf16 tile), and the
// tensor core runs a plain bf16 UMMA against the un-quantised bf16 activations, accumulating
// over all of K in TMEM. No activation quantisation, no per-block rescaling, half the bytes.
constexpr int kWaConvWarps = 16;  // the expansion is latency bound: 4 warps per scheduler hide it
constexpr int kWaConvBufs = 4;    // converted k-blocks in flight between converters and MMA
constexpr int kWaThreads = 64 + 32 * kWaConvWarps + 128;  // TMA, MMA, converters, 4 epilogue warps
constexpr uint32_t kWaConvBytes = 128 * 256;  // one converted k-block: 128 rows x 128 k bf16

struct WaArgs {
  int N, M, K;
  int bn, stages, splits, kblocks_per_split, kblocks_total, tiles;
  int out_f32;
  long long ldo, partial_stride;
  void* out;
  const float* sw;
  long long ld_sw;
  int* status;
  int peer_cols;
  long long peer_row_off;
  __nv_bfloat16* peer_out[16];
};

__global__ void __launch_bounds__(kWaThreads, 1)
gemm_w8a16_kernel(const __grid_constant__ CUtensorMap tmap_w,
                  const __grid_constant__ CUtensorMap tmap_x, const WaArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t x_bytes = (uint32_t)p.bn * 256u;        // two 64-wide k atoms of bn rows
  const uint32_t raw_bytes = kF8ABytes + x_bytes;
  uint8_t* conv = smem + (size_t)p.stages * raw_bytes;   // converted buffers
  uint64_t* bars = reinterpret_cast<uint64_t*>(conv + kWaConvBufs * kWaConvBytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kF8MaxStages + 2 * kWaConvBufs + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t conv_base = smem_u32(conv);
  const uint32_t bb = smem_u32(bars);
  auto full_bar = [&](int s) { return bb + 8u * s; };
  auto empty_bar = [&](int s) { return bb + 8u * (kF8MaxStages + s); };
  auto cfull_bar = [&](int c) { return bb + 8u * (2 * kF8MaxStages + c); };
  auto cempty_bar = [&](int c) { return bb + 8u * (2 * kF8MaxStages + kWaConvBufs + c); };
  auto tfull_bar = [&](int a) { return bb + 8u * (2 * kF8MaxStages + 2 * kWaConvBufs + a); };
  auto tempty_bar = [&](int a) { return bb + 8u * (2 * kF8MaxStages + 2 * kWaConvBufs + 2 + a); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t tmem_cols = p.bn <= 16 ? 32u : (p.bn <= 32 ? 64u : (p.bn <= 64 ? 128u : 256u));

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int c = 0; c < kWaConvBufs; ++c) {
      mbar_init(cfull_bar(c), kWaConvWarps);
      mbar_init(cempty_bar(c), 1);
    }
    for (int c = 0; c < 2; ++c) {
      mbar_init(tfull_bar(c), 1);
      mbar_init(tempty_bar(c), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_w);
    prefetch_tensormap(&tmap_x);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t acc_stride = tmem_cols / 2;
  const int total_work = p.tiles * p.splits;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int tile = w % p.tiles;
        const int split = w / p.tiles;
        const int kb0 = split * p.kblocks_per_split;
        const int kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 2100 + stage, kb)) {
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(full_bar(stage), raw_bytes);
          const uint32_t dst = smem_base + (uint32_t)stage * raw_bytes;
          tma_load_2d(dst, &tmap_w, full_bar(stage), kb * 128, tile * 128);
          tma_load_2d(dst + kF8ABytes, &tmap_x, full_bar(stage), kb * 128, 0);
          tma_load_2d(dst + kF8ABytes + (uint32_t)p.bn * 128u, &tmap_x, full_bar(stage),
                      kb * 128 + 64, 0);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // A = converted weights (bf16), B = activations (bf16)
      const uint32_t idesc = make_idesc(128, (uint32_t)p.bn, 1, 1, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t it = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int split = w / p.tiles;
        const int kb0 = split * p.kblocks_per_split;
        const int kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 2200 + acc, w)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * acc_stride;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int c = it % kWaConvBufs;
          const uint32_t cph = (it / kWaConvBufs) & 1u;
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 2300 + stage, kb) ||
              !mbar_wait(cfull_bar(c), cph, abort_flag, p.status, 2400 + c, kb)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = conv_base + (uint32_t)c * kWaConvBytes;
          const uint32_t x_addr = smem_base + (uint32_t)stage * raw_bytes + kF8ABytes;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint64_t ad = make_desc_kmajor_sw128(a_addr + (uint32_t)(k / 4) * 16384u) + 2u * (k % 4);
            const uint64_t bd =
                make_desc_kmajor_sw128(x_addr + (uint32_t)(k / 4) * (uint32_t)p.bn * 128u) + 2u * (k % 4);
            umma_f16_ss(d_tmem, ad, bd, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          tc_commit(empty_bar(stage));
          tc_commit(cempty_bar(c));
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit(tfull_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp < 2 + kWaConvWarps) {
    // ------------------------------ converters: fp8 tile -> scaled bf16 tile ------------------
    const int ct = threadIdx.x - 64;  // 0 .. 32 * kWaConvWarps - 1
    int stage = 0;
    uint32_t phase = 0;
    uint32_t it = 0;
    bool ok = true;
    float s_lane = 0.f;
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      const int tile = w % p.tiles;
      const int split = w / p.tiles;
      const int kb0 = split * p.kblocks_per_split;
      const int kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int c = it % kWaConvBufs;
        const uint32_t cph = (it / kWaConvBufs) & 1u;
        // e4m3 -> bf16 without conversion instructions: the 7 magnitude bits of an e4m3 byte,
        // shifted into a bf16's exponent/mantissa position, read as the same value times 2^-120
        // (bias 7 vs 127; subnormals line up too), so one packed bf16 multiply by
        // (block scale * 2^120) finishes the job. Integer ops and HMUL2 run at full rate, the
        // cvt path would not. Block scales come 32 k-blocks at a time, one per lane.
        if (((kb - kb0) & 31) == 0)
          s_lane = (kb + lane < kb1) ? p.sw[(long long)tile * p.ld_sw + kb + lane] : 0.f;
        const float s = __shfl_sync(0xffffffffu, s_lane, (kb - kb0) & 31) * 1.329227995784916e36f;
        const __nv_bfloat162 s2 = __float2bfloat162_rn(s);
        if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 2500 + stage, kb) ||
            !mbar_wait(cempty_bar(c), cph ^ 1u, abort_flag, p.status, 2600 + c, kb)) {
          ok = false;
          break;
        }
        const uint8_t* raw = smem + (size_t)stage * raw_bytes;
        uint8_t* dst = conv + (size_t)c * kWaConvBytes;
        // 128 rows x 16 eight-byte pieces of fp8: sixteen lanes read one row's 128 bytes, eight
        // lanes write one row's eight 16-byte chunks of an atom (no bank conflicts)
#pragma unroll
        for (int u = 0; u < 2048 / (32 * kWaConvWarps); ++u) {
          const int task = ct + u * (32 * kWaConvWarps);
          const int r = task >> 4;
          const int h = task & 15;
          const uint2 q = *reinterpret_cast<const uint2*>(raw + r * 128 + (((h >> 1) ^ (r & 7)) << 4) +
                                                          ((h & 1) << 3));
          const uint32_t in[2] = {q.x, q.y};
          uint32_t o[4];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const uint32_t lo = __byte_perm(in[e], 0u, 0x4140);  // bytes 0,1 -> bits 0..7, 16..23
            const uint32_t hi = __byte_perm(in[e], 0u, 0x4342);  // bytes 2,3
            const uint32_t blo = ((lo << 8) & 0x80008000u) | ((lo << 4) & 0x07F007F0u);
            const uint32_t bhi = ((hi << 8) & 0x80008000u) | ((hi << 4) & 0x07F007F0u);
            const __nv_bfloat162 vlo = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&blo), s2);
            const __nv_bfloat162 vhi = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&bhi), s2);
            o[2 * e] = *reinterpret_cast<const uint32_t*>(&vlo);
            o[2 * e + 1] = *reinterpret_cast<const uint32_t*>(&vhi);
          }
          // k = 8 h .. 8 h + 7 -> atom h / 8, logical chunk h % 8
          *reinterpret_cast<uint4*>(dst + (size_t)(h >> 3) * 16384 + r * 128 + (((h & 7) ^ (r & 7)) << 4)) =
              make_uint4(o[0], o[1], o[2], o[3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(cfull_bar(c));
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else {
    // --------------------------------- epilogue (out^T in TMEM) -------------------------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
      const int tile = w % p.tiles;
      const int split = w / p.tiles;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, 2700 + acc, w)) break;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (uint32_t)acc * acc_stride + ((uint32_t)(quad * 32) << 16);
      const long long n = (long long)tile * 128 + row;
      const bool row_ok = n < p.N;
      for (int c0 = 0; c0 < p.bn; c0 += 16) {
        uint32_t r[16];
        __syncwarp();
        tmem_ld_x16(t_addr + (uint32_t)c0, r);
        tmem_ld_wait();
        if (!row_ok) continue;
        if (p.out_f32) {
          float* o = reinterpret_cast<float*>(p.out) + (long long)split * p.partial_stride;
#pragma unroll
          for (int t = 0; t < 16; ++t)
            if (c0 + t < p.M) o[(long long)(c0 + t) * p.ldo + n] = __uint_as_float(r[t]);
        } else {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out);
          long long o_col = n, o_off = 0;
          if (p.peer_cols > 0) {
            o = p.peer_out[n / p.peer_cols];
            o_col = n % p.peer_cols;
            o_off = p.peer_row_off;
          }
#pragma unroll
          for (int t = 0; t < 16; ++t)
            if (c0 + t < p.M)
              o[(long long)(c0 + t + o_off) * p.ldo + o_col] = __float2bfloat16(__uint_as_float(r[t]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// partial[s][m][n] -> bf16 out[m][n]
__global__ void fp8_splitk_reduce_kernel(const float* __restrict__ partial, int splits,
                                         long long stride, int M, int N,
                                         __nv_bfloat16* __restrict__ out, long long ldo) {
  const long long n4 = N / 4;
  const long long total = (long long)M * n4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / n4, n = (i % n4) * 4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(partial + s * stride + m * (long long)N + n);
      a.x += v.x;
      a.y += v.y;
      a.z += v.z;
      a.w += v.w;
    }
    uint2 q;
    q.x = pack_bf16x2(a.x, a.y);
    q.y = pack_bf16x2(a.z, a.w);
    *reinterpret_cast<uint2*>(out + m * ldo + n) = q;
  }
}

// ------------------------------------------------------------------ activation quantisation
// x [M, K] bf16 (row stride ldx) -> xq [M, K] e4m3, sx_t [K/128][ld_sx] fp32 with
// sx = max(|x|) / 448 per (token, 128-wide k group). 16 threads per group, 8 elements each.
__global__ void __launch_bounds__(256)
quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, long long ldx, uint8_t* __restrict__ xq,
                 long long ldq, float* __restrict__ sx_t, long long ld_sx, long long M, int K) {
  const int groups_per_row = K / 128;
  const long long total_groups = M * groups_per_row;
  const long long gid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) / 16;
  const int sub = threadIdx.x & 15;
  if (gid >= total_groups) return;
  const long long m = gid / groups_per_row;
  const int g = (int)(gid % groups_per_row);
  const uint4 raw = *reinterpret_cast<const uint4*>(x + m * ldx + (long long)g * 128 + sub * 8);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float v[8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
    amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
  }
  // the other 16-thread group of this warp may have left already (tail): shuffle within ours
  const unsigned gmask = (threadIdx.x & 16) ? 0xffff0000u : 0x0000ffffu;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, o, 16));
  const float scale = fmaxf(amax, 1e-10f) / 448.f;
  const float inv = 1.f / scale;
  uint2 q;
  uint32_t w[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const __nv_fp8x2_storage_t lo =
        __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i] * inv, v[4 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi =
        __nv_cvt_float2_to_fp8x2(make_float2(v[4 * i + 2] * inv, v[4 * i + 3] * inv), __NV_SATFINITE, __NV_E4M3);
    w[i] = (uint32_t)lo | ((uint32_t)hi << 16);
  }
  q.x = w[0];
  q.y = w[1];
  *reinterpret_cast<uint2*>(xq + m * ldq + (long long)g * 128 + sub * 8) = q;
  if (sub == 0) sx_t[(long long)g * ld_sx + m] = scale;
}

// wq [N, K] e4m3 (row stride ldw) with 128x128 block scales -> bf16 [N, K] (row stride ldo).
// Used when a long prefill amortises one expansion of the weight over thousands of tokens.
__global__ void __launch_bounds__(256)
dequant_fp8_kernel(const uint8_t* __restrict__ wq, long long ldw, const float* __restrict__ sw,
                   long long ld_sw, __nv_bfloat16* __restrict__ out, long long ldo, long long N,
                   int K) {
  const long long vec_per_row = K / 16;
  const long long total = N * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long n = i / vec_per_row;
    const long long k = (i % vec_per_row) * 16;
    const float s = sw[(n / 128) * ld_sw + k / 128];
    const uint4 raw = *reinterpret_cast<const uint4*>(wq + n * ldw + k);
    const __nv_fp8x2_storage_t* p2 = reinterpret_cast<const __nv_fp8x2_storage_t*>(&raw);
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(p2[j], __NV_E4M3);
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
      o[j] = pack_bf16x2(f.x * s, f.y * s);
    }
    uint4* dst = reinterpret_cast<uint4*>(out + n * ldo + k);
    dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
    dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

static int f8_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace ab200

using namespace ab200;

extern "C" {

int ab200_quant_fp8(const void* x, long long ldx, void* xq, long long ldq, void* sx_t,
                    long long ld_sx, long long M, int K, cudaStream_t stream) {
  if (M <= 0) return 0;
  if ((K % 128) || (ldx % 8) || (ldq % 16)) return -2;
  const long long threads = M * (K / 128) * 16;
  quant_fp8_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<uint8_t*>(xq), ldq,
      reinterpret_cast<float*>(sx_t), ld_sx, M, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_dequant_fp8(const void* wq, long long ldw, const void* sw, long long ld_sw, void* out,
                      long long ldo, long long N, int K, cudaStream_t stream) {
  if (N <= 0) return 0;
  if ((K % 128) || (ldw % 16) || (ldo % 8)) return -2;
  const long long total = N * (K / 16);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  dequant_fp8_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(wq), ldw, reinterpret_cast<const float*>(sw), ld_sw,
      reinterpret_cast<__nv_bfloat16*>(out), ldo, N, K);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// Weight-only fp8 linear for few tokens: x bf16 [M, K] (M <= 128), wq/sw as above.
int ab200_linear_w8a16(const void* x, long long ldx, const void* wq, long long ldw, const void* sw,
                       long long ld_sw, void* out, long long ldo, int M, int N, int K,
                       void* workspace, size_t workspace_bytes, int force_splits,
                       const void* const* peer_ptrs, int world, int peer_cols,
                       long long peer_row_off, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (M > 128 || (K % 128) || (N % 128) || (ldx % 8) || (ldw % 16) ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(wq) & 15))
    return -2;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -3;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_w8a16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             227 * 1024) != cudaSuccess)
      return -3;
    attr_set[dev] = true;
  }
  WaArgs a;
  memset(&a, 0, sizeof(a));
  a.N = N;
  a.M = M;
  a.K = K;
  a.bn = ((M + 15) / 16) * 16;
  a.kblocks_total = K / 128;
  a.tiles = N / 128;
  a.sw = reinterpret_cast<const float*>(sw);
  a.ld_sw = ld_sw;
  a.status = status;
  a.out = out;
  a.ldo = ldo;
  if (peer_cols > 0) {
    if (world < 1 || world > 16 || (peer_cols % 128) || N != world * peer_cols) return -2;
    a.peer_cols = peer_cols;
    a.peer_row_off = peer_row_off;
    for (int i = 0; i < world; ++i)
      a.peer_out[i] = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(peer_ptrs[i]));
    force_splits = 1;
  }
  const int sms = f8_sms();
  int splits = force_splits;
  if (splits <= 0) {
    splits = 1;
    while (a.tiles * splits * 2 <= sms + sms / 4 && splits < 8 && a.kblocks_total / (splits * 2) >= 4)
      splits *= 2;
  }
  if (splits > 8) splits = 8;
  if (splits > a.kblocks_total) splits = a.kblocks_total;
  if (splits > 1 && (workspace == nullptr || workspace_bytes < (size_t)splits * M * N * sizeof(float)))
    splits = 1;
  a.kblocks_per_split = (a.kblocks_total + splits - 1) / splits;
  a.splits = (a.kblocks_total + a.kblocks_per_split - 1) / a.kblocks_per_split;
  const int raw_bytes = (int)kF8ABytes + a.bn * 256;
  a.stages = (227 * 1024 - 2048 - kWaConvBufs * (int)kWaConvBytes) / raw_bytes;
  if (a.stages > kF8MaxStages) a.stages = kF8MaxStages;
  if (a.stages < 2) return -2;
  void* final_out = out;
  if (a.splits > 1) {
    a.out_f32 = 1;
    a.out = workspace;
    a.ldo = N;
    a.partial_stride = (long long)M * N;
  }
  CUtensorMap tw, tx;
  if (make_tmap_2d(&tw, wq, CU_TENSOR_MAP_DATA_TYPE_UINT8, (uint64_t)N, (uint64_t)K, (uint64_t)ldw,
                   128, 128) != 0)
    return -4;
  if (make_tmap_2d(&tx, x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (uint64_t)M, (uint64_t)K,
                   (uint64_t)ldx * 2, (uint32_t)a.bn, 64) != 0)
    return -4;
  const int total = a.tiles * a.splits;
  const int grid = total < sms ? total : sms;
  const size_t smem = (size_t)a.stages * raw_bytes + kWaConvBufs * kWaConvBytes + 512 + 1024;
  gemm_w8a16_kernel<<<grid, kWaThreads, smem, stream>>>(tw, tx, a);
  if (cudaGetLastError() != cudaSuccess) return -5;
  if (a.splits > 1) {
    const long long total4 = (long long)M * (N / 4);
    int blocks = (int)((total4 + 255) / 256);
    if (blocks > sms * 8) blocks = sms * 8;
    fp8_splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const float*>(workspace), a.splits, a.partial_stride, M, N,
        reinterpret_cast<__nv_bfloat16*>(final_out), ldo);
    if (cudaGetLastError() != cudaSuccess) return -5;
  }
  return 0;
}

size_t ab200_linear_fp8_workspace_bytes(int M, int N, int K) {
  (void)K;
  if (M > 128) return 0;
  return (size_t)8 * (size_t)M * (size_t)N * sizeof(float);
}

// xq [M,K] e4m3 (row stride ldxq bytes), sx_t [K/128][ld_sx]; wq [N,K] e4m3 (row stride ldw),
// sw [N/128][ld_sw]; out bf16 [M,N] (row stride ldo), or scattered to peers when peer_cols > 0
// (see ab200_linear_bf16_scatter). N and K must be multiples of 128.
int ab200_linear_fp8(const void* xq, long long ldxq, const void* sx_t, long long ld_sx,
                     const void* wq, long long ldw, const void* sw, long long ld_sw, void* out,
                     long long ldo, int M, int N, int K, void* workspace, size_t workspace_bytes,
                     int force_splits, const void* const* peer_ptrs, int world, int peer_cols,
                     long long peer_row_off, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 128) || (N % 128) || (ldxq % 16) || (ldw % 16) || (ldo % 8) ||
      (reinterpret_cast<uintptr_t>(xq) & 15) || (reinterpret_cast<uintptr_t>(wq) & 15))
    return -2;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -3;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             227 * 1024) != cudaSuccess)
      return -3;
    attr_set[dev] = true;
  }
  Fp8Args a;
  memset(&a, 0, sizeof(a));
  a.K = K;
  a.kblocks_total = K / kF8BlockK;
  a.status = status;
  a.sx_t = reinterpret_cast<const float*>(sx_t);
  a.ld_sx = ld_sx;
  a.sw = reinterpret_cast<const float*>(sw);
  a.ld_sw = ld_sw;
  a.out = out;
  a.ldo = ldo;
  a.splits = 1;
  if (peer_cols > 0) {
    if (world < 1 || world > 16 || (peer_cols % 128) || N != world * peer_cols) return -2;
    a.peer_cols = peer_cols;
    a.peer_row_off = peer_row_off;
    for (int i = 0; i < world; ++i)
      a.peer_out[i] = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(peer_ptrs[i]));
    force_splits = 1;
  }
  const void *pa, *pb;
  long long lda, ldb;
  const int sms = f8_sms();
  if (M <= 128) {
    a.transposed = 1;
    a.rows_a = N;
    a.rows_b = M;
    a.bn = ((M + 31) / 32) * 32;
    pa = wq;
    lda = ldw;
    pb = xq;
    ldb = ldxq;
    a.tiles_a = N / 128;
    a.tiles_b = 1;
    int splits = force_splits;
    if (splits <= 0) {
      splits = 1;
      while (a.tiles_a * splits * 2 <= sms + sms / 4 && splits < 8 &&
             a.kblocks_total / (splits * 2) >= 4)
        splits *= 2;
    }
    if (splits > 8) splits = 8;
    if (splits > a.kblocks_total) splits = a.kblocks_total;
    if (splits > 1 &&
        (workspace == nullptr || workspace_bytes < (size_t)splits * M * N * sizeof(float)))
      splits = 1;
    a.splits = splits;
  } else {
    a.transposed = 0;
    a.rows_a = M;
    a.rows_b = N;
    a.bn = (N % 256 == 0) ? 256 : 128;
    if (peer_cols > 0 && (peer_cols % a.bn)) a.bn = 128;
    pa = xq;
    lda = ldxq;
    pb = wq;
    ldb = ldw;
    a.tiles_a = (M + 127) / 128;
    a.tiles_b = N / a.bn;
  }
  a.kblocks_per_split = (a.kblocks_total + a.splits - 1) / a.splits;
  a.splits = (a.kblocks_total + a.kblocks_per_split - 1) / a.kblocks_per_split;
  const int stage_bytes = (int)kF8ABytes + a.bn * kF8BlockK;
  a.stages = (227 * 1024 - 2048) / stage_bytes;
  if (a.stages > kF8MaxStages) a.stages = kF8MaxStages;
  void* final_out = out;
  if (a.splits > 1) {
    a.out_f32 = 1;
    a.out = workspace;
    a.ldo = N;
    a.partial_stride = (long long)M * N;
  }
  CUtensorMap ta, tb;
  if (make_tmap_2d(&ta, pa, CU_TENSOR_MAP_DATA_TYPE_UINT8, (uint64_t)a.rows_a, (uint64_t)K,
                   (uint64_t)lda, 128, kF8BlockK) != 0)
    return -4;
  if (make_tmap_2d(&tb, pb, CU_TENSOR_MAP_DATA_TYPE_UINT8, (uint64_t)a.rows_b, (uint64_t)K,
                   (uint64_t)ldb, (uint32_t)a.bn, kF8BlockK) != 0)
    return -4;
  const int total = a.tiles_a * a.tiles_b * a.splits;
  const int grid = total < sms ? total : sms;
  const size_t smem = (size_t)a.stages * stage_bytes + 256 + 1024;
  gemm_fp8_kernel<<<grid, kF8Threads, smem, stream>>>(ta, tb, a);
  if (cudaGetLastError() != cudaSuccess) return -5;
  if (a.splits > 1) {
    const long long total4 = (long long)M * (N / 4);
    int blocks = (int)((total4 + 255) / 256);
    if (blocks > sms * 8) blocks = sms * 8;
    fp8_splitk_reduce_kernel<<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const float*>(workspace), a.splits, a.partial_stride, M, N,
        reinterpret_cast<__nv_bfloat16*>(final_out), ldo);
    if (cudaGetLastError() != cudaSuccess) return -5;
  }
  return 0;
}

}  // extern "C"
