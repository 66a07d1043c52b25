// bf16 linear layer  out[M,N] = x[M,K] * w[N,K]^T  (+bias)(+residual)(activation)
// for sm_100a: a persistent, warp-specialised kernel in which one thread issues
// tcgen05.mma (UMMA 128 x bn x 16, fp32 accumulators in tensor memory), one
// thread feeds a ring of 128B-swizzled shared-memory stages with TMA, and four
// epilogue warps drain the double-buffered TMEM accumulators with tcgen05.ld.
//
// Two orientations share the kernel:
//   * token-major  (M > 256): A operand = x tile (128 tokens), B = w tile (bn features)
//   * feature-major (M <= 256, decode): A operand = w tile (128 features), B = all
//     tokens (bn = M rounded up to 16); the accumulator holds out^T and the
//     epilogue stores it transposed. Every SM then streams weights even when
//     only a handful of tokens are in flight, and split-K adds parallelism when
//     N/128 alone cannot fill 148 SMs. Split-K partial sums go to an fp32
//     scratch buffer supplied by the caller and are folded by a second kernel.
//
// The same kernel runs W8A8 fp8 linears whose scales are one per token and one per output
// feature (ab200_linear_fp8_row): the operands are e4m3 bytes (a 128-byte swizzle atom is then
// 128 k-elements and one kind::f8f6f4 instruction covers 32 of them), the whole K loop
// accumulates in tensor memory with no rescaling on the way, and the epilogue multiplies each
// accumulator by scale_token * scale_feature. An instruction of either kind is accepted at
// the same interval, so the fp8 form does twice the work per unit time.
//
// The reference relies on library GEMMs for these layers (vLLM linear layers
// reached from arctic_inference/vllm/swiftkv/llama_swiftkv.py:165-202; fp8 with per-token and
// per-channel scales: arctic_inference/vllm/spec_dec/fp8.py:34-309).

#include <math.h>
#include <stdlib.h>
#include <mutex>
#include <unordered_map>

#include "api.h"
#include "common/pdl.cuh"
#include "common/peer.cuh"
#include "common/ptx.cuh"
#include "common/tensormap.h"

namespace ab200 {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;  // bf16 elements: one 128-byte swizzle atom per row
constexpr int kBlockKFp8 = 128;  // e4m3 elements in the same 128 bytes
constexpr int kBlockKBytes = 128;
constexpr int kUmmaK = 16;
constexpr int kGemmThreads = 192;
constexpr int kMaxStages = 8;
constexpr uint32_t kABytes = kBlockM * kBlockK * 2;
// Per-epilogue-warp staging tile for coalesced stores: 32 rows x 64 bf16, rows padded to 144
// bytes so that the 16-byte accesses of eight lanes fall in distinct banks both ways.
constexpr int kStoreStagePitch = 144;
constexpr int kStoreStageBytes = 32 * kStoreStagePitch;

struct GemmArgs {
  int rows_a, rows_b, K;
  int bn, stages, splits, kblocks_per_split, kblocks_total;
  int tiles_a, tiles_b;
  int transposed;  // 0: out[a_row*ldo + b_row], 1: out[b_row*ldo + a_row]
  int out_f32;     // 1: write fp32 partial sums (split-K), no bias/residual/activation
  int act;         // 0 none, 1 gelu (erf)
  int b_mn_major;  // 1: the B operand is given as [K, rows_b] (rows_b contiguous)
  int coalesce;    // 1: bf16 row-major output goes through a shared-memory transpose so that a
                   //    warp stores whole 128-byte lines (what NVLink and L2 both want)
  int a_tiled, b_tiled;  // the operand is an fp8 weight stored as [rows/16][K/128][16][128]
  int fp8;         // 1: operands are e4m3 bytes (kind::f8f6f4), 128 k-elements per stage
  int kblock_elems;  // k-elements per stage: 64 (bf16) or 128 (fp8)
  int prefetch_w;    // 1: the weight operand is written by no kernel of the stream (a parameter)
  int b_parts;       // TMA boxes per B stage (1, or more boxes of bn / b_parts rows each)
  // Scatter epilogue: every rank walks the B tiles starting this many tiles in, i.e. at its own
  // share of the columns, so that at any moment the ranks store into different destination
  // ranks. With all ranks starting at tile 0 they all store into rank 0 first, then rank 1,
  // ...: one NVLink ingress carries everything while the others idle.
  int tile_b_rot;
  // > 1: the launch is made of clusters of this many CTAs. The CTAs of a cluster share one
  // output tile and split its K range; they exchange their fp32 partial sums through each
  // other's shared memory and each finishes and stores bn / cluster_splits columns (the
  // split-K of a one-row-of-tiles GEMM with no workspace traffic and no second kernel).
  int cluster_splits;
  const float* scale_a;  // fp8: one factor per A-operand row (null = 1)
  const float* scale_b;  // fp8: one factor per B-operand row
  uint32_t tmem_cols;
  long long ldo, ldr, partial_stride;
  void* out;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  int* status;
  // Peer scatter (Ulysses sequence->head exchange fused into the epilogue): when
  // peer_cols > 0, output feature f goes to buffer peer_out[f / peer_cols], column
  // f % peer_cols, row (token + peer_row_off). The buffers are the ranks' symmetric heaps,
  // reached with plain peer stores over NVLink.
  int peer_cols;
  long long peer_row_off;
  __nv_bfloat16* peer_out[16];
  // Cross-rank ordering without a barrier kernel (common/peer.cuh): `wait` holds back the
  // first operand load until every rank's producer of the A operand has signalled (the
  // head->sequence exchange lands in this rank's heap); `sig` tells every rank when the last
  // block of this kernel has finished storing (scatter epilogue, or a partial product that the
  // peers will reduce).
  PeerWait wait;
  TailSignal sig;
};

__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
}

// Work item -> (A tile, B tile, K split). Cluster launches hold one item per CTA, the K splits
// of a tile being the consecutive CTAs of one cluster.
__device__ __forceinline__ void decode_work(const GemmArgs& p, int w, int& tile_a, int& tile_b,
                                            int& split) {
  if (p.cluster_splits > 1) {
    tile_a = 0;
    split = w % p.cluster_splits;
    tile_b = w / p.cluster_splits + p.tile_b_rot;
    if (tile_b >= p.tiles_b) tile_b -= p.tiles_b;
    return;
  }
  tile_a = w % p.tiles_a;
  const int rest = w / p.tiles_a;
  tile_b = rest % p.tiles_b;
  split = rest / p.tiles_b;
  if (p.tile_b_rot) {
    tile_b += p.tile_b_rot;
    if (tile_b >= p.tiles_b) tile_b -= p.tiles_b;
  }
}

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b, const GemmArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t b_bytes = (uint32_t)p.bn * kBlockK * 2;
  const uint32_t stage_bytes = kABytes + b_bytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t)p.stages * stage_bytes);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* store_stage = reinterpret_cast<uint8_t*>(bars) + 256;
  // the tile's per-column scales, fetched while the k-loop runs (a lone tile per CTA pays for
  // every load that waits until the accumulator is complete)
  // (one private copy per epilogue warp, so that no barrier between warps is involved)
  float* col_scale = reinterpret_cast<float*>(store_stage + 4 * kStoreStageBytes) +
                     ((threadIdx.x >> 5) & 3) * 256;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bars_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bars_base + 8u * s; };
  auto empty_bar = [&](int s) { return bars_base + 8u * (kMaxStages + s); };
  auto tfull_bar = [&](int a) { return bars_base + 8u * (2 * kMaxStages + a); };
  auto tempty_bar = [&](int a) { return bars_base + 8u * (2 * kMaxStages + 2 + a); };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // the next kernel of the stream may be placed as SMs free up; it waits for this one itself
  pdl_trigger();

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t acc_stride = p.tmem_cols / 2;

  const int total_work = p.tiles_a * p.tiles_b * p.splits;
  bool cluster_acc_ok = false;   // epilogue threads of a cluster launch: the accumulator is complete

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    // The weight operand is written by no kernel, so its first tiles are requested before
    // this kernel waits for the one before it in the stream: the stream of weights starts
    // while that kernel drains. Each of these stages has had its weight bytes announced to
    // its full barrier; the activation tile and the barrier's arrival follow after the wait.
    const bool w_is_b = !p.transposed;
    int pre = 0;
    if (lane == 0 && p.prefetch_w && blockIdx.x < total_work) {
      int tile_a0, tile_b0, split0;
      decode_work(p, blockIdx.x, tile_a0, tile_b0, split0);
      const int kb00 = split0 * p.kblocks_per_split;
      const int kb01 = min(kb00 + p.kblocks_per_split, p.kblocks_total);
      pre = min(p.stages, kb01 - kb00);
      for (int s = 0; s < pre; ++s) {
        const int kb = kb00 + s;
        const uint32_t dst = smem_base + (uint32_t)s * stage_bytes;
        if (w_is_b) {
          mbar_expect_tx(full_bar(s), b_bytes);
          const int pr = p.bn / p.b_parts;
          for (int h = 0; h < p.b_parts; ++h) {
            const uint32_t d2 = dst + kABytes + (uint32_t)(h * pr) * 128u;
            if (p.b_tiled)
              tma_load_4d(d2, &tmap_b, full_bar(s), 0, 0, kb, tile_b0 * (p.bn / 16) + h * (pr / 16));
            else
              tma_load_2d(d2, &tmap_b, full_bar(s), kb * p.kblock_elems, tile_b0 * p.bn + h * pr);
          }
        } else {
          mbar_expect_tx(full_bar(s), kABytes);
          if (p.a_tiled)
            tma_load_4d(dst, &tmap_a, full_bar(s), 0, 0, kb, tile_a0 * (kBlockM / 16));
          else
            tma_load_2d(dst, &tmap_a, full_bar(s), kb * p.kblock_elems, tile_a0 * kBlockM);
        }
      }
    }
    pdl_wait();
    bool peers_ok = true;
    if (p.wait.world > 0) {
      peers_ok = wait_peers(p.wait, p.status, kWaitLimitNs);
      fence_proxy_async_global();
      if (!peers_ok && lane == 0) *abort_flag = 1;
    }
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = peers_ok;
      if (!ok) {
        // the prefetched weight tiles still land: let their barriers complete, then leave
        for (int s = 0; s < pre; ++s) {
          mbar_arrive(full_bar(s));
          mbar_drain(full_bar(s), 0);
        }
      }
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        int tile_a, tile_b, split;
        decode_work(p, w, tile_a, tile_b, split);
        const int kb0 = split * p.kblocks_per_split;
        const int kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.status, 100 + stage, kb)) {
            ok = false;
            break;
          }
          const bool have_w = issued < pre;   // this stage's weight tile is already on its way
          const bool load_a = !(have_w && !w_is_b);
          const bool load_b = !(have_w && w_is_b);
          mbar_arrive_expect_tx(full_bar(stage),
                                have_w ? (w_is_b ? (uint32_t)kABytes : b_bytes) : stage_bytes);
          const uint32_t a_dst = smem_base + (uint32_t)stage * stage_bytes;
          if (load_a) {
            if (p.a_tiled)
              tma_load_4d(a_dst, &tmap_a, full_bar(stage), 0, 0, kb, tile_a * (kBlockM / 16));
            else
              tma_load_2d(a_dst, &tmap_a, full_bar(stage), kb * p.kblock_elems, tile_a * kBlockM);
          }
          if (!load_b) {
          } else if (!p.b_mn_major) {
            // tiled storage: 2 KB pieces (16 rows x 128 bytes) that are contiguous in memory
            const int pr = p.bn / p.b_parts;
            for (int h = 0; h < p.b_parts; ++h) {
              const uint32_t d2 = a_dst + kABytes + (uint32_t)(h * pr) * 128u;
              if (p.b_tiled)
                tma_load_4d(d2, &tmap_b, full_bar(stage), 0, 0, kb,
                            tile_b * (p.bn / 16) + h * (pr / 16));
              else
                tma_load_2d(d2, &tmap_b, full_bar(stage), kb * p.kblock_elems,
                            tile_b * p.bn + h * pr);
            }
          } else {
            // [64 k-rows][64 n] boxes, one per 64-wide atom along N
            for (int j = 0; j < p.bn / 64; ++j)
              tma_load_2d(a_dst + kABytes + (uint32_t)j * 8192u, &tmap_b, full_bar(stage),
                          tile_b * p.bn + j * 64, kb * kBlockK);
          }
          ++issued;
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Unwinding: give copies that were already issued a short time to land.
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
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      const uint32_t idesc =
          p.fp8 ? make_idesc(kBlockM, (uint32_t)p.bn, 0, 0, 0, 0)
                : make_idesc(kBlockM, (uint32_t)p.bn, 1, 1, 0, p.b_mn_major ? 1u : 0u);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        int tile_a, tile_b, split;
        decode_work(p, w, tile_a, tile_b, split);
        const int kb0 = split * p.kblocks_per_split;
        const int kb1 = min(kb0 + p.kblocks_per_split, p.kblocks_total);
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.status, 200 + acc, w)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)acc * acc_stride;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, 300 + stage, kb)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_base + (uint32_t)stage * stage_bytes;
          const uint64_t a_desc = make_desc_kmajor_sw128(a_addr);
          const uint64_t b_desc = p.b_mn_major ? make_desc_mnmajor_sw128(a_addr + kABytes, 8192u)
                                               : make_desc_kmajor_sw128(a_addr + kABytes);
          // K-major: 16 bf16 or 32 e4m3 (32 bytes) further inside the swizzle atom = +2 in the
          // encoded address; MN-major: 16 rows of 128 bytes further = +128.
          const uint64_t b_step = p.b_mn_major ? 128u : 2u;
          if (p.fp8) {
#pragma unroll
            for (int k = 0; k < kBlockKBytes / 32; ++k) {
              umma_f8_ss(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + (uint64_t)(2 * k), idesc,
                         (kb > kb0 || k > 0) ? 1u : 0u);
            }
          } else {
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
              umma_f16_ss(d_tmem, a_desc + (uint64_t)(2 * k), b_desc + b_step * (uint64_t)k, idesc,
                          (kb > kb0 || k > 0) ? 1u : 0u);
            }
          }
          tc_commit(empty_bar(stage));
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
  } else {
    // --------------------------------- epilogue --------------------------------
    pdl_wait();  // scales, bias and residual come from earlier kernels; the output may still be read by one
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const int row = quad * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool scaled = p.scale_a != nullptr && !p.out_f32;
    if (p.cluster_splits > 1) {
      // one work item per CTA; what follows the accumulator is the cluster exchange below
      if (scaled) {
        const int cw = p.bn / p.cluster_splits;
        int ta, tb, sp;
        decode_work(p, (int)blockIdx.x, ta, tb, sp);
        const long long c0 = (long long)tb * p.bn + (long long)sp * cw;
        for (int i = lane; i < cw; i += 32)
          col_scale[i] = (c0 + i < p.rows_b) ? p.scale_b[c0 + i] : 0.f;
        __syncwarp();
      }
      cluster_acc_ok = mbar_wait(tfull_bar(0), 0, abort_flag, p.status, 400, (int)blockIdx.x);
      tc_fence_after();
    } else
    for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
      int tile_a, tile_b, split;
      decode_work(p, w, tile_a, tile_b, split);
      const long long a_row = (long long)tile_a * kBlockM + row;
      const bool row_ok = a_row < p.rows_a;
      const long long b0 = (long long)tile_b * p.bn;
      const float sa = (scaled && row_ok) ? p.scale_a[a_row] : 1.f;
      if (scaled) {
        __syncwarp();   // the previous tile's reads are done
        for (int i = lane; i < p.bn; i += 32)
          col_scale[i] = (b0 + i < p.rows_b) ? p.scale_b[b0 + i] : 0.f;
        __syncwarp();
      }
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.status, 400 + acc, w)) break;
      tc_fence_after();
      const uint32_t t_addr =
          tmem_base + (uint32_t)acc * acc_stride + ((uint32_t)(quad * 32) << 16);

      if (p.coalesce) {
        // 64 output columns at a time: each thread converts its row, the warp transposes
        // through its private staging tile, and every store instruction then writes four
        // full 128-byte lines (rows) instead of 32 scattered 16-byte pieces.
        uint8_t* stg = store_stage + (size_t)quad * kStoreStageBytes;
        for (int c0 = 0; c0 < p.bn; c0 += 64) {
          uint32_t r0[32], r1[32];
          __syncwarp();
          tmem_ld_x32(t_addr + (uint32_t)c0, r0);
          tmem_ld_x32(t_addr + (uint32_t)(c0 + 32), r1);
          tmem_ld_wait();
          const long long col = b0 + c0;
          if (row_ok) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float v[8];
#pragma unroll
              for (int t = 0; t < 8; ++t)
                v[t] = __uint_as_float(j < 4 ? r0[8 * j + t] : r1[8 * (j - 4) + t]);
              const long long cj = col + 8 * j;
              if (cj + 8 <= p.rows_b && c0 + 8 * j + 8 <= p.bn) {
                if (scaled) {
                  const float4 s0 = *reinterpret_cast<const float4*>(col_scale + c0 + 8 * j);
                  const float4 s1 = *reinterpret_cast<const float4*>(col_scale + c0 + 8 * j + 4);
                  v[0] *= sa * s0.x; v[1] *= sa * s0.y; v[2] *= sa * s0.z; v[3] *= sa * s0.w;
                  v[4] *= sa * s1.x; v[5] *= sa * s1.y; v[6] *= sa * s1.z; v[7] *= sa * s1.w;
                }
                if (p.bias != nullptr) {
                  const uint4 q = *reinterpret_cast<const uint4*>(p.bias + cj);
                  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
                  for (int u = 0; u < 4; ++u) {
                    const float2 f = __bfloat1622float2(h[u]);
                    v[2 * u] += f.x;
                    v[2 * u + 1] += f.y;
                  }
                }
                if (p.act == 1) {
#pragma unroll
                  for (int t = 0; t < 8; ++t) v[t] = gelu_erf(v[t]);
                }
                if (p.residual != nullptr) {
                  const uint4 q = *reinterpret_cast<const uint4*>(p.residual + a_row * p.ldr + cj);
                  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
                  for (int u = 0; u < 4; ++u) {
                    const float2 f = __bfloat1622float2(h[u]);
                    v[2 * u] += f.x;
                    v[2 * u + 1] += f.y;
                  }
                }
              }
              uint4 q;
              q.x = pack_bf16x2(v[0], v[1]);
              q.y = pack_bf16x2(v[2], v[3]);
              q.z = pack_bf16x2(v[4], v[5]);
              q.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(stg + lane * kStoreStagePitch + 16 * j) = q;
            }
          }
          __syncwarp();
          __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(p.out) + col;
          long long row_off = 0;
          if (p.peer_cols > 0) {  // a 64-column group never straddles a destination
            base = p.peer_out[col / p.peer_cols] + col % p.peer_cols;
            row_off = p.peer_row_off;
          }
          const int ch = lane & 7;
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + (lane >> 3);
            const long long grow = (long long)tile_a * kBlockM + quad * 32 + rr;
            if (grow < p.rows_a && col + 8 * ch + 8 <= p.rows_b && c0 + 8 * ch + 8 <= p.bn) {
              const uint4 q = *reinterpret_cast<const uint4*>(stg + rr * kStoreStagePitch + 16 * ch);
              *reinterpret_cast<uint4*>(base + (grow + row_off) * p.ldo + 8 * ch) = q;
            }
          }
        }
      } else
      for (int c0 = 0; c0 < p.bn; c0 += 16) {
        uint32_t r[16];
        __syncwarp();
        tmem_ld_x16(t_addr + (uint32_t)c0, r);
        tmem_ld_wait();
        float v[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) v[t] = __uint_as_float(r[t]);
        if (!row_ok) continue;
        if (p.out_f32) {
          float* o = reinterpret_cast<float*>(p.out) + (long long)split * p.partial_stride;
          if (!p.transposed) {
            float* dst = o + a_row * p.ldo + b0 + c0;
#pragma unroll
            for (int t = 0; t < 16; t += 4) {
              if (b0 + c0 + t + 4 <= p.rows_b)
                *reinterpret_cast<float4*>(dst + t) = make_float4(v[t], v[t + 1], v[t + 2], v[t + 3]);
            }
          } else {
#pragma unroll
            for (int t = 0; t < 16; ++t) {
              const long long b_row = b0 + c0 + t;
              if (b_row < p.rows_b) o[b_row * p.ldo + a_row] = v[t];
            }
          }
          continue;
        }
        if (scaled) {
#pragma unroll
          for (int t = 0; t < 16; ++t) v[t] *= sa * col_scale[c0 + t];
        }
        if (!p.transposed) {
          const long long col = b0 + c0;
          if (p.bias != nullptr) {
#pragma unroll
            for (int t = 0; t < 16; ++t)
              if (col + t < p.rows_b) v[t] += __bfloat162float(p.bias[col + t]);
          }
          if (p.act == 1) {
#pragma unroll
            for (int t = 0; t < 16; ++t) v[t] = gelu_erf(v[t]);
          }
          if (p.residual != nullptr) {
            const __nv_bfloat16* rs = p.residual + a_row * p.ldr + col;
#pragma unroll
            for (int t = 0; t < 16; t += 8) {
              if (col + t + 8 <= p.rows_b) {
                const uint4 q = *reinterpret_cast<const uint4*>(rs + t);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  const float2 f = __bfloat1622float2(h[u]);
                  v[t + 2 * u] += f.x;
                  v[t + 2 * u + 1] += f.y;
                }
              }
            }
          }
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + a_row * p.ldo + col;
          if (p.peer_cols > 0)  // a 16-column chunk never straddles a destination (peer_cols % 16 == 0)
            dst = p.peer_out[col / p.peer_cols] + (a_row + p.peer_row_off) * p.ldo +
                  col % p.peer_cols;
#pragma unroll
          for (int t = 0; t < 16; t += 8) {
            if (col + t + 8 <= p.rows_b) {
              uint4 q;
              q.x = pack_bf16x2(v[t], v[t + 1]);
              q.y = pack_bf16x2(v[t + 2], v[t + 3]);
              q.z = pack_bf16x2(v[t + 4], v[t + 5]);
              q.w = pack_bf16x2(v[t + 6], v[t + 7]);
              *reinterpret_cast<uint4*>(dst + t) = q;
            }
          }
        } else {
          // accumulator holds out^T: this thread owns output feature a_row
          const float bias = (p.bias != nullptr) ? __bfloat162float(p.bias[a_row]) : 0.f;
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out);
          long long o_col = a_row, o_row_off = 0;
          if (p.peer_cols > 0) {
            o = p.peer_out[a_row / p.peer_cols];
            o_col = a_row % p.peer_cols;
            o_row_off = p.peer_row_off;
          }
#pragma unroll
          for (int t = 0; t < 16; ++t) {
            const long long b_row = b0 + c0 + t;
            if (b_row < p.rows_b) {
              float x = v[t] + bias;
              if (p.act == 1) x = gelu_erf(x);
              if (p.residual != nullptr) x += __bfloat162float(p.residual[b_row * p.ldr + a_row]);
              o[(b_row + o_row_off) * p.ldo + o_col] = __float2bfloat16(x);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;

    }
  }

  if (p.cluster_splits > 1) {
    // ---- split-K inside a cluster: partial sums cross through shared memory ----
    // CTA r of the cluster owns columns [r * cw, (r + 1) * cw) of the tile. Every CTA writes,
    // for each owner, its fp32 partial sums of the owner's columns into the owner's shared
    // memory (the pipeline stages, idle by now), slot [source CTA][row][cw + 4 pad]; the
    // owner adds the slots in source order, so the result does not depend on timing.
    const int ns = p.cluster_splits;
    const int cw = p.bn / ns;
    const int pitch = cw + 4;   // words; 16 B of padding keeps 16-byte row accesses of a warp
                                // on distinct banks
    const uint32_t my = cluster_ctarank();
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    // first barrier: every CTA of the cluster has consumed its last pipeline stage (its
    // epilogue warps arrive only after their accumulator is complete)
    cluster_sync();
    if (warp >= 2 && cluster_acc_ok) {
      const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16);
      for (int c0 = 0; c0 < p.bn; c0 += 16) {
        uint32_t r[16];
        __syncwarp();
        tmem_ld_x16(t_addr + (uint32_t)c0, r);
        tmem_ld_wait();
        const uint32_t owner = (uint32_t)(c0 / cw);
        const uint32_t local =
            smem_base + (uint32_t)(((int)my * kBlockM + row) * pitch + (c0 % cw)) * 4u;
        const uint32_t remote = map_to_cta(local, owner);
#pragma unroll
        for (int t = 0; t < 16; t += 4)
          st_cluster_v4(remote + 4u * t, r[t], r[t + 1], r[t + 2], r[t + 3]);
      }
    }
    // second barrier: all partial sums have landed (release / acquire at cluster scope)
    cluster_sync();
    if (warp >= 2 && cluster_acc_ok && !*abort_flag) {
      int tile_a, tile_b, split;
      decode_work(p, (int)blockIdx.x, tile_a, tile_b, split);
      const long long a_row = row;
      const bool row_ok = a_row < p.rows_a;
      const long long col0 = (long long)tile_b * p.bn + (long long)my * cw;
      const float sa = (p.scale_a != nullptr && row_ok) ? p.scale_a[a_row] : 1.f;
      const float* slots = reinterpret_cast<const float*>(smem);
      for (int j = 0; j < cw; j += 8) {
        float v[8];
#pragma unroll
        for (int t = 0; t < 8; ++t) v[t] = 0.f;
        for (int src = 0; src < ns; ++src) {
          const float* q = slots + ((size_t)src * kBlockM + row) * pitch + j;
          const float4 x0 = *reinterpret_cast<const float4*>(q);
          const float4 x1 = *reinterpret_cast<const float4*>(q + 4);
          v[0] += x0.x; v[1] += x0.y; v[2] += x0.z; v[3] += x0.w;
          v[4] += x1.x; v[5] += x1.y; v[6] += x1.z; v[7] += x1.w;
        }
        const long long col = col0 + j;
        if (!row_ok || col + 8 > p.rows_b) continue;
        if (p.scale_a != nullptr) {
          const float4 s0 = *reinterpret_cast<const float4*>(col_scale + j);
          const float4 s1 = *reinterpret_cast<const float4*>(col_scale + j + 4);
          v[0] *= sa * s0.x; v[1] *= sa * s0.y; v[2] *= sa * s0.z; v[3] *= sa * s0.w;
          v[4] *= sa * s1.x; v[5] *= sa * s1.y; v[6] *= sa * s1.z; v[7] *= sa * s1.w;
        }
        if (p.bias != nullptr) {
          const uint4 q = *reinterpret_cast<const uint4*>(p.bias + col);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float2 f = __bfloat1622float2(h[u]);
            v[2 * u] += f.x;
            v[2 * u + 1] += f.y;
          }
        }
        if (p.act == 1) {
#pragma unroll
          for (int t = 0; t < 8; ++t) v[t] = gelu_erf(v[t]);
        }
        if (p.residual != nullptr) {
          const uint4 q = *reinterpret_cast<const uint4*>(p.residual + a_row * p.ldr + col);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float2 f = __bfloat1622float2(h[u]);
            v[2 * u] += f.x;
            v[2 * u + 1] += f.y;
          }
        }
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + a_row * p.ldo + col;
        if (p.peer_cols > 0)  // eight columns never straddle a destination (peer_cols % 8 == 0)
          dst = p.peer_out[col / p.peer_cols] + (a_row + p.peer_row_off) * p.ldo +
                col % p.peer_cols;
        uint4 q;
        q.x = pack_bf16x2(v[0], v[1]);
        q.y = pack_bf16x2(v[2], v[3]);
        q.z = pack_bf16x2(v[4], v[5]);
        q.w = pack_bf16x2(v[6], v[7]);
        *reinterpret_cast<uint4*>(dst) = q;
      }
    }
  }

  tail_signal(p.sig, gridDim.x);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

// out[m,n] = sum_s partial[s][m,n] (+bias[n]) -> activation -> (+residual[m,n])
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int splits,
                                     long long partial_stride, int M, int N,
                                     __nv_bfloat16* __restrict__ out, long long ldo,
                                     const __nv_bfloat16* __restrict__ bias,
                                     const __nv_bfloat16* __restrict__ residual, long long ldr,
                                     int act, const float* __restrict__ scale_m,
                                     const float* __restrict__ scale_n, const TailSignal sig) {
  pdl_wait();
  pdl_trigger();
  const long long n4 = N / 4;
  const long long total = (long long)M * n4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long m = i / n4;
    const long long n = (i % n4) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float4 v =
          *reinterpret_cast<const float4*>(partial + s * partial_stride + m * (long long)N + n);
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    float v[4] = {acc.x, acc.y, acc.z, acc.w};
    if (scale_m != nullptr) {
      const float sm = scale_m[m];
#pragma unroll
      for (int t = 0; t < 4; ++t) v[t] *= sm * scale_n[n + t];
    }
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      if (bias != nullptr) v[t] += __bfloat162float(bias[n + t]);
      if (act == 1) v[t] = gelu_erf(v[t]);
      if (residual != nullptr) v[t] += __bfloat162float(residual[m * ldr + n + t]);
    }
    uint2 q;
    q.x = pack_bf16x2(v[0], v[1]);
    q.y = pack_bf16x2(v[2], v[3]);
    *reinterpret_cast<uint2*>(out + m * ldo + n) = q;
  }
  tail_signal(sig, gridDim.x);
}

// ------------------------------- host side ---------------------------------
struct TmapKey {
  const void* ptr;
  uint64_t rows, cols, ld;
  uint32_t box_rows;  // bit 31 set: e4m3 bytes instead of bf16
  uint64_t tile_stride_n = 0;  // tiled fp8 weights: bytes between 16-row tiles (0: row-major)
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld &&
           box_rows == o.box_rows && tile_stride_n == o.tile_stride_n;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= k.rows * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.cols * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= k.ld * 0x165667B19E3779F9ull + (h << 6) + (h >> 2);
    h ^= k.box_rows * 0x27D4EB2F165667C5ull + (h << 6) + (h >> 2);
    h ^= k.tile_stride_n * 0x9FB21C651E98DF25ull + (h << 6) + (h >> 2);
    return h;
  }
};

static int get_tmap(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                    uint32_t box_rows, bool fp8, uint64_t tile_stride_n = 0);
static int get_tmap_bf16(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols,
                         uint64_t ld, uint32_t box_rows) {
  return get_tmap(out, ptr, rows, cols, ld, box_rows, false);
}
// tile_stride_n > 0: the matrix is an fp8 weight stored as [rows/16][K/128][16][128] bytes;
// `ld` is then the byte distance between consecutive k-tiles of one 16-row tile and
// tile_stride_n the distance between 16-row tiles (views of a larger tiled matrix keep their
// parent's strides). A box of box_rows rows is box_rows/16 contiguous 2 KB pieces.
static int get_tmap(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                    uint32_t box_rows, bool fp8, uint64_t tile_stride_n) {
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  TmapKey key{ptr, rows, cols, ld, box_rows | (fp8 ? 0x80000000u : 0u), tile_stride_n};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  CUtensorMap m;
  int rc;
  if (tile_stride_n > 0) {
    const uint64_t dims[4] = {128, 16, cols / 128, (rows + 15) / 16};
    const uint64_t strides[3] = {128, ld, tile_stride_n};
    const uint32_t box[4] = {128, 16, 1, box_rows / 16};
    rc = make_tmap_nd(&m, ptr, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, dims, strides, box);
  } else
  rc = fp8 ? make_tmap_2d(&m, ptr, CU_TENSOR_MAP_DATA_TYPE_UINT8, rows, cols, ld, box_rows,
                              kBlockKFp8)
               : make_tmap_2d(&m, ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rows, cols, ld * 2,
                              box_rows, kBlockK);
  if (rc != 0) return rc;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return 0;
}

static int g_num_sms = 0;
static int num_sms() {
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (g_num_sms <= 0) g_num_sms = 148;
  }
  return g_num_sms;
}

static int pick_stages(int bn) {
  const int stage_bytes = (int)kABytes + bn * kBlockK * 2;
  int s = (227 * 1024 - 6144 - 4 * kStoreStageBytes) / stage_bytes;
  if (s > kMaxStages) s = kMaxStages;
  return s;
}

// How many clusters of `cs` CTAs (one CTA per SM: the kernel takes an SM's shared memory) the
// device can hold at once; 0 when such a cluster cannot be placed.
static int cluster_capacity(int cs, size_t smem) {
  static int cache[64][4];   // [device][log2 cs]: 0 unknown, -1 none, else capacity
  int dev = 0;
  cudaGetDevice(&dev);
  int lg = cs == 2 ? 1 : cs == 4 ? 2 : cs == 8 ? 3 : -1;
  if (dev < 0 || dev >= 64 || lg < 0) return 0;
  if (cache[dev][lg] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)cs * 16);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cs;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_bf16_kernel, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    cache[dev][lg] = n > 0 ? n : -1;
  }
  return cache[dev][lg] > 0 ? cache[dev][lg] : 0;
}

// Rough time (us) of a one-row-of-tiles GEMM plan: every wave pays its k-loop (four MMA
// instructions per k-block at the measured issue interval, ~0.45 us per k-block with its
// stage turnaround) plus a fixed ramp; split-K through the workspace pays the fp32 partials'
// round trip and a second kernel, split-K inside a cluster a shared-memory exchange.
static double plan_cost_us(int tiles, int splits, int kblocks, int capacity, bool cluster, int M,
                           int N) {
  const int ctas = tiles * splits;
  const int waves = (ctas + capacity - 1) / capacity;
  const int per = (kblocks + splits - 1) / splits;
  double t = waves * (per * 0.45 + 2.0);
  if (splits > 1)
    t += cluster ? 1.0 : 3.0 + 2.0 * splits * (double)M * N * 4.0 / 3.0e6;
  return t;
}

static uint32_t pow2_at_least(uint32_t v) {
  uint32_t p = 32;
  while (p < v) p <<= 1;
  return p;
}

}  // namespace ab200

using namespace ab200;

extern "C" {

// Number of fp32 scratch bytes ab200_linear_bf16 may need for (M, N, K).
size_t ab200_linear_bf16_workspace_bytes(int M, int N, int K) {
  if (M > 256) return 0;
  return (size_t)(M <= 128 ? 16 : 8) * (size_t)M * (size_t)N * sizeof(float);
}

// One tcgen05.mma (cta_group::1) is accepted every ~186 SM cycles whatever its shape
// (measured on B200 for M = 64/128, N = 16..256, bf16 and fp8), so a k-loop is bound by its
// instruction count unless every instruction carries enough work. With few tokens the
// weights therefore go on the N side, 256 features per instruction, and the tokens on the
// (padded) M side; split-K then spreads the instructions over all SMs.
constexpr double kMmaIssueCycles = 186.0;

// Split-K factor for a one-row-of-tiles (M <= 128) token-major GEMM: the smallest estimate of
// max(instruction-issue time, HBM time incl. fp32 partials) plus a reduce-launch penalty.
static int pick_token_major_splits(int tiles_b, int kblocks, int M, int N, int K, int sms,
                                   size_t workspace_bytes, int elem_bytes) {
  int best = 1;
  double best_t = 1e30;
  for (int s = 1; s <= 16; s *= 2) {
    if (s > 1 && (kblocks / s < 4 || (size_t)s * M * N * sizeof(float) > workspace_bytes)) break;
    const int per_split = (kblocks + s - 1) / s;
    const int waves = (tiles_b * s + sms - 1) / sms;
    const double issue_us = waves * per_split * (kBlockK / kUmmaK) * kMmaIssueCycles / 1.9e3;
    const double bytes = (double)elem_bytes * N * K + (s > 1 ? 2.0 * s * M * (double)N * 4.0 : 0.0);
    const double hbm_us = bytes / 6.5e6;
    const double t = (issue_us > hbm_us ? issue_us : hbm_us) + (s > 1 ? 4.0 : 0.0);
    if (t < best_t - 0.25) {
      best_t = t;
      best = s;
    }
  }
  return best;
}

static int launch_linear(const void* x, long long ldx, const void* w, long long ldw, void* out,
                         long long ldo, int M, int N, int K, const void* bias,
                         const void* residual, long long ldr, int act, void* workspace,
                         size_t workspace_bytes, int force_splits, int* status,
                         cudaStream_t stream, const void* const* peer_ptrs, int world,
                         int peer_cols, long long peer_row_off, const float* scale_x = nullptr,
                         const float* scale_w = nullptr, const Ab200PeerSync* sync = nullptr,
                         long long w_tile_stride_n = 0, long long w_tile_stride_k = 0,
                         int w_static = 0) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const bool fp8 = scale_x != nullptr;  // e4m3 operands with per-token / per-feature scales
  const int opa = fp8 ? 16 : 8;         // operand rows must start on 16-byte boundaries
  if ((K % opa) || (N % 8) || (ldx % opa) || (ldw % opa) || (ldo % 8) ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return -2;
  if (fp8 && (scale_w == nullptr || (reinterpret_cast<uintptr_t>(scale_w) & 15))) return -2;
  const bool w_tiled = w_tile_stride_n > 0;
  if (w_tiled && (!fp8 || (K % 128) || (N % 16) || (w_tile_stride_n % 16) ||
                  (w_tile_stride_k % 16) || w_tile_stride_k < 2048))
    return -2;
  if (residual != nullptr && ((ldr % 8) || (reinterpret_cast<uintptr_t>(residual) & 15))) return -2;

  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -3;
  if (!attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return -3;
    attr_set[dev] = true;
  }

  GemmArgs a;
  memset(&a, 0, sizeof(a));
  if (peer_cols > 0) {
    if (world < 1 || world > 16 || (peer_cols % 16) || N != world * peer_cols) return -2;
    a.peer_cols = peer_cols;
    a.peer_row_off = peer_row_off;
    for (int i = 0; i < world; ++i)
      a.peer_out[i] = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(peer_ptrs[i]));
    force_splits = 1;  // partial sums would need the scatter in the reduce kernel as well
  }
  a.K = K;
  a.fp8 = fp8 ? 1 : 0;
  a.kblock_elems = fp8 ? kBlockKFp8 : kBlockK;
  a.kblocks_total = (K + a.kblock_elems - 1) / a.kblock_elems;
  a.status = status;
  a.act = act;
  a.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  a.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  a.ldr = ldr;
  a.ldo = ldo;
  a.out = out;
  a.splits = 1;

  const void* pa;
  const void* pb;
  long long lda, ldb;
  const int sms = num_sms();
  if (M > kBlockM && M <= 256) {
    // feature-major: weights are the 128-row operand, all tokens form the N side
    a.transposed = 1;
    a.rows_a = N;
    a.rows_b = M;
    a.bn = ((M + 15) / 16) * 16;
    pa = w;
    lda = ldw;
    pb = x;
    ldb = ldx;
    a.tiles_a = (N + kBlockM - 1) / kBlockM;
    a.tiles_b = 1;
    a.scale_a = scale_w;
    a.scale_b = scale_x;
    int splits = force_splits;
    if (splits <= 0) {
      splits = 1;
      while (a.tiles_a * splits * 2 <= sms + sms / 4 && splits < 8 &&
             a.kblocks_total / (splits * 2) >= 8)
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
    pa = x;
    lda = ldx;
    pb = w;
    ldb = ldw;
    a.tiles_a = (M + kBlockM - 1) / kBlockM;
    a.scale_a = scale_x;
    a.scale_b = scale_w;
    const int tiles256 = a.tiles_a * ((N + 255) / 256);
    a.bn = ((tiles256 >= sms || a.tiles_a == 1) && N >= 256) ? 256 : 128;
    if (N < 128) a.bn = ((N + 15) / 16) * 16;
    if (a.tiles_a == 1 && peer_cols == 0 && a.bn == 256) {
      // One row of tiles that streams the whole weight matrix (decode): when 256-wide tiles
      // leave a good part of the SMs without one (gate/up of an 8B model: 112 tiles on 148
      // SMs), narrow them to the widest size that still fits one wave. A narrower tile is also
      // a smaller pipeline stage, i.e. one more stage of loads in flight per SM.
      const int t256 = (N + 255) / 256;
      if (t256 * 4 > sms * 2 && t256 * 8 < sms * 7) {
        int bn = 256;
        while (bn > 128 && (N + (bn - 16) - 1) / (bn - 16) <= sms) bn -= 16;
        a.bn = bn;
      }
    }
    if (a.tiles_a == 1 && peer_cols > 0 && N >= 256) {
      // One row of tiles and no split-K (the scatter epilogue writes final values): a CTA
      // streams its weight tile at a fraction of an SM's share of HBM bandwidth, so narrow the
      // tiles until most SMs hold one.
      while (a.bn > 64 && (N + a.bn - 1) / a.bn < (sms * 3) / 5) a.bn /= 2;
    }
    a.tiles_b = (N + a.bn - 1) / a.bn;
    if (a.tiles_a == 1) {
      int splits = force_splits;
      if (splits <= 0)
        splits = (N % 4 == 0 && workspace != nullptr)
                     ? pick_token_major_splits(a.tiles_b, a.kblocks_total, M, N, K, sms,
                                               workspace_bytes, fp8 ? 1 : 2)
                     : 1;
      if (splits > 16) splits = 16;
      if (splits > a.kblocks_total) splits = a.kblocks_total;
      if (splits > 1 && (workspace == nullptr || (N % 4) ||
                         workspace_bytes < (size_t)splits * M * N * sizeof(float)))
        splits = 1;
      a.splits = splits;
    }
  }
  // One row of tiles (at most 128 tokens): consider splitting K inside thread-block clusters
  // instead of through the workspace. The scatter epilogue qualifies too: the CTA that
  // finishes a column range stores it to the rank that owns it.
  static const bool cluster_off = [] {
    const char* e = getenv("AB200_GEMM_CLUSTER");
    return e != nullptr && e[0] == '0';
  }();
  if (!a.transposed && a.tiles_a == 1 && !cluster_off && (force_splits == 0 || peer_cols > 0) &&
      N % 8 == 0 && ldo % 8 == 0 && (peer_cols == 0 || peer_cols % 8 == 0) &&
      (reinterpret_cast<uintptr_t>(bias) % 16) == 0 && (residual == nullptr || ldr % 8 == 0)) {
    double best = plan_cost_us(a.tiles_b, a.splits, a.kblocks_total, sms, false, M, N);
    int best_bn = 0, best_s = 0, best_ctas = 0;
    const size_t smem_full = 227 * 1024 - 1024;
    for (int bn = 256; bn >= 64; bn -= 64) {
      if (bn > ((N + 63) / 64) * 64) continue;
      const int tiles = (N + bn - 1) / bn;
      for (int cs = 2; cs <= 8; cs *= 2) {
        // (each CTA keeps at least 8 k-blocks: with fewer, the cluster's placement and its two
        // barriers cost more than the shorter loop saves; measured on the 4096 x 4096 o_proj)
        if (bn % (16 * cs) != 0 || a.kblocks_total < 8 * cs) continue;
        const int per = (a.kblocks_total + cs - 1) / cs;
        if ((a.kblocks_total + per - 1) / per != cs) continue;   // every CTA of a cluster has work
        const int cap = cluster_capacity(cs, smem_full) * cs;
        if (cap <= 0 || tiles * cs > 4 * cap) continue;
        const double c = plan_cost_us(tiles, cs, a.kblocks_total, cap, true, M, N);
        if (c < best - 0.25 || (c < best + 0.25 && best_s > 0 && tiles * cs > best_ctas)) {
          best = c < best ? c : best;
          best_bn = bn;
          best_s = cs;
          best_ctas = tiles * cs;
        }
      }
    }
    if (best_s > 0) {
      a.bn = best_bn;
      a.tiles_b = (N + a.bn - 1) / a.bn;
      a.splits = best_s;
      a.cluster_splits = best_s;
    }
  }
  a.kblocks_per_split = (a.kblocks_total + a.splits - 1) / a.splits;
  a.splits = (a.kblocks_total + a.kblocks_per_split - 1) / a.kblocks_per_split;
  a.stages = pick_stages(a.bn);
  a.tmem_cols = pow2_at_least(2u * (uint32_t)a.bn);
  if (a.cluster_splits > 1 &&
      (size_t)a.stages * (kABytes + (size_t)a.bn * kBlockK * 2) <
          (size_t)kBlockM * (a.bn + 4 * a.cluster_splits) * sizeof(float)) {
    return -2;   // cannot happen for the tile sizes above: the exchange slots fit the pipeline
  }

  a.coalesce = !a.transposed && a.splits == 1 && a.bn % 8 == 0 &&
               N % 8 == 0 && ldo % 8 == 0 &&
               (peer_cols == 0 || (peer_cols % 64 == 0 && a.bn % 64 == 0)) &&
               (reinterpret_cast<uintptr_t>(bias) % 16) == 0 &&
               (residual == nullptr || ldr % 8 == 0);

  TailSignal sig;
  memset(&sig, 0, sizeof(sig));
  if (sync != nullptr) {
    if (sync->wait_world < 0 || sync->wait_world > kMaxPeers || sync->sig_world < 0 ||
        sync->sig_world > kMaxPeers)
      return -2;
    a.wait.flags = reinterpret_cast<const unsigned int*>(sync->wait_flags);
    a.wait.epoch_ctr = reinterpret_cast<const unsigned int*>(sync->wait_epoch_ctr);
    a.wait.world = sync->wait_world;
    if (sync->sig_world > 0) {
      for (int i = 0; i < sync->sig_world; ++i)
        sig.flags[i] = reinterpret_cast<unsigned int*>(const_cast<void*>(sync->sig_flag_ptrs[i]));
      sig.done_ctr = reinterpret_cast<unsigned int*>(sync->sig_done_ctr);
      sig.epoch_ctr = reinterpret_cast<unsigned int*>(sync->sig_epoch_ctr);
      sig.my_rank = sync->sig_rank;
      sig.world = sync->sig_world;
    }
  }
  if (peer_cols > 0 && sig.world > 1)
    a.tile_b_rot = (int)(((long long)sig.my_rank * a.tiles_b) / sig.world);
  void* final_out = out;
  const bool ws_split = a.splits > 1 && a.cluster_splits <= 1;
  if (!ws_split) a.sig = sig;   // with split-K through the workspace the reduce kernel writes the output
  if (ws_split) {
    a.out_f32 = 1;
    a.out = workspace;
    a.ldo = N;  // partials are stored as [split][M][N] regardless of orientation
    a.partial_stride = (long long)M * N;
  }

  CUtensorMap ta, tb;
  a.a_tiled = (w_tiled && a.transposed) ? 1 : 0;
  a.b_tiled = (w_tiled && !a.transposed) ? 1 : 0;
  a.prefetch_w = w_static ? 1 : 0;
  // One row of tiles over a row-major weight: two half-height boxes per stage instead of one
  // (the same bytes in flight as twice as many TMA operations: 35.6 -> 33.8 us on the 128-token
  // gate/up projection; thirteen 16-row boxes, in contrast, took 54 us).
  a.b_parts = (a.tiles_a == 1 && !a.transposed && !a.b_tiled && a.bn % 16 == 0) ? 2 : 1;
  if (get_tmap(&ta, pa, (uint64_t)a.rows_a, (uint64_t)K,
               a.a_tiled ? (uint64_t)w_tile_stride_k : (uint64_t)lda, kBlockM, fp8,
               a.a_tiled ? (uint64_t)w_tile_stride_n : 0) != 0)
    return -4;
  if (get_tmap(&tb, pb, (uint64_t)a.rows_b, (uint64_t)K,
               a.b_tiled ? (uint64_t)w_tile_stride_k : (uint64_t)ldb,
               (uint32_t)(a.bn / a.b_parts), fp8,
               a.b_tiled ? (uint64_t)w_tile_stride_n : 0) != 0)
    return -4;

  const int total = a.tiles_a * a.tiles_b * a.splits;
  const int grid = (a.cluster_splits > 1 || total < sms) ? total : sms;
  const size_t smem =
      (size_t)a.stages * (kABytes + (size_t)a.bn * kBlockK * 2) + 256 + 4 * kStoreStageBytes + 4096 + 1024;
  if (launch_pdl_cluster(gemm_bf16_kernel, dim3(grid), dim3(kGemmThreads), smem, stream,
                         a.cluster_splits > 1 ? (unsigned)a.cluster_splits : 1u, ta, tb,
                         a) != cudaSuccess)
    return -5;

  if (ws_split) {
    const long long total4 = (long long)M * (N / 4);
    int blocks = (int)((total4 + 255) / 256);
    if (blocks > sms * 8) blocks = sms * 8;
    if (launch_pdl(splitk_reduce_kernel, dim3(blocks), dim3(256), 0, stream,
                   reinterpret_cast<const float*>(workspace), a.splits, a.partial_stride, M, N,
                   reinterpret_cast<__nv_bfloat16*>(final_out), ldo,
                   reinterpret_cast<const __nv_bfloat16*>(bias),
                   reinterpret_cast<const __nv_bfloat16*>(residual), ldr, act, scale_x, scale_w,
                   sig) != cudaSuccess)
      return -5;
  }
  return 0;
}


// force_splits: 0 = heuristic, >0 = use exactly this split-K factor (feature-major only).
int ab200_linear_bf16(const void* x, long long ldx, const void* w, long long ldw, void* out,
                      long long ldo, int M, int N, int K, const void* bias, const void* residual,
                      long long ldr, int act, void* workspace, size_t workspace_bytes,
                      int force_splits, int* status, cudaStream_t stream) {
  return launch_linear(x, ldx, w, ldw, out, ldo, M, N, K, bias, residual, ldr, act, workspace,
                       workspace_bytes, force_splits, status, stream, nullptr, 0, 0, 0);
}

// Linear layer whose output columns are scattered to `world` peer buffers: feature f of
// token m lands in peer_ptrs[f / peer_cols] at row (m + peer_row_off), column f % peer_cols
// (row stride ldo). N must equal world * peer_cols. The caller synchronises the ranks
// (ab200_barrier) before the destination buffers are read.
int ab200_linear_bf16_scatter(const void* x, long long ldx, const void* w, long long ldw,
                              const void* const* peer_ptrs, int world, int peer_cols,
                              long long peer_row_off, long long ldo, int M, int N, int K,
                              int* status, cudaStream_t stream) {
  if (peer_cols <= 0 || world <= 0) return -2;
  return launch_linear(x, ldx, w, ldw, const_cast<void*>(peer_ptrs[0]), ldo, M, N, K, nullptr,
                       nullptr, 0, 0, nullptr, 0, 1, status, stream, peer_ptrs, world, peer_cols,
                       peer_row_off);
}

// W8A8 fp8 linear with one scale per token and one per output feature:
//   out[m,n] = sx[m] * sw[n] * sum_k xq[m,k] * wq[n,k]   (+bias)(activation)(+residual)
// xq [M,K] and wq [N,K] are e4m3 bytes (row strides in elements, multiples of 16), sx fp32 [M],
// sw fp32 [N] (16-byte aligned). With peer_ptrs the output columns are scattered to the ranks'
// buffers as in ab200_linear_bf16_scatter (pass world = 0 for a plain output).
int ab200_linear_fp8_row(const void* xq, long long ldx, const void* sx, const void* wq,
                         long long ldw, const void* sw, void* out, long long ldo, int M, int N,
                         int K, const void* bias, const void* residual, long long ldr, int act,
                         void* workspace, size_t workspace_bytes, int force_splits,
                         const void* const* peer_ptrs, int world, int peer_cols,
                         long long peer_row_off, int* status, cudaStream_t stream) {
  if (sx == nullptr || sw == nullptr) return -2;
  if (world > 0 && peer_cols > 0) {
    return launch_linear(xq, ldx, wq, ldw, const_cast<void*>(peer_ptrs[0]), ldo, M, N, K, nullptr,
                         nullptr, 0, 0, nullptr, 0, 1, status, stream, peer_ptrs, world, peer_cols,
                         peer_row_off, reinterpret_cast<const float*>(sx),
                         reinterpret_cast<const float*>(sw));
  }
  return launch_linear(xq, ldx, wq, ldw, out, ldo, M, N, K, bias, residual, ldr, act, workspace,
                       workspace_bytes, force_splits, status, stream, nullptr, 0, 0, 0,
                       reinterpret_cast<const float*>(sx), reinterpret_cast<const float*>(sw));
}

// One entry point for every form of the linear layer, described by a struct: bf16 operands
// (sx == null) or e4m3 operands with per-token / per-feature scales, plain or peer-scattered
// output, and optional cross-rank ordering (wait for the producers of x, signal completion).
int ab200_linear_desc(const Ab200LinearDesc* d, cudaStream_t stream) {
  if (d == nullptr) return -2;
  const bool scatter = d->world > 0 && d->peer_cols > 0;
  if (scatter && d->peer_ptrs == nullptr) return -2;
  if ((d->sx == nullptr) != (d->sw == nullptr)) return -2;
  return launch_linear(d->x, d->ldx, d->w, d->ldw,
                       scatter ? const_cast<void*>(d->peer_ptrs[0]) : d->out, d->ldo, d->M, d->N,
                       d->K, scatter ? nullptr : d->bias, scatter ? nullptr : d->residual,
                       scatter ? 0 : d->ldr, scatter ? 0 : d->act, scatter ? nullptr : d->workspace,
                       scatter ? 0 : d->workspace_bytes, scatter ? 1 : d->force_splits, d->status,
                       stream, scatter ? d->peer_ptrs : nullptr, scatter ? d->world : 0,
                       scatter ? d->peer_cols : 0, scatter ? d->peer_row_off : 0,
                       reinterpret_cast<const float*>(d->sx), reinterpret_cast<const float*>(d->sw),
                       &d->sync, d->w_tile_stride_n, d->w_tile_stride_k, d->w_static);
}

// out[M,N] = x[M,K] * wt[K,N] with wt row-major (N contiguous): exercises the
// MN-major shared-memory descriptor for the B operand. N must be a multiple of 64.
int ab200_gemm_bf16_nn(const void* x, long long ldx, const void* wt, long long ldw, void* out,
                       long long ldo, int M, int N, int K, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 8) || (N % 64) || (ldx % 8) || (ldw % 8) || (ldo % 8)) return -2;
  if (cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           227 * 1024) != cudaSuccess)
    return -3;
  GemmArgs a;
  memset(&a, 0, sizeof(a));
  a.K = K;
  a.kblock_elems = kBlockK;
  a.kblocks_total = (K + kBlockK - 1) / kBlockK;
  a.kblocks_per_split = a.kblocks_total;
  a.splits = 1;
  a.status = status;
  a.ldo = ldo;
  a.out = out;
  a.rows_a = M;
  a.rows_b = N;
  a.b_mn_major = 1;
  a.b_parts = 1;
  a.bn = (N % 128 == 0) ? 128 : 64;
  a.tiles_a = (M + kBlockM - 1) / kBlockM;
  a.tiles_b = N / a.bn;
  a.stages = pick_stages(a.bn);
  a.tmem_cols = pow2_at_least(2u * (uint32_t)a.bn);
  CUtensorMap ta, tb;
  if (get_tmap_bf16(&ta, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx, kBlockM) != 0) return -4;
  if (make_tmap_2d(&tb, wt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (uint64_t)K, (uint64_t)N,
                   (uint64_t)ldw * 2, 64, 64) != 0)
    return -4;
  const int total = a.tiles_a * a.tiles_b;
  const int sms = num_sms();
  const int grid = total < sms ? total : sms;
  const size_t smem =
      (size_t)a.stages * (kABytes + (size_t)a.bn * kBlockK * 2) + 256 + 4 * kStoreStageBytes + 4096 + 1024;
  gemm_bf16_kernel<<<grid, kGemmThreads, smem, stream>>>(ta, tb, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // extern "C"
