// Flash attention for sm_100a on tensor memory: one kernel serves chunked
// prefill, decode (with split-KV) and the bidirectional encoder.
//
// A CTA owns 128 "rows": 128/G consecutive query tokens times the G query heads
// that share one KV head (GQA packing), so K and V are fetched once per KV head.
// Per 128-key tile:  S = Q K^T  is a tcgen05.mma into TMEM (K-major operands
// straight from TMA, 128B swizzle); four softmax warps read their own row of S
// with tcgen05.ld, keep the running max/sum, write P (bf16) into swizzled shared
// memory; P V is a second tcgen05.mma whose B operand is the V tile in its
// natural [key][d] layout (an MN-major descriptor), so nothing is transposed.
// S is double-buffered in TMEM: QK^T of tile j+1 runs on the tensor core while the
// softmax warps work on tile j. With 128-key tiles P is double-buffered in shared memory as
// well, so the softmax of tile j+1 does not wait for P(j) V(j) to finish unless it has to
// rescale O: the tensor core then goes from one product straight into the next.
// The output accumulator lives in TMEM as well: P V
// accumulates in place, and a warp rescales its rows of O (tcgen05.ld / multiply /
// tcgen05.st) only in the tiles where one of its running maxima moved, which after
// the first few tiles is rare. Key tiles are 128 wide for prefill; decode-shaped
// calls (a handful of query rows per sequence) use 64-wide tiles, whose smaller
// footprint (112 KB of shared memory, 256 TMEM columns, < 170 registers) lets two
// CTAs share an SM and overlap one CTA's softmax with the other's loads.
//
// K/V come either from a paged cache [num_blocks, Hkv, block_size, D] through a
// block table (one TMA box per block) or from a contiguous [T, Hkv*D]-strided
// tensor (encoder). With several KV splits per sequence each CTA writes a
// normalised fp32 partial and its log-sum-exp; attention_merge_kernel folds them.
//
// The reference obtains attention from vLLM's FlashAttention wrappers
// (arctic_inference/vllm/attention/flash_attn_forest_cascade.py:1004-1026,
// 1725-1796), which on this architecture run the sm_80 mma.sync kernels.

#include <float.h>
#include <math.h>
#include <string.h>

#include "api.h"
#include "common/pdl.cuh"
#include "common/peer.cuh"
#include "common/ptx.cuh"
#include "common/tensormap.h"

namespace ab200 {

// Softmax warps: eight for 128-key tiles (two per TMEM lane quadrant, each taking half of the
// columns of S, of P and of O of the quadrant's 32 rows: one warp per scheduler cannot hide the
// latency of its TMEM reads and exponentials, and the softmax, not the tensor core, was the
// longest stage of a prefill tile), four for the 64-key decode tiles, whose two CTAs per SM
// already give every scheduler two softmax warps. Then the TMA warp and the MMA warp.
template <int TK>
struct AttnShape {
  static constexpr int kSoftmaxWarps = (TK == 128) ? 8 : 4;
  static constexpr int kThreads = (kSoftmaxWarps + 2) * 32;
};

struct AttnArgs {
  const int* work;          // [num_work][8], see AttnWork
  const int* block_tables;  // [num_seqs][max_blocks] (paged mode)
  int max_blocks;
  int block_size;  // 0 = contiguous K/V
  int G;           // query heads per KV head
  int Hq, Hkv;
  int causal;
  float scale_log2;  // softmax scale * log2(e)
  float scale;
  __nv_bfloat16* out;  // [T, Hq*D], row stride ldo
  long long ldo;
  float* o_part;    // [max_splits][T][Hq][D]
  float* lse_part;  // [max_splits][T][Hq]
  float* lse_out;   // optional [T][Hq]
  long long T;
  int* status;
  // Peer scatter (Ulysses head->sequence exchange fused into the epilogue): when
  // peer_tokens > 0, the output row of token t is written into peer_out[t / peer_tokens] at
  // row t % peer_tokens (the pointers already include this rank's column offset).
  int peer_tokens;
  __nv_bfloat16* peer_out[16];
  // completion signal to every rank once the last block has stored its rows (common/peer.cuh);
  // with split-KV the merge kernel sends it instead
  TailSignal sig;
};

// work item layout (int32 x 8)
//  0 seq index   1 first query token (row of q/out)   2 number of query tokens (0 = no-op)
//  3 position of the first query token   4 kv_start   5 kv_end (exclusive)
//  6 split index   7 number of splits of this sequence
//  In contiguous mode field 0 is the row of the sequence's first key in the K/V tensor.

template <int D, int TK>
__global__ void __launch_bounds__(AttnShape<TK>::kThreads, (TK == 64 ? 2 : 1))
attention_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const AttnArgs p) {
  constexpr int kHalves = D / 64;
  constexpr uint32_t kQBytes = 128 * D * 2;
  constexpr uint32_t kKVBytes = TK * D * 2;
  constexpr uint32_t kPBytes = 128 * TK * 2;
  constexpr uint32_t kHalf = TK * 128;     // bytes of one 64-wide d half of a K/V stage
  constexpr int kChunks = TK / 32;         // 32-column chunks of a row of S
  constexpr uint32_t kTmemCols = (TK == 128) ? 512 : 256;  // 2 S buffers + O
  constexpr int kPStages = (TK == 128) ? 2 : 1;  // decode tiles share the SM with a second CTA
  constexpr int kSW = AttnShape<TK>::kSoftmaxWarps;
  constexpr int kHalves2 = kSW / 4;                // warps per lane quadrant
  constexpr int kAttThreads = AttnShape<TK>::kThreads;
  constexpr int kTmaWarp = kSW, kMmaWarp = kSW + 1;
  // per-row values the two warps of a quadrant hand each other: tile maxima (double-buffered
  // by tile parity) and, at the end, the partial row sums
  // (1.5 KB: with 224 KB of tiles the CTA is within 3 KB of the 227 KB a block may own, so the
  // maxima travel as bf16, rounded up; the same words carry the fp32 row sums at the end)
  __shared__ __align__(16) __nv_bfloat16 pair_max[2][2][128];
  __shared__ short pair_seq[2][128];   // how many values thread (half, row) has published

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  const unsigned int total_blocks = gridDim.x;
  // The kernel before this one in the stream may still be running (programmatic dependent
  // launch): barrier and TMEM set-up and the clearing of the K/V stages below overlap its
  // tail. The work list is uploaded by the host before the step's first kernel and is the
  // only global memory read ahead of pdl_wait(); nothing is written before it.
  pdl_trigger();
  if (smem_u32(smem) & 1023u) {  // swizzled tiles need 1024-byte alignment
    pdl_wait();
    if (threadIdx.x == 0) report_error(p.status, kErrBadArgument, 900, (int)(smem_u32(smem) & 1023u));
    tail_signal(p.sig, total_blocks);
    return;
  }
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + kQBytes;          // 2 stages
  const uint32_t sV = sK + 2 * kKVBytes;     // 2 stages
  const uint32_t sP = sV + 2 * kKVBytes;
  uint8_t* pP = smem + kQBytes + 4 * kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kQBytes + 4 * kKVBytes + kPStages * kPBytes);
  const uint32_t bb = smem_u32(bars);
  // barrier indices
  const uint32_t q_full = bb;
  auto k_full = [&](int s) { return bb + 8u * (1 + s); };
  auto k_empty = [&](int s) { return bb + 8u * (3 + s); };
  auto v_full = [&](int s) { return bb + 8u * (5 + s); };
  auto v_empty = [&](int s) { return bb + 8u * (7 + s); };
  auto s_full = [&](int s) { return bb + 8u * (9 + s); };
  auto s_empty = [&](int s) { return bb + 8u * (11 + s); };
  auto o_full = [&](int s) { return bb + 8u * (13 + s); };
  auto o_empty = [&](int s) { return bb + 8u * (15 + s); };
  auto p_full = [&](int s) { return bb + 8u * (17 + s); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // one block per (work item, KV head), work item major: blocks start in work-list order, so
  // the planner's order (heaviest items first, the pieces of cut sequences last) is the order
  // in which the GPU picks them up
  const int* wk = p.work + (long long)(blockIdx.x / p.Hkv) * 8;
  const int seq = wk[0];
  const int q_tok0 = wk[1];
  const int n_q_tok = wk[2];
  if (n_q_tok <= 0) {  // padding entry of a fixed-size work list
    pdl_wait();
    tail_signal(p.sig, total_blocks);
    return;
  }
  const int q_pos0 = wk[3];
  const int kv_start = wk[4];
  int kv_end = wk[5];
  const int split = wk[6];
  const int num_splits = wk[7];
  const int kvh = blockIdx.x % p.Hkv;
  if (p.causal) kv_end = min(kv_end, q_pos0 + n_q_tok);
  const int n_tiles = kv_end > kv_start ? (kv_end - kv_start + TK - 1) / TK : 0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full(s), 1);
      mbar_init(k_empty(s), 1);
      mbar_init(v_full(s), 1);
      mbar_init(v_empty(s), 1);
      mbar_init(s_full(s), 1);
      mbar_init(s_empty(s), kSW);
      mbar_init(o_full(s), 1);
      mbar_init(o_empty(s), 4);
    }
    mbar_init(p_full(0), kSW);
    mbar_init(p_full(1), kSW);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  // Stale shared memory may hold non-finite bit patterns; keys that are never
  // loaded (past the end of a sequence) are multiplied by P = 0 and must be finite.
  for (int i = threadIdx.x; i < 256; i += kAttThreads) (&pair_seq[0][0])[i] = 0;
  // (counts stay far below 32767: a sequence of 2^21 keys is 16384 tiles)
  {
    uint4* z = reinterpret_cast<uint4*>(smem + kQBytes);
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int i = threadIdx.x; i < (int)(4 * kKVBytes / 16); i += kAttThreads) z[i] = zero;
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS = tmem_base;           // S buffers at columns 0, TK
  const uint32_t tO = tmem_base + 2 * TK;  // output accumulator, D columns

  if (warp == kTmaWarp) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, kQBytes);
      for (int h = 0; h < kHalves; ++h)
        tma_load_4d(sQ + h * 16384u, &tmap_q, q_full, h * 64, 0, kvh, q_tok0);
    }
    const int bs = p.block_size;
    const int* bt = bs > 0 ? p.block_tables + (long long)seq * p.max_blocks : nullptr;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j & 1;
      const uint32_t ph = (uint32_t)(j >> 1) & 1u;
      const int key0 = kv_start + j * TK;
      const int nkeys = min(TK, kv_end - key0);
      for (int kv = 0; kv < 2; ++kv) {
        const uint32_t full = kv == 0 ? k_full(st) : v_full(st);
        const uint32_t empty = kv == 0 ? k_empty(st) : v_empty(st);
        const uint32_t dst = (kv == 0 ? sK : sV) + (uint32_t)st * kKVBytes;
        const CUtensorMap* tm = kv == 0 ? &tmap_k : &tmap_v;
        if (!mbar_wait(empty, ph ^ 1u, abort_flag, p.status, 500 + kv * 10 + st, j)) {
          ok = false;
          break;
        }
        if (bs > 0) {
          const int nblk = (nkeys + bs - 1) / bs;
          if (lane == 0) mbar_arrive_expect_tx(full, (uint32_t)(nblk * bs * D * 2));
          __syncwarp();
          if (lane < nblk) {
            const int bid = bt[key0 / bs + lane];
            for (int h = 0; h < kHalves; ++h)
              tma_load_4d(dst + h * kHalf + (uint32_t)(lane * bs) * 128u, tm, full, h * 64, 0, kvh,
                          bid);
          }
        } else {
          if (lane == 0) {
            mbar_arrive_expect_tx(full, kKVBytes);
            for (int h = 0; h < kHalves; ++h)
              tma_load_3d(dst + h * kHalf, tm, full, h * 64, kvh, seq + key0);
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0 && n_tiles > 0) {
      const uint32_t idesc_s = make_idesc(128, TK, 1, 1, 0, 0);
      const uint32_t idesc_pv = make_idesc(128, D, 1, 1, 0, 1);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, 600, 0);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (!mbar_wait(k_full(st), ph, abort_flag, p.status, 610 + st, j)) return false;
        if (!mbar_wait(s_empty(st), ph ^ 1u, abort_flag, p.status, 620 + st, j)) return false;
        tc_fence_after();
        const uint32_t kb = sK + (uint32_t)st * kKVBytes;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t qd = make_desc_kmajor_sw128(sQ + (uint32_t)(k / 4) * 16384u) + 2u * (k % 4);
          const uint64_t kd = make_desc_kmajor_sw128(kb + (uint32_t)(k / 4) * kHalf) + 2u * (k % 4);
          umma_f16_ss(tS + (uint32_t)st * TK, qd, kd, idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(k_empty(st));
        tc_commit(s_full(st));
        return true;
      };
      auto issue_pv = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (!mbar_wait(v_full(st), ph, abort_flag, p.status, 630 + st, j)) return false;
        // P(j) sits in buffer j % kPStages; its barrier completes once per use of that buffer
        const int pst = j % kPStages;
        const uint32_t pph = (uint32_t)(j / kPStages) & 1u;
        if (!mbar_wait(p_full(pst), pph, abort_flag, p.status, 640, j)) return false;
        tc_fence_after();
        const uint32_t vb = sV + (uint32_t)st * kKVBytes;
        const uint32_t pb = sP + (uint32_t)pst * kPBytes;
#pragma unroll
        for (int k = 0; k < TK / 16; ++k) {
          const uint64_t pd = make_desc_kmajor_sw128(pb + (uint32_t)(k / 4) * 16384u) + 2u * (k % 4);
          const uint64_t vd = make_desc_mnmajor_sw128(vb, kHalf) + 128u * k;
          // O accumulates in tensor memory across key tiles
          umma_f16_ss(tO, pd, vd, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(v_empty(st));
        tc_commit(o_full(st));
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_s(j + 1);
        if (ok) ok = issue_pv(j);
      }
    }
  } else {
    // ------------------------------ softmax warps ------------------------------
    const int quad = warp & 3;          // TMEM lane quadrant this warp may read
    const int half = warp >> 2;         // which half of the quadrant's columns it takes
    const int row = quad * 32 + lane;
    // The two warps of a quadrant hand each other per-row values through shared memory: a
    // thread publishes a value, then its count of published values; its partner (same lane of
    // the other warp) polls that count, bounded like every other wait of the kernel.
    int published = 0;
    auto pair_publish = [&]() {
      __threadfence_block();
      ++published;
      *reinterpret_cast<volatile short*>(&pair_seq[half][row]) = (short)published;
    };
    auto pair_wait = [&]() -> bool {
      volatile short* seq = reinterpret_cast<volatile short*>(&pair_seq[half ^ 1][row]);
      unsigned int spins = 0;
      unsigned long long t0 = 0;
      while (*seq < published) {
        if ((++spins & 63u) == 0u) {
          if (*abort_flag) return false;
          if (t0 == 0) t0 = globaltimer_ns();
          else if (globaltimer_ns() - t0 > kWaitLimitNs) {
            *abort_flag = 1;
            report_error(p.status, kErrBarrierTimeout, 730, published);
            return false;
          }
        }
      }
      __threadfence_block();
      return true;
    };
    constexpr int kLocalChunks = kChunks / kHalves2;   // 32-column chunks of S per warp
    const int c_first = half * kLocalChunks;
    const int tok_local = row / p.G;
    const int g = row % p.G;
    const bool valid_row = tok_local < n_q_tok;
    const int q_pos = q_pos0 + tok_local;
    const int limit = p.causal ? min(q_pos, kv_end - 1) : kv_end - 1;  // last visible key
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    float m = -INFINITY;
    float l = 0.f;
    uint8_t* p_row0 = pP + (size_t)row * 128;
    bool ok = true;
    const uint32_t to = tO + lane_off;

    // Decode tiles hold a few valid rows: warps whose 32 rows are all padding only keep the
    // barrier protocol going (their rows of P are never read back by anyone).
    const bool warp_active = quad * 32 < n_q_tok * p.G;
    const float sc = p.scale_log2;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j & 1;
      const uint32_t ph = (uint32_t)(j >> 1) & 1u;
      const int key0 = kv_start + j * TK;
      if (!mbar_wait(s_full(st), ph, abort_flag, p.status, 700 + st, j)) {
        ok = false;
        break;
      }
      if (!warp_active) {
        // staying one product behind the active warps keeps the arrival counts of
        // consecutive tiles apart
        if (j > 0 && !mbar_wait(o_full((j - 1) & 1), (uint32_t)((j - 1) >> 1) & 1u, abort_flag,
                                p.status, 711, j)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          mbar_arrive(s_empty(st));
          mbar_arrive(p_full(j % kPStages));
        }
        continue;
      }
      tc_fence_after();
      const uint32_t ts = tS + (uint32_t)st * TK + lane_off;
      const bool need_mask = key0 + TK - 1 > limit;
      uint32_t ra[32], rb[32];
      // pass 1: row maximum (four independent chains; one warp per scheduler cannot hide a
      // long dependent chain). TMEM reads are software-pipelined.
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
      tmem_ld_x32(ts + (uint32_t)c_first * 32u, ra);
#pragma unroll
      for (int cl = 0; cl < kLocalChunks; ++cl) {
        const int c = c_first + cl;
        uint32_t(&cur)[32] = (cl & 1) ? rb : ra;
        uint32_t(&nxt)[32] = (cl & 1) ? ra : rb;
        tmem_ld_wait_dep(cur);
        // next chunk; after the last one, this warp's first chunk again for pass 2
        tmem_ld_x32(ts + (uint32_t)(c_first + (cl + 1) % kLocalChunks) * 32u, nxt);
        if (need_mask) {
#pragma unroll
          for (int t = 0; t < 32; t += 4) {
            const int k = key0 + c * 32 + t;
            mx0 = fmaxf(mx0, k + 0 <= limit ? __uint_as_float(cur[t + 0]) : -INFINITY);
            mx1 = fmaxf(mx1, k + 1 <= limit ? __uint_as_float(cur[t + 1]) : -INFINITY);
            mx2 = fmaxf(mx2, k + 2 <= limit ? __uint_as_float(cur[t + 2]) : -INFINITY);
            mx3 = fmaxf(mx3, k + 3 <= limit ? __uint_as_float(cur[t + 3]) : -INFINITY);
          }
        } else {
#pragma unroll
          for (int t = 0; t < 32; t += 4) {
            mx0 = fmaxf(mx0, __uint_as_float(cur[t + 0]));
            mx1 = fmaxf(mx1, __uint_as_float(cur[t + 1]));
            mx2 = fmaxf(mx2, __uint_as_float(cur[t + 2]));
            mx3 = fmaxf(mx3, __uint_as_float(cur[t + 3]));
          }
        }
      }
      float m_tile = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      if (kHalves2 == 2) {
        // the row's maximum over the other warp's columns
        // Any common upper bound of the row's scores serves as the softmax reference point, so
        // each warp rounds its maximum up to bf16 and both use the larger of the two.
        const __nv_bfloat16 mine = __float2bfloat16_ru(m_tile);
        *reinterpret_cast<volatile unsigned short*>(&pair_max[j & 1][half][row]) =
            __bfloat16_as_ushort(mine);
        pair_publish();
        if (!__all_sync(0xffffffffu, pair_wait())) {
          ok = false;
          break;
        }
        const unsigned short theirs =
            *reinterpret_cast<volatile unsigned short*>(&pair_max[j & 1][half ^ 1][row]);
        m_tile = fmaxf(__bfloat162float(mine), __bfloat162float(__ushort_as_bfloat16(theirs)));
      }
      const float m_new = fmaxf(m, m_tile);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      // rows that have seen no key yet (m = -inf) hold O = 0 and l = 0: nothing to rescale
      const float alpha = (m == -INFINITY) ? 1.0f : ex2_approx((m - m_safe) * sc);
      const float neg_ms = -m_safe * sc;
      // A rescale of O must not race with PV(j-1) accumulating into it, and P(j) overwrites the
      // buffer that PV(j - kPStages) reads from: wait for the later of the products concerned.
      // The running maxima settle after a few tiles; from then on the softmax of tile j runs
      // while PV(j-1) is still on the tensor core (two P buffers) and only rare tiles rescale.
      if (j > 0) {
        const bool rescale = !__all_sync(0xffffffffu, alpha == 1.0f);
        const int jw = (kPStages == 1 || rescale) ? j - 1 : j - 2;
        if (jw >= 0 && !mbar_wait(o_full(jw & 1), (uint32_t)(jw >> 1) & 1u, abort_flag, p.status,
                                  710, j)) {
          ok = false;
          break;
        }
        if (rescale) {
          tc_fence_after();
          uint32_t rc[32];
#pragma unroll
          for (int cl = 0; cl < D / 32 / kHalves2; ++cl) {
            const int c = half * (D / 32 / kHalves2) + cl;
            tmem_ld_x32(to + (uint32_t)c * 32u, rc);
            tmem_ld_wait_dep(rc);
#pragma unroll
            for (int t = 0; t < 32; ++t) rc[t] = __float_as_uint(__uint_as_float(rc[t]) * alpha);
            tmem_st_x32(to + (uint32_t)c * 32u, rc);
          }
          tmem_st_wait();
        }
      }
      // pass 2: probabilities -> swizzled shared memory (chunk 0 is already in flight in the
      // buffer pass 1 left as "next")
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
      for (int cl = 0; cl < kLocalChunks; ++cl) {
        const int c = c_first + cl;
        constexpr int kFlip = kLocalChunks & 1;  // parity of the buffer that holds the first chunk
        uint32_t(&cur)[32] = ((cl + kFlip) & 1) ? rb : ra;
        uint32_t(&nxt)[32] = ((cl + kFlip) & 1) ? ra : rb;
        tmem_ld_wait_dep(cur);
        if (cl + 1 < kLocalChunks) tmem_ld_x32(ts + (uint32_t)(c + 1) * 32u, nxt);
        uint32_t pk[16];
#pragma unroll
        for (int t = 0; t < 32; t += 4) {
          float e0 = ex2_approx(fmaf(__uint_as_float(cur[t + 0]), sc, neg_ms));
          float e1 = ex2_approx(fmaf(__uint_as_float(cur[t + 1]), sc, neg_ms));
          float e2 = ex2_approx(fmaf(__uint_as_float(cur[t + 2]), sc, neg_ms));
          float e3 = ex2_approx(fmaf(__uint_as_float(cur[t + 3]), sc, neg_ms));
          if (need_mask) {
            const int k = key0 + c * 32 + t;
            e0 = k + 0 <= limit ? e0 : 0.f;
            e1 = k + 1 <= limit ? e1 : 0.f;
            e2 = k + 2 <= limit ? e2 : 0.f;
            e3 = k + 3 <= limit ? e3 : 0.f;
          }
          s0 += e0;
          s1 += e1;
          s2 += e2;
          s3 += e3;
          pk[t / 2] = pack_bf16x2(e0, e1);
          pk[t / 2 + 1] = pack_bf16x2(e2, e3);
        }
        uint8_t* line = p_row0 + (size_t)(j % kPStages) * kPBytes + (size_t)(c >> 1) * 16384;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int chunk = ((c & 1) * 4 + i) ^ (row & 7);
          *reinterpret_cast<uint4*>(line + chunk * 16) =
              make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
        }
      }
      l = l * alpha + ((s0 + s1) + (s2 + s3));
      m = m_new;
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(s_empty(st));
        mbar_arrive(p_full(j % kPStages));
      }
    }
    if (ok && n_tiles > 0 && warp_active) {
      const int jl = n_tiles - 1;
      if (!mbar_wait(o_full(jl & 1), (uint32_t)(jl >> 1) & 1u, abort_flag, p.status, 720, jl))
        ok = false;
      tc_fence_after();
    }
    if (ok && warp_active && kHalves2 == 2) {
      // each warp summed the probabilities of its own columns: the row's sum is both parts
      // The fp32 sums reuse the words of the maxima: one more round first, after which the
      // partner has read the last tile's maximum.
      float* sums = reinterpret_cast<float*>(&pair_max[0][0][0]);   // [2][128]
      pair_publish();
      bool got = __all_sync(0xffffffffu, pair_wait());
      if (got) {
        *reinterpret_cast<volatile float*>(&sums[half * 128 + row]) = l;
        pair_publish();
        got = __all_sync(0xffffffffu, pair_wait());
      }
      if (!got) ok = false;
      else l += *reinterpret_cast<volatile float*>(&sums[(half ^ 1) * 128 + row]);
    }
    if (ok && warp_active) {  // warp-uniform: every lane takes part in the TMEM reads
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const long long tok = (long long)q_tok0 + tok_local;
      const int head = kvh * p.G + g;
      const float lse = l > 0.f ? m * p.scale + logf(l) : -INFINITY;
      __nv_bfloat16* dst16 = p.out + tok * p.ldo + (long long)head * D;
      if (p.peer_tokens > 0)
        dst16 = p.peer_out[tok / p.peer_tokens] + (tok % p.peer_tokens) * p.ldo + (long long)head * D;
      float* dst32 = p.o_part + (((long long)split * p.T + tok) * p.Hq + head) * D;
      if (num_splits <= 1 && n_tiles > 0) {
        // Normalised rows go through the Q tile's shared memory (free once the last product
        // has completed; same 128-byte swizzle, so the writes are conflict-free) and leave as
        // whole rows: one store instruction covers 32 / (D / 8) complete rows of D bf16 instead
        // of 16-byte pieces of 32 different rows -- what a peer's memory over NVLink needs.
        constexpr int kCh = D / 8;  // 16-byte chunks per row
        uint8_t* my_row = smem + (size_t)row * 128;
#pragma unroll
        for (int cl = 0; cl < D / 32 / kHalves2; ++cl) {
          const int c = half * (D / 32 / kHalves2) + cl;   // this warp's share of O's columns
          uint32_t rc[32];
          tmem_ld_x32(to + (uint32_t)c * 32u, rc);
          tmem_ld_wait_dep(rc);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int j = c * 4 + i;
            uint4 q;
            q.x = pack_bf16x2(__uint_as_float(rc[8 * i]) * inv_l, __uint_as_float(rc[8 * i + 1]) * inv_l);
            q.y = pack_bf16x2(__uint_as_float(rc[8 * i + 2]) * inv_l, __uint_as_float(rc[8 * i + 3]) * inv_l);
            q.z = pack_bf16x2(__uint_as_float(rc[8 * i + 4]) * inv_l, __uint_as_float(rc[8 * i + 5]) * inv_l);
            q.w = pack_bf16x2(__uint_as_float(rc[8 * i + 6]) * inv_l, __uint_as_float(rc[8 * i + 7]) * inv_l);
            *reinterpret_cast<uint4*>(my_row + (size_t)(j >> 3) * 16384 + (((j & 7) ^ (row & 7)) * 16)) = q;
          }
        }
        __syncwarp();
        bool staged = true;
        if (kHalves2 == 2) {   // the other warp's columns of the same rows
          pair_publish();
          staged = __all_sync(0xffffffffu, pair_wait());
        }
        const unsigned long long my_dst =
            (valid_row && staged) ? reinterpret_cast<unsigned long long>(dst16) : 0ull;
        const int j = lane % kCh;
#pragma unroll
        for (int it = 0; it < kCh; ++it) {
          if (it % kHalves2 != half) continue;            // the pair shares the rows' stores
          const int rl = it * (32 / kCh) + lane / kCh;  // row of this quadrant
          const int rr = quad * 32 + rl;
          const unsigned long long d = __shfl_sync(0xffffffffu, my_dst, rl);
          if (d != 0ull) {
            const uint4 q = *reinterpret_cast<const uint4*>(
                smem + (size_t)(j >> 3) * 16384 + (size_t)rr * 128 + (((j & 7) ^ (rr & 7)) * 16));
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(d) + 8 * j) = q;
          }
        }
        if (valid_row && p.lse_out && half == 0) p.lse_out[tok * p.Hq + head] = lse;
      } else {
#pragma unroll
      for (int cl = 0; cl < D / 32 / kHalves2; ++cl) {
        const int c = half * (D / 32 / kHalves2) + cl;
        uint32_t rc[32];
        if (n_tiles > 0) {
          tmem_ld_x32(to + (uint32_t)c * 32u, rc);
          tmem_ld_wait_dep(rc);
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t) rc[t] = 0u;
        }
        if (valid_row) {
          if (num_splits <= 1) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 q;
              q.x = pack_bf16x2(__uint_as_float(rc[i]) * inv_l, __uint_as_float(rc[i + 1]) * inv_l);
              q.y = pack_bf16x2(__uint_as_float(rc[i + 2]) * inv_l, __uint_as_float(rc[i + 3]) * inv_l);
              q.z = pack_bf16x2(__uint_as_float(rc[i + 4]) * inv_l, __uint_as_float(rc[i + 5]) * inv_l);
              q.w = pack_bf16x2(__uint_as_float(rc[i + 6]) * inv_l, __uint_as_float(rc[i + 7]) * inv_l);
              *reinterpret_cast<uint4*>(dst16 + c * 32 + i) = q;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              *reinterpret_cast<float4*>(dst32 + c * 32 + i) = make_float4(
                  __uint_as_float(rc[i]) * inv_l, __uint_as_float(rc[i + 1]) * inv_l,
                  __uint_as_float(rc[i + 2]) * inv_l, __uint_as_float(rc[i + 3]) * inv_l);
          }
        }
      }
      if (valid_row && half == 0) {
        if (num_splits <= 1) {
          if (p.lse_out) p.lse_out[tok * p.Hq + head] = lse;
        } else {
          p.lse_part[((long long)split * p.T + tok) * p.Hq + head] = lse;
        }
      }
      }
    }
  }

  tail_signal(p.sig, total_blocks);
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Fold split-KV partials: out = sum_s w_s O_s / sum_s w_s, w_s = exp(lse_s - max lse).
// tok_splits[t] = number of splits that cover token t (<= 1: nothing to do).
template <int D>
__global__ void attention_merge_kernel(const float* __restrict__ o_part,
                                       const float* __restrict__ lse_part,
                                       const int* __restrict__ tok_splits, long long T, int Hq,
                                       __nv_bfloat16* __restrict__ out, long long ldo,
                                       float* __restrict__ lse_out, AttnArgs pa) {
  pdl_wait();
  pdl_trigger();
  const long long tok = blockIdx.x;
  const int ns = tok_splits[tok];
  if (ns <= 1) {
    tail_signal(pa.sig, gridDim.x);
    return;
  }
  long long out_row = tok;
  if (pa.peer_tokens > 0) {
    out = pa.peer_out[tok / pa.peer_tokens];
    out_row = tok % pa.peer_tokens;
  }
  for (int idx = threadIdx.x; idx < Hq * (D / 4); idx += blockDim.x) {
    const int head = idx / (D / 4);
    const int d4 = (idx % (D / 4)) * 4;
    float mx = -INFINITY;
    for (int s = 0; s < ns; ++s) mx = fmaxf(mx, lse_part[((long long)s * T + tok) * Hq + head]);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float wsum = 0.f;
    for (int s = 0; s < ns; ++s) {
      const float lse = lse_part[((long long)s * T + tok) * Hq + head];
      const float w = (lse == -INFINITY) ? 0.f : __expf(lse - mx);
      const float4 v =
          *reinterpret_cast<const float4*>(o_part + (((long long)s * T + tok) * Hq + head) * D + d4);
      acc.x += w * v.x;
      acc.y += w * v.y;
      acc.z += w * v.z;
      acc.w += w * v.w;
      wsum += w;
    }
    const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
    uint2 q;
    q.x = pack_bf16x2(acc.x * inv, acc.y * inv);
    q.y = pack_bf16x2(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(out + out_row * ldo + (long long)head * D + d4) = q;
    if (lse_out && d4 == 0) lse_out[tok * Hq + head] = wsum > 0.f ? mx + logf(wsum) : -INFINITY;
  }
  tail_signal(pa.sig, gridDim.x);
}

template <int D, int TK>
static int launch_attention(const void* q, long long ldq, const void* k, const void* v,
                            long long ld_kv, long long num_blocks, int block_size,
                            const int* block_tables, int max_blocks, const int* work, int num_work,
                            const int* tok_splits, int max_splits, long long T, int Hq, int Hkv,
                            int causal, float scale, void* out, long long ldo, float* o_part,
                            float* lse_part, float* lse_out, int* status, cudaStream_t stream,
                            const void* const* peer_ptrs = nullptr, int world = 0,
                            int peer_tokens = 0, const Ab200PeerSync* sync = nullptr) {
  const int G = Hq / Hkv;
  if (peer_tokens > 0 && (world < 1 || world > 16 || peer_ptrs == nullptr)) return -2;
  if (G <= 0 || Hq % Hkv || 128 % G) return -2;
  if (block_size > 0 && (TK % block_size || block_size < 8)) return -2;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return -3;
  const size_t smem =
      128 * D * 2 + 4 * (size_t)TK * D * 2 + (TK == 128 ? 2 : 1) * (size_t)128 * TK * 2 + 256;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(attention_kernel<D, TK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return -3;
    attr_set[dev] = true;
  }
  CUtensorMap tq, tk, tv;
  {
    // q viewed as [T][Hkv][G][D]
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)G, (uint64_t)Hkv, (uint64_t)T};
    const uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)G * D * 2, (uint64_t)ldq * 2};
    const uint32_t box[4] = {64, (uint32_t)G, 1, (uint32_t)(128 / G)};
    if (make_tmap_nd(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dims, strides, box) != 0) return -4;
  }
  if (block_size > 0) {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)block_size, (uint64_t)Hkv, (uint64_t)num_blocks};
    const uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)block_size * D * 2,
                                 (uint64_t)Hkv * block_size * D * 2};
    const uint32_t box[4] = {64, (uint32_t)block_size, 1, 1};
    if (make_tmap_nd(&tk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dims, strides, box) != 0) return -4;
    if (make_tmap_nd(&tv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dims, strides, box) != 0) return -4;
  } else {
    // contiguous: k/v rows are tokens with stride ld_kv, heads packed [Hkv][D]
    const uint64_t dims[3] = {(uint64_t)D, (uint64_t)Hkv, (uint64_t)num_blocks /* = rows */};
    const uint64_t strides[2] = {(uint64_t)D * 2, (uint64_t)ld_kv * 2};
    const uint32_t box[3] = {64, 1, (uint32_t)TK};
    if (make_tmap_nd(&tk, k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box) != 0) return -4;
    if (make_tmap_nd(&tv, v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box) != 0) return -4;
  }
  AttnArgs a;
  memset(&a, 0, sizeof(a));
  a.peer_tokens = peer_tokens;
  for (int i = 0; i < world && peer_tokens > 0; ++i)
    a.peer_out[i] = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(peer_ptrs[i]));
  a.work = work;
  a.block_tables = block_tables;
  a.max_blocks = max_blocks;
  a.block_size = block_size;
  a.G = G;
  a.Hq = Hq;
  a.Hkv = Hkv;
  a.causal = causal;
  a.scale = scale;
  a.scale_log2 = scale * 1.4426950408889634f;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.ldo = ldo;
  a.o_part = o_part;
  a.lse_part = lse_part;
  a.lse_out = lse_out;
  a.T = T;
  a.status = status;
  TailSignal sig;
  memset(&sig, 0, sizeof(sig));
  if (sync != nullptr && sync->sig_world > 0) {
    if (sync->sig_world > kMaxPeers) return -2;
    for (int i = 0; i < sync->sig_world; ++i)
      sig.flags[i] = reinterpret_cast<unsigned int*>(const_cast<void*>(sync->sig_flag_ptrs[i]));
    sig.done_ctr = reinterpret_cast<unsigned int*>(sync->sig_done_ctr);
    sig.epoch_ctr = reinterpret_cast<unsigned int*>(sync->sig_epoch_ctr);
    sig.my_rank = sync->sig_rank;
    sig.world = sync->sig_world;
  }
  if (max_splits <= 1) a.sig = sig;
  dim3 grid((unsigned)num_work * (unsigned)Hkv);
  (void)launch_pdl(attention_kernel<D, TK>, grid, dim3(AttnShape<TK>::kThreads), smem, stream, tq,
                   tk, tv, a);
  if (cudaGetLastError() != cudaSuccess) return -5;
  a.sig = sig;
  if (max_splits > 1) {
    (void)launch_pdl(attention_merge_kernel<D>, dim3((unsigned)T), dim3(128), 0, stream, o_part,
                     lse_part, tok_splits, T, Hq, reinterpret_cast<__nv_bfloat16*>(out), ldo,
                     lse_out, a);
    if (cudaGetLastError() != cudaSuccess) return -5;
  }
  return 0;
}

}  // namespace ab200

using namespace ab200;

extern "C" {

#define AB200_ATTN_DISPATCH(...)                                                       \
  do {                                                                                 \
    const bool small = tile_keys == 64 && (block_size == 0 || block_size <= 64);        \
    if (D == 128) return small ? launch_attention<128, 64>(__VA_ARGS__)                \
                               : launch_attention<128, 128>(__VA_ARGS__);              \
    if (D == 64) return small ? launch_attention<64, 64>(__VA_ARGS__)                  \
                              : launch_attention<64, 128>(__VA_ARGS__);                \
    return -2;                                                                         \
  } while (0)

// q: [T, Hq*D] rows with stride ldq. Paged mode (block_size > 0): k/v are caches
// [num_blocks, Hkv, block_size, D]. Contiguous mode (block_size == 0): k/v are
// [num_blocks(=rows), Hkv*D] with row stride ld_kv. `work` is an int32 [num_work, 8]
// device array (layout above). With max_splits > 1, o_part/lse_part/tok_splits
// must be given: o_part fp32 [max_splits, T, Hq, D], lse_part fp32 [max_splits, T, Hq].
// tile_keys: 128 (prefill) or 64 (decode-shaped calls: few query rows per sequence).
int ab200_attention(const void* q, long long ldq, const void* k, const void* v, long long ld_kv,
                    long long num_blocks, int block_size, const void* block_tables, int max_blocks,
                    const void* work, int num_work, const void* tok_splits, int max_splits,
                    long long T, int Hq, int Hkv, int D, int causal, float scale, void* out,
                    long long ldo, void* o_part, void* lse_part, void* lse_out, int tile_keys,
                    int* status, cudaStream_t stream) {
  if (num_work <= 0 || T <= 0) return 0;
  if ((ldq % 8) || (ldo % 8) || (ld_kv % 8)) return -2;
  if (max_splits > 1 && (o_part == nullptr || lse_part == nullptr || tok_splits == nullptr)) return -2;
  AB200_ATTN_DISPATCH(q, ldq, k, v, ld_kv, num_blocks, block_size,
                      reinterpret_cast<const int*>(block_tables), max_blocks,
                      reinterpret_cast<const int*>(work), num_work,
                      reinterpret_cast<const int*>(tok_splits), max_splits, T, Hq, Hkv, causal, scale,
                      out, ldo, reinterpret_cast<float*>(o_part), reinterpret_cast<float*>(lse_part),
                      reinterpret_cast<float*>(lse_out), status, stream);
}

// Paged attention whose output rows are scattered to `world` peer buffers (see AttnArgs):
// token t goes to peer_ptrs[t / peer_tokens], row t % peer_tokens, row stride ldo.
int ab200_attention_scatter(const void* q, long long ldq, const void* k, const void* v,
                            long long num_blocks, int block_size, const void* block_tables,
                            int max_blocks, const void* work, int num_work,
                            const void* tok_splits, int max_splits, long long T, int Hq, int Hkv,
                            int D, float scale, const void* const* peer_ptrs, int world,
                            int peer_tokens, long long ldo, void* o_part, void* lse_part,
                            int tile_keys, int* status, cudaStream_t stream) {
  return ab200_attention_scatter_sync(q, ldq, k, v, num_blocks, block_size, block_tables, max_blocks,
                                      work, num_work, tok_splits, max_splits, T, Hq, Hkv, D, scale,
                                      peer_ptrs, world, peer_tokens, ldo, o_part, lse_part,
                                      tile_keys, nullptr, status, stream);
}

// The same with a completion signal to every rank (sync->sig_*) instead of a barrier kernel
// after it: the consumers of the scattered rows wait for the signal themselves.
int ab200_attention_scatter_sync(const void* q, long long ldq, const void* k, const void* v,
                                 long long num_blocks, int block_size, const void* block_tables,
                                 int max_blocks, const void* work, int num_work,
                                 const void* tok_splits, int max_splits, long long T, int Hq,
                                 int Hkv, int D, float scale, const void* const* peer_ptrs,
                                 int world, int peer_tokens, long long ldo, void* o_part,
                                 void* lse_part, int tile_keys, const Ab200PeerSync* sync,
                                 int* status, cudaStream_t stream) {
  if (num_work <= 0 || T <= 0) return 0;
  if ((ldq % 8) || (ldo % 8) || peer_tokens <= 0) return -2;
  if (max_splits > 1 && (o_part == nullptr || lse_part == nullptr || tok_splits == nullptr)) return -2;
  AB200_ATTN_DISPATCH(q, ldq, k, v, 0, num_blocks, block_size,
                      reinterpret_cast<const int*>(block_tables), max_blocks,
                      reinterpret_cast<const int*>(work), num_work,
                      reinterpret_cast<const int*>(tok_splits), max_splits, T, Hq, Hkv, 1, scale,
                      const_cast<void*>(peer_ptrs[0]), ldo, reinterpret_cast<float*>(o_part),
                      reinterpret_cast<float*>(lse_part), nullptr, status, stream, peer_ptrs, world,
                      peer_tokens, sync);
}

}  // extern "C"
