// Draft-model (Arctic speculator) kernels for sm_100a and greedy draft verification.
//
//   spec_ln        y = x * rsqrt(mean(x^2) + eps) [* w] [+ b]          (one pass, row in registers)
//   mlp_spec_step  state = GELU(LN(proj + scale * E[tok]))              (MLP speculator head)
//   sum_lstm       the LSTM-style head: gates = proj + alpha * repeat4(E[tok]),
//                  c = c_prev * sig(f) + GELU(LN_c(g_c)) * sig(i),  h = GELU(LN_s(c)) * sig(o)
//                  with the embedding gather fused in and the row held in registers, so the
//                  cell is a single pass over HBM
//   verify_greedy  per request: longest prefix of the draft that equals the target's arg-max,
//                  the bonus token, and the row whose hidden state seeds the next draft
//
// The reference implements the normalisation and the cell as separate multi-pass kernels
// (csrc/custom_ops/speculator_ln.cu:21-150, csrc/custom_ops/sum_lstm.cu:28-291) and takes
// verification / next-token preparation from vLLM (arctic_inference/vllm/model_runner.py:594-617,
// arctic_inference/vllm/spec_dec/arctic_proposer.py:239-290).

#include <math.h>

#include "api.h"
#include "common/pdl.cuh"
#include "common/ptx.cuh"

namespace ab200 {

typedef __nv_bfloat16 bf16;
constexpr int kSpecThreads = 256;
constexpr int kSpecMaxPerThread = 32;  // elements of a row per thread -> rows up to 8192

__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < (kSpecThreads / 32) ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float gelu_f(float x, int tanh_approx) {
  if (tanh_approx) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.f + tanhf(u));
  }
  return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
}
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float ldf(const bf16* p, long long i) { return __bfloat162float(p[i]); }

// ---------------------------------------------------------------------------- spec_ln
__global__ void __launch_bounds__(kSpecThreads)
spec_ln_kernel(const bf16* __restrict__ x, long long ldx, const bf16* __restrict__ w,
               const bf16* __restrict__ b, bf16* __restrict__ y, long long ldy, int hidden,
               float eps, float out_scale) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[32];
  const long long row = blockIdx.x;
  float v[kSpecMaxPerThread];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kSpecMaxPerThread; ++j) {
    const int i = threadIdx.x + j * kSpecThreads;
    v[j] = i < hidden ? ldf(x, row * ldx + i) : 0.f;
    ss += v[j] * v[j];
  }
  const float inv = rsqrtf(block_sum_256(ss, red) / (float)hidden + eps) * out_scale;
#pragma unroll
  for (int j = 0; j < kSpecMaxPerThread; ++j) {
    const int i = threadIdx.x + j * kSpecThreads;
    if (i < hidden) {
      float o = v[j] * inv;
      if (w) o *= ldf(w, i);
      if (b) o += ldf(b, i);
      y[row * ldy + i] = __float2bfloat16(o);
    }
  }
}

// ---------------------------------------------------------------------- mlp_spec_step
__global__ void __launch_bounds__(kSpecThreads)
mlp_spec_step_kernel(const bf16* __restrict__ proj, long long ldp, const bf16* __restrict__ emb,
                     const long long* __restrict__ tok, float emb_scale,
                     const bf16* __restrict__ ln_w, const bf16* __restrict__ ln_b,
                     bf16* __restrict__ out, long long ldo, int dim, float eps, int tanh_approx) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const bf16* e = emb + tok[row] * (long long)dim;
  float v[kSpecMaxPerThread];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kSpecMaxPerThread; ++j) {
    const int i = threadIdx.x + j * kSpecThreads;
    v[j] = i < dim ? ldf(proj, row * ldp + i) + emb_scale * ldf(e, i) : 0.f;
    ss += v[j] * v[j];
  }
  const float inv = rsqrtf(block_sum_256(ss, red) / (float)dim + eps);
#pragma unroll
  for (int j = 0; j < kSpecMaxPerThread; ++j) {
    const int i = threadIdx.x + j * kSpecThreads;
    if (i < dim) {
      float o = v[j] * inv;
      if (ln_w) o *= ldf(ln_w, i);
      if (ln_b) o += ldf(ln_b, i);
      out[row * ldo + i] = __float2bfloat16(gelu_f(o, tanh_approx));
    }
  }
}

// --------------------------------------------------------------------------- sum_lstm
// gates: [B, 4*D] in the order forget, input, output, cell. emb: table [V, D] (shared by the
// four gates) or [V, 4*D] (emb_cols = 4*D). prev_c may be null (zero cell state).
__global__ void __launch_bounds__(kSpecThreads)
sum_lstm_kernel(const bf16* __restrict__ gates, long long ldg, const bf16* __restrict__ emb,
                int emb_cols, const long long* __restrict__ tok, float alpha,
                const bf16* __restrict__ prev_c, long long ldc, const bf16* __restrict__ w_cell,
                const bf16* __restrict__ b_cell, const bf16* __restrict__ w_state,
                const bf16* __restrict__ b_state, bf16* __restrict__ c_out,
                bf16* __restrict__ h_out, long long ldo, int D, float eps, int tanh_approx) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const bf16* e = emb + tok[row] * (long long)emb_cols;
  const bf16* g = gates + row * ldg;
  constexpr int kPer = kSpecMaxPerThread / 2;  // D <= 4096
  float pf[kPer], pi[kPer], po[kPer], pc[kPer];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int i = threadIdx.x + j * kSpecThreads;
    if (i < D) {
      const float e0 = ldf(e, i);
      const float ef = alpha * e0;
      const float ei = alpha * (emb_cols == D ? e0 : ldf(e, D + i));
      const float eo = alpha * (emb_cols == D ? e0 : ldf(e, 2 * D + i));
      const float ec = alpha * (emb_cols == D ? e0 : ldf(e, 3 * D + i));
      pf[j] = ldf(g, i) + ef;
      pi[j] = ldf(g, D + i) + ei;
      po[j] = ldf(g, 2 * D + i) + eo;
      pc[j] = ldf(g, 3 * D + i) + ec;
      ss += pc[j] * pc[j];
    } else {
      pf[j] = pi[j] = po[j] = pc[j] = 0.f;
    }
  }
  const float inv_c = rsqrtf(block_sum_256(ss, red) / (float)D + eps);
  float ss2 = 0.f;
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int i = threadIdx.x + j * kSpecThreads;
    if (i < D) {
      float n = pc[j] * inv_c;
      if (w_cell) n *= ldf(w_cell, i);
      if (b_cell) n += ldf(b_cell, i);
      const float cp = prev_c ? ldf(prev_c, row * ldc + i) : 0.f;
      const float c = cp * sigmoid_f(pf[j]) + gelu_f(n, tanh_approx) * sigmoid_f(pi[j]);
      // the cell state is stored in bf16; normalise what is stored
      const bf16 cb = __float2bfloat16(c);
      c_out[row * ldo + i] = cb;
      pc[j] = __bfloat162float(cb);
      ss2 += pc[j] * pc[j];
    }
  }
  const float inv_s = rsqrtf(block_sum_256(ss2, red) / (float)D + eps);
#pragma unroll
  for (int j = 0; j < kPer; ++j) {
    const int i = threadIdx.x + j * kSpecThreads;
    if (i < D) {
      float n = pc[j] * inv_s;
      if (w_state) n *= ldf(w_state, i);
      if (b_state) n += ldf(b_state, i);
      h_out[row * ldo + i] = __float2bfloat16(gelu_f(n, tanh_approx) * sigmoid_f(po[j]));
    }
  }
}

// ----------------------------------------------------------------------- verify_greedy
// Request r fed rows [row_start[r], row_start[r] + 1 + num_draft[r]): its last accepted token
// followed by its draft tokens. target[row] is the model's arg-max after that row.
// accepted[r]   = number of draft tokens that match
// next_tok[r]   = target at the first mismatch (the bonus token when everything matched)
// sel_row[r]    = row whose hidden state conditions the next draft
// out_tokens    = [R, max_draft + 1] accepted tokens then the bonus token, -1 padded
__global__ void verify_greedy_kernel(const long long* __restrict__ input_ids,
                                     const long long* __restrict__ target,
                                     const int* __restrict__ row_start,
                                     const int* __restrict__ num_draft, int R, int max_draft,
                                     int* __restrict__ accepted, long long* __restrict__ next_tok,
                                     long long* __restrict__ sel_row,
                                     long long* __restrict__ out_tokens) {
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  const int s = row_start[r];
  const int nd = num_draft[r];
  int a = 0;
  if (s >= 0) {
    while (a < nd && input_ids[s + a + 1] == target[s + a]) ++a;
  }
  accepted[r] = a;
  const long long nt = s >= 0 ? target[s + a] : 0;
  next_tok[r] = nt;
  sel_row[r] = s >= 0 ? s + a : 0;
  long long* o = out_tokens + (long long)r * (max_draft + 1);
  for (int j = 0; j <= max_draft; ++j) o[j] = (s >= 0 && j <= a) ? target[s + j] : -1;
}

}  // namespace ab200

using namespace ab200;

extern "C" {

int ab200_spec_ln(const void* x, long long ldx, const void* w, const void* b, void* y,
                  long long ldy, long long rows, int hidden, float eps, float out_scale,
                  cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (hidden > kSpecThreads * kSpecMaxPerThread) return -2;
  (void)launch_pdl(spec_ln_kernel, dim3((unsigned)rows), dim3(kSpecThreads), 0, stream, 
      reinterpret_cast<const bf16*>(x), ldx, reinterpret_cast<const bf16*>(w),
      reinterpret_cast<const bf16*>(b), reinterpret_cast<bf16*>(y), ldy, hidden, eps, out_scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_mlp_spec_step(const void* proj, long long ldp, const void* emb, const void* tok,
                        float emb_scale, const void* ln_w, const void* ln_b, void* out,
                        long long ldo, long long rows, int dim, float eps, int tanh_approx,
                        cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (dim > kSpecThreads * kSpecMaxPerThread) return -2;
  (void)launch_pdl(mlp_spec_step_kernel, dim3((unsigned)rows), dim3(kSpecThreads), 0, stream, 
      reinterpret_cast<const bf16*>(proj), ldp, reinterpret_cast<const bf16*>(emb),
      reinterpret_cast<const long long*>(tok), emb_scale, reinterpret_cast<const bf16*>(ln_w),
      reinterpret_cast<const bf16*>(ln_b), reinterpret_cast<bf16*>(out), ldo, dim, eps, tanh_approx);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_sum_lstm(const void* gates, long long ldg, const void* emb, int emb_cols,
                   const void* tok, float alpha, const void* prev_c, long long ldc,
                   const void* w_cell, const void* b_cell, const void* w_state,
                   const void* b_state, void* c_out, void* h_out, long long ldo, long long rows,
                   int D, float eps, int tanh_approx, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (D > kSpecThreads * kSpecMaxPerThread / 2 || (emb_cols != D && emb_cols != 4 * D)) return -2;
  (void)launch_pdl(sum_lstm_kernel, dim3((unsigned)rows), dim3(kSpecThreads), 0, stream, 
      reinterpret_cast<const bf16*>(gates), ldg, reinterpret_cast<const bf16*>(emb), emb_cols,
      reinterpret_cast<const long long*>(tok), alpha, reinterpret_cast<const bf16*>(prev_c), ldc,
      reinterpret_cast<const bf16*>(w_cell), reinterpret_cast<const bf16*>(b_cell),
      reinterpret_cast<const bf16*>(w_state), reinterpret_cast<const bf16*>(b_state),
      reinterpret_cast<bf16*>(c_out), reinterpret_cast<bf16*>(h_out), ldo, D, eps, tanh_approx);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int ab200_verify_greedy(const void* input_ids, const void* target, const void* row_start,
                        const void* num_draft, int R, int max_draft, void* accepted,
                        void* next_tok, void* sel_row, void* out_tokens, cudaStream_t stream) {
  if (R <= 0) return 0;
  (void)launch_pdl(verify_greedy_kernel, dim3((R + 127) / 128), dim3(128), 0, stream, 
      reinterpret_cast<const long long*>(input_ids), reinterpret_cast<const long long*>(target),
      reinterpret_cast<const int*>(row_start), reinterpret_cast<const int*>(num_draft), R,
      max_draft, reinterpret_cast<int*>(accepted), reinterpret_cast<long long*>(next_tok),
      reinterpret_cast<long long*>(sel_row), reinterpret_cast<long long*>(out_tokens));
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

}  // extern "C"
