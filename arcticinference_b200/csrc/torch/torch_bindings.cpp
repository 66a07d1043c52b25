// torch.ops.arcticinference_b200.* : the kernels of _kernels.so as dispatcher ops, for users
// who compose them with other PyTorch code (autograd-free, CUDA only). The engine itself calls
// the C entry points directly (ops/native.py); both routes reach the same kernels.
//
// The reference registers its four kernels the same way
// (csrc/custom_ops/torch_bindings.cpp:6-51): reshape_and_cache_flash_bulk,
// reshape_and_cache_flash_fp4, speculator_ln, sum_lstm. Their counterparts here are
// kv_bulk_write, kv_write_fp4, spec_ln and sum_lstm; linear, rmsnorm, silu_mul, mlp_spec_step,
// the per-token fp8 quantisers (stand-alone, fused with RMSNorm, fused with SiLU*mul), the
// fp8 linear with per-token / per-feature scales, RoPE + paged cache write and paged
// attention are offered in addition.

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include "../api.h"

namespace {

cudaStream_t stream_of(const at::Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()); }

const void* opt_ptr(const c10::optional<at::Tensor>& t) {
  return t.has_value() && t->defined() ? t->data_ptr() : nullptr;
}

void check(int rc, const char* what) {
  TORCH_CHECK(rc == 0, "arcticinference_b200::", what, " failed with code ", rc);
}

void check_bf16_2d(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.stride(1) == 1,
              name, " must be a CUDA bf16 matrix with unit inner stride");
}

at::Tensor status_buffer(const at::Tensor& like) {
  static std::vector<at::Tensor> bufs(64);
  const int dev = like.get_device();
  if (!bufs[dev].defined())
    bufs[dev] = at::zeros({8}, at::TensorOptions().dtype(at::kInt).device(like.device()));
  return bufs[dev];
}

at::Tensor workspace(const at::Tensor& like) {
  static std::vector<at::Tensor> bufs(64);
  const int dev = like.get_device();
  if (!bufs[dev].defined())
    bufs[dev] = at::empty({96ll << 20}, at::TensorOptions().dtype(at::kByte).device(like.device()));
  return bufs[dev];
}

// out = act(x @ w^T + bias) + residual
at::Tensor linear(const at::Tensor& x, const at::Tensor& w, const c10::optional<at::Tensor>& bias,
                  const c10::optional<at::Tensor>& residual, int64_t act) {
  check_bf16_2d(x, "x");
  check_bf16_2d(w, "w");
  TORCH_CHECK(x.size(1) == w.size(1), "inner dimensions differ");
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor out = at::empty({x.size(0), w.size(0)}, x.options());
  if (x.size(0) == 0) return out;
  at::Tensor ws = workspace(x), st = status_buffer(x);
  const long long ldr = residual.has_value() && residual->defined() ? residual->stride(0) : 0;
  check(ab200_linear_bf16(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(),
                          out.stride(0), (int)x.size(0), (int)w.size(0), (int)x.size(1),
                          opt_ptr(bias), opt_ptr(residual), ldr, (int)act, ws.data_ptr(),
                          (size_t)ws.numel(), 0, st.data_ptr<int>(), stream_of(x)),
        "linear");
  return out;
}

// y = rmsnorm(x (+ residual)); residual is updated in place with x + residual
at::Tensor rmsnorm(const at::Tensor& x, const at::Tensor& weight, double eps,
                   const c10::optional<at::Tensor>& residual) {
  check_bf16_2d(x, "x");
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty({x.size(0), x.size(1)}, x.options());
  void* res = residual.has_value() && residual->defined() ? residual->data_ptr() : nullptr;
  check(ab200_rmsnorm(x.data_ptr(), x.stride(0), res, weight.data_ptr(), y.data_ptr(), y.stride(0),
                      x.size(0), (int)x.size(1), (float)eps, stream_of(x)),
        "rmsnorm");
  return y;
}

// x: [T, nblk * 2 * I] blocks of (gate | up) -> [T, nblk * I]
at::Tensor silu_mul(const at::Tensor& x, int64_t nblk) {
  check_bf16_2d(x, "x");
  TORCH_CHECK(x.is_contiguous() && nblk >= 1 && x.size(1) % (2 * nblk) == 0, "bad shape");
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t inter = x.size(1) / (2 * nblk);
  at::Tensor out = at::empty({x.size(0), nblk * inter}, x.options());
  check(ab200_silu_mul(x.data_ptr(), out.data_ptr(), x.size(0), (int)inter, (int)nblk, stream_of(x)),
        "silu_mul");
  return out;
}

at::Tensor spec_ln(const at::Tensor& x, const c10::optional<at::Tensor>& weight,
                   const c10::optional<at::Tensor>& bias, double eps, double out_scale) {
  check_bf16_2d(x, "x");
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty({x.size(0), x.size(1)}, x.options());
  check(ab200_spec_ln(x.data_ptr(), x.stride(0), opt_ptr(weight), opt_ptr(bias), y.data_ptr(),
                      y.stride(0), x.size(0), (int)x.size(1), (float)eps, (float)out_scale,
                      stream_of(x)),
        "spec_ln");
  return y;
}

at::Tensor mlp_spec_step(const at::Tensor& proj, const at::Tensor& emb, const at::Tensor& tok,
                         double emb_scale, const at::Tensor& ln_w,
                         const c10::optional<at::Tensor>& ln_b, double eps, bool tanh_approx) {
  check_bf16_2d(proj, "proj");
  TORCH_CHECK(tok.scalar_type() == at::kLong && tok.is_contiguous(), "tok must be int64");
  const c10::cuda::CUDAGuard guard(proj.device());
  at::Tensor out = at::empty({proj.size(0), proj.size(1)}, proj.options());
  check(ab200_mlp_spec_step(proj.data_ptr(), proj.stride(0), emb.data_ptr(), tok.data_ptr(),
                            (float)emb_scale, ln_w.data_ptr(), opt_ptr(ln_b), out.data_ptr(),
                            out.stride(0), proj.size(0), (int)proj.size(1), (float)eps,
                            tanh_approx ? 1 : 0, stream_of(proj)),
        "mlp_spec_step");
  return out;
}

// gates [B, 4D] (f, i, o, c) + alpha * emb[tok] (emb has D or 4D columns) -> (c_new, state)
std::tuple<at::Tensor, at::Tensor> sum_lstm(
    const at::Tensor& gates, const at::Tensor& emb, const at::Tensor& tok, double alpha,
    const c10::optional<at::Tensor>& prev_c, const at::Tensor& w_cell,
    const c10::optional<at::Tensor>& b_cell, const at::Tensor& w_state,
    const c10::optional<at::Tensor>& b_state, double eps, bool tanh_approx) {
  check_bf16_2d(gates, "gates");
  TORCH_CHECK(gates.size(1) % 4 == 0, "gates must have 4*D columns");
  TORCH_CHECK(tok.scalar_type() == at::kLong && tok.is_contiguous(), "tok must be int64");
  const c10::cuda::CUDAGuard guard(gates.device());
  const int64_t D = gates.size(1) / 4;
  at::Tensor c = at::empty({gates.size(0), D}, gates.options());
  at::Tensor h = at::empty({gates.size(0), D}, gates.options());
  const bool has_c = prev_c.has_value() && prev_c->defined();
  check(ab200_sum_lstm(gates.data_ptr(), gates.stride(0), emb.data_ptr(), (int)emb.size(1),
                       tok.data_ptr(), (float)alpha, has_c ? prev_c->data_ptr() : nullptr,
                       has_c ? prev_c->stride(0) : 0, w_cell.data_ptr(), opt_ptr(b_cell),
                       w_state.data_ptr(), opt_ptr(b_state), c.data_ptr(), h.data_ptr(), D,
                       gates.size(0), (int)D, (float)eps, tanh_approx ? 1 : 0, stream_of(gates)),
        "sum_lstm");
  return {c, h};
}

// K/V of L layers at once: kv [T, L*2*Hkv*D]; caches given by device pointer tables (int64 [L])
void kv_bulk_write(const at::Tensor& kv, const at::Tensor& positions, const at::Tensor& slots,
                   const at::Tensor& inv_freq, const at::Tensor& k_ptrs, const at::Tensor& v_ptrs,
                   const c10::optional<at::Tensor>& k_scales,
                   const c10::optional<at::Tensor>& v_scales, int64_t Hkv, int64_t D,
                   int64_t block_size, int64_t num_slots, bool fp8) {
  check_bf16_2d(kv, "kv");
  const c10::cuda::CUDAGuard guard(kv.device());
  at::Tensor st = status_buffer(kv);
  check(ab200_kv_bulk_write(kv.data_ptr(), kv.stride(0), positions.data_ptr(), slots.data_ptr(),
                            inv_freq.data_ptr(), k_ptrs.data_ptr(), v_ptrs.data_ptr(),
                            opt_ptr(k_scales), opt_ptr(v_scales), kv.size(0), (int)k_ptrs.numel(),
                            (int)Hkv, (int)D, (int)block_size, num_slots, fp8 ? 1 : 0,
                            st.data_ptr<int>(), stream_of(kv)),
        "kv_bulk_write");
}

void kv_write_fp4(const at::Tensor& k, const at::Tensor& v, const at::Tensor& slots,
                  at::Tensor k_codes, at::Tensor v_codes, at::Tensor k_scales, at::Tensor v_scales) {
  check_bf16_2d(k, "k");
  check_bf16_2d(v, "v");
  TORCH_CHECK(k_codes.dim() == 4, "codes must be [num_blocks, Hkv, block_size, D/2]");
  const c10::cuda::CUDAGuard guard(k.device());
  const int Hkv = (int)k_codes.size(1), bs = (int)k_codes.size(2), D = (int)k_codes.size(3) * 2;
  at::Tensor st = status_buffer(k);
  check(ab200_kv_write_fp4(k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), slots.data_ptr(),
                           k_codes.data_ptr(), v_codes.data_ptr(), k_scales.data_ptr(),
                           v_scales.data_ptr(), k.size(0), Hkv, D, bs, k_codes.size(0) * bs,
                           st.data_ptr<int>(), stream_of(k)),
        "kv_write_fp4");
}

at::Tensor fp8_like(const at::Tensor& x, int64_t rows, int64_t cols) {
  return at::empty({rows, cols}, x.options().dtype(at::kFloat8_e4m3fn));
}

// x bf16 [M, K] -> (e4m3 codes [M, K], fp32 scale per row)
std::tuple<at::Tensor, at::Tensor> quant_fp8_row(const at::Tensor& x) {
  check_bf16_2d(x, "x");
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor q = fp8_like(x, x.size(0), x.size(1));
  at::Tensor s = at::empty({x.size(0)}, x.options().dtype(at::kFloat));
  check(ab200_quant_fp8_row(x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0), s.data_ptr(),
                            x.size(0), (int)x.size(1), stream_of(x)),
        "quant_fp8_row");
  return {q, s};
}

// RMSNorm(x (+ residual, updated in place)) -> (e4m3 codes, fp32 scale per row)
std::tuple<at::Tensor, at::Tensor> rmsnorm_quant(const at::Tensor& x, const at::Tensor& weight,
                                                 double eps,
                                                 const c10::optional<at::Tensor>& residual) {
  check_bf16_2d(x, "x");
  const c10::cuda::CUDAGuard guard(x.device());
  at::Tensor q = fp8_like(x, x.size(0), x.size(1));
  at::Tensor s = at::empty({x.size(0)}, x.options().dtype(at::kFloat));
  void* res = residual.has_value() && residual->defined() ? residual->data_ptr() : nullptr;
  check(ab200_rmsnorm_quant(x.data_ptr(), x.stride(0), res, weight.data_ptr(), q.data_ptr(),
                            q.stride(0), s.data_ptr(), nullptr, 0, x.size(0), (int)x.size(1),
                            (float)eps, stream_of(x)),
        "rmsnorm_quant");
  return {q, s};
}

// x = nblk fused (gate | up) blocks -> (e4m3 codes of SiLU(gate) * up, fp32 scale per row)
std::tuple<at::Tensor, at::Tensor> silu_mul_quant(const at::Tensor& x, int64_t nblk) {
  check_bf16_2d(x, "x");
  TORCH_CHECK(x.is_contiguous() && nblk >= 1 && x.size(1) % (2 * nblk) == 0, "bad gate/up layout");
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t inter = x.size(1) / (2 * nblk);
  at::Tensor q = fp8_like(x, x.size(0), nblk * inter);
  at::Tensor s = at::empty({x.size(0)}, x.options().dtype(at::kFloat));
  check(ab200_silu_mul_quant(x.data_ptr(), q.data_ptr(), q.stride(0), s.data_ptr(), x.size(0),
                             (int)inter, (int)nblk, stream_of(x)),
        "silu_mul_quant");
  return {q, s};
}

// out[m, n] = sx[m] * sw[n] * sum_k xq[m, k] * wq[n, k]  (+ bias)(activation)(+ residual)
at::Tensor linear_fp8_row(const at::Tensor& xq, const at::Tensor& sx, const at::Tensor& wq,
                          const at::Tensor& sw, const c10::optional<at::Tensor>& bias,
                          const c10::optional<at::Tensor>& residual, int64_t act) {
  TORCH_CHECK(xq.is_cuda() && xq.dim() == 2 && wq.dim() == 2 && xq.element_size() == 1 &&
                  wq.element_size() == 1 && xq.stride(1) == 1 && wq.stride(1) == 1,
              "xq and wq must be CUDA e4m3 matrices with unit inner stride");
  TORCH_CHECK(xq.size(1) == wq.size(1), "inner dimensions differ");
  TORCH_CHECK(sx.scalar_type() == at::kFloat && sw.scalar_type() == at::kFloat &&
                  sx.numel() == xq.size(0) && sw.numel() == wq.size(0),
              "scales must be fp32, one per row of xq and of wq");
  const c10::cuda::CUDAGuard guard(xq.device());
  at::Tensor out = at::empty({xq.size(0), wq.size(0)}, xq.options().dtype(at::kBFloat16));
  if (xq.size(0) == 0) return out;
  at::Tensor ws = workspace(xq), st = status_buffer(xq);
  const long long ldr = residual.has_value() && residual->defined() ? residual->stride(0) : 0;
  check(ab200_linear_fp8_row(xq.data_ptr(), xq.stride(0), sx.data_ptr(), wq.data_ptr(),
                             wq.stride(0), sw.data_ptr(), out.data_ptr(), out.stride(0),
                             (int)xq.size(0), (int)wq.size(0), (int)xq.size(1), opt_ptr(bias),
                             opt_ptr(residual), ldr, (int)act, ws.data_ptr(), (size_t)ws.numel(), 0,
                             nullptr, 0, 0, 0, st.data_ptr<int>(), stream_of(xq)),
        "linear_fp8_row");
  return out;
}

// Rotates q and k of qkv [T, (Hq + 2 Hkv) D] in place and writes k, v into the paged caches
// [num_blocks, Hkv, block_size, D] at `slots` (slots < 0 are skipped).
void rope_cache(at::Tensor qkv, const at::Tensor& positions, const at::Tensor& slots,
                const at::Tensor& inv_freq, at::Tensor k_cache, at::Tensor v_cache, int64_t Hq,
                int64_t Hkv, int64_t D) {
  check_bf16_2d(qkv, "qkv");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous(),
              "caches must be contiguous [num_blocks, Hkv, block_size, D]");
  const c10::cuda::CUDAGuard guard(qkv.device());
  at::Tensor st = status_buffer(qkv);
  const int64_t bs = k_cache.size(2);
  check(ab200_rope_cache(qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), slots.data_ptr(),
                         inv_freq.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), qkv.size(0),
                         (int)Hq, (int)Hkv, (int)D, (int)bs, k_cache.size(0) * bs, 1,
                         st.data_ptr<int>(), stream_of(qkv)),
        "rope_cache");
}

// Paged attention over a host-planned work list (ops.plan_attention_work): q [T, Hq D],
// caches [num_blocks, Hkv, block_size, D], block_tables int32 [num_seqs, max_blocks],
// work int32 [n, 8], tok_splits int32 [T]. Returns [T, Hq D].
at::Tensor attention(const at::Tensor& q, const at::Tensor& k_cache, const at::Tensor& v_cache,
                     const at::Tensor& block_tables, const at::Tensor& work,
                     const at::Tensor& tok_splits, int64_t max_splits, int64_t Hq, int64_t Hkv,
                     int64_t D, bool causal, double scale, int64_t tile_keys) {
  check_bf16_2d(q, "q");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.is_contiguous() && v_cache.is_contiguous(),
              "caches must be contiguous [num_blocks, Hkv, block_size, D]");
  TORCH_CHECK(block_tables.scalar_type() == at::kInt && block_tables.is_contiguous() &&
                  work.scalar_type() == at::kInt && work.is_contiguous() && work.size(1) == 8 &&
                  tok_splits.scalar_type() == at::kInt,
              "block_tables, work and tok_splits must be contiguous int32");
  const c10::cuda::CUDAGuard guard(q.device());
  const int64_t T = q.size(0);
  at::Tensor out = at::empty({T, Hq * D}, q.options());
  at::Tensor o_part, lse_part;
  if (max_splits > 1) {
    o_part = at::empty({max_splits, T, Hq, D}, q.options().dtype(at::kFloat));
    lse_part = at::empty({max_splits, T, Hq}, q.options().dtype(at::kFloat));
  }
  at::Tensor st = status_buffer(q);
  check(ab200_attention(q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), 0,
                        k_cache.size(0), (int)k_cache.size(2), block_tables.data_ptr(),
                        (int)block_tables.size(1), work.data_ptr(), (int)work.size(0),
                        tok_splits.data_ptr(), (int)max_splits, T, (int)Hq, (int)Hkv, (int)D,
                        causal ? 1 : 0, (float)scale, out.data_ptr(), out.stride(0),
                        max_splits > 1 ? o_part.data_ptr() : nullptr,
                        max_splits > 1 ? lse_part.data_ptr() : nullptr, nullptr, (int)tile_keys,
                        st.data_ptr<int>(), stream_of(q)),
        "attention");
  return out;
}

}  // namespace

TORCH_LIBRARY(arcticinference_b200, m) {
  m.def("linear(Tensor x, Tensor w, Tensor? bias=None, Tensor? residual=None, int act=0) -> Tensor");
  m.def("rmsnorm(Tensor x, Tensor weight, float eps, Tensor(a!)? residual=None) -> Tensor");
  m.def("silu_mul(Tensor x, int nblk=1) -> Tensor");
  m.def("spec_ln(Tensor x, Tensor? weight, Tensor? bias, float eps, float out_scale=1.0) -> Tensor");
  m.def("mlp_spec_step(Tensor proj, Tensor emb, Tensor tok, float emb_scale, Tensor ln_w, "
        "Tensor? ln_b, float eps, bool tanh_approx=False) -> Tensor");
  m.def("sum_lstm(Tensor gates, Tensor emb, Tensor tok, float alpha, Tensor? prev_c, Tensor w_cell, "
        "Tensor? b_cell, Tensor w_state, Tensor? b_state, float eps, bool tanh_approx=False) "
        "-> (Tensor, Tensor)");
  m.def("kv_bulk_write(Tensor kv, Tensor positions, Tensor slots, Tensor inv_freq, Tensor k_ptrs, "
        "Tensor v_ptrs, Tensor? k_scales, Tensor? v_scales, int Hkv, int D, int block_size, "
        "int num_slots, bool fp8=False) -> ()");
  m.def("kv_write_fp4(Tensor k, Tensor v, Tensor slots, Tensor(a!) k_codes, Tensor(b!) v_codes, "
        "Tensor(c!) k_scales, Tensor(d!) v_scales) -> ()");
  m.def("quant_fp8_row(Tensor x) -> (Tensor, Tensor)");
  m.def("rmsnorm_quant(Tensor x, Tensor weight, float eps, Tensor(a!)? residual=None) "
        "-> (Tensor, Tensor)");
  m.def("silu_mul_quant(Tensor x, int nblk=1) -> (Tensor, Tensor)");
  m.def("linear_fp8_row(Tensor xq, Tensor sx, Tensor wq, Tensor sw, Tensor? bias=None, "
        "Tensor? residual=None, int act=0) -> Tensor");
  m.def("rope_cache(Tensor(a!) qkv, Tensor positions, Tensor slots, Tensor inv_freq, "
        "Tensor(b!) k_cache, Tensor(c!) v_cache, int Hq, int Hkv, int D) -> ()");
  m.def("attention(Tensor q, Tensor k_cache, Tensor v_cache, Tensor block_tables, Tensor work, "
        "Tensor tok_splits, int max_splits, int Hq, int Hkv, int D, bool causal, float scale, "
        "int tile_keys=128) -> Tensor");
}

TORCH_LIBRARY_IMPL(arcticinference_b200, CUDA, m) {
  m.impl("linear", &linear);
  m.impl("rmsnorm", &rmsnorm);
  m.impl("silu_mul", &silu_mul);
  m.impl("spec_ln", &spec_ln);
  m.impl("mlp_spec_step", &mlp_spec_step);
  m.impl("sum_lstm", &sum_lstm);
  m.impl("kv_bulk_write", &kv_bulk_write);
  m.impl("kv_write_fp4", &kv_write_fp4);
  m.impl("quant_fp8_row", &quant_fp8_row);
  m.impl("rmsnorm_quant", &rmsnorm_quant);
  m.impl("silu_mul_quant", &silu_mul_quant);
  m.impl("linear_fp8_row", &linear_fp8_row);
  m.impl("rope_cache", &rope_cache);
  m.impl("attention", &attention);
}
