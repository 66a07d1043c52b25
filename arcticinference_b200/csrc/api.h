// C entry points of the kernel library (all launch on the given stream and
// return 0 on success, a negative code when an argument is rejected or a launch
// fails). Pointers are device pointers unless stated otherwise. `status` is an
// int32[8] device buffer that kernels use to report bounded-wait timeouts and
// failed index checks instead of trapping; see common/ptx.cuh.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Cross-rank ordering of a kernel without a barrier launch (csrc/common/peer.cuh). All
// pointers are device pointers into the ranks' symmetric heaps, except the pointer array.
typedef struct Ab200PeerSync {
  // signal every rank when the kernel's last block has finished storing (sig_world = 0: off)
  const void* const* sig_flag_ptrs;  // host array: rank r's arrival words of the channel
  void* sig_done_ctr;                // this rank's block counter of the channel
  void* sig_epoch_ctr;               // this rank's epoch counter of the channel
  int sig_rank;
  int sig_world;
  // before reading its input, wait until every rank has signalled on this channel
  // (wait_world = 0: off)
  const void* wait_flags;            // this rank's arrival words of the channel
  const void* wait_epoch_ctr;        // this rank's epoch counter of the channel
  int wait_world;
} Ab200PeerSync;

typedef struct Ab200LinearDesc {
  const void* x; long long ldx; const void* sx;   // sx != null: e4m3 rows + fp32 scale per token
  const void* w; long long ldw; const void* sw;   // sw != null: e4m3 rows + fp32 scale per feature
  void* out; long long ldo;
  int M, N, K;
  const void* bias; const void* residual; long long ldr; int act;
  void* workspace; size_t workspace_bytes; int force_splits;
  const void* const* peer_ptrs; int world; int peer_cols; long long peer_row_off;  // scatter
  Ab200PeerSync sync;
  int* status;
  // fp8 weight stored in 16-row x 128-byte tiles, [N/16][K/128][16][128]: byte distance between
  // 16-row tiles and between k-tiles (both 0: row-major). `ldw` is ignored for a tiled weight.
  long long w_tile_stride_n;
  long long w_tile_stride_k;
  // 1: w is a parameter that no kernel of the stream writes; its first tiles may then be
  // requested before the kernel waits for the kernel launched before it
  int w_static;
} Ab200LinearDesc;

// ---- gemm_bf16.cu
int ab200_linear_desc(const Ab200LinearDesc* d, cudaStream_t stream);
size_t ab200_linear_bf16_workspace_bytes(int M, int N, int K);
int ab200_linear_bf16(const void* x, long long ldx, const void* w, long long ldw, void* out,
                      long long ldo, int M, int N, int K, const void* bias, const void* residual,
                      long long ldr, int act, void* workspace, size_t workspace_bytes,
                      int force_splits, int* status, cudaStream_t stream);
int ab200_gemm_bf16_nn(const void* x, long long ldx, const void* wt, long long ldw, void* out,
                       long long ldo, int M, int N, int K, int* status, cudaStream_t stream);

// ---- elementwise.cu
int ab200_embedding(const void* ids, const void* table, void* out, long long T, int hidden,
                    long long vocab, long long vocab_start, cudaStream_t stream);
int ab200_rmsnorm(const void* x, long long ldx, void* residual, const void* weight, void* y,
                  long long ldy, long long T, int hidden, float eps, cudaStream_t stream);
int ab200_layernorm(const void* x, const void* residual, const void* gamma, const void* beta,
                    void* y, long long T, int hidden, float eps, cudaStream_t stream);
int ab200_silu_mul(const void* x, void* out, long long T, int inter, int nblk,
                   cudaStream_t stream);
int ab200_rope_cache(void* qkv, long long ld, const void* positions, const void* slots,
                     const void* inv_freq, void* k_cache, void* v_cache, long long T, int Hq,
                     int Hkv, int D, int block_size, long long num_slots, int rotate_q, int* status,
                     cudaStream_t stream);
int ab200_gather_rows(const void* src, long long ld, const void* idx, void* dst, long long R,
                      int hidden, cudaStream_t stream);
// encoder.cu
int ab200_bert_embed_ln(const void* ids, const void* positions, const void* type_ids,
                        const void* word, const void* pos, const void* type, const void* gamma,
                        const void* beta, void* out, long long T, int hidden, long long vocab,
                        long long max_pos, long long n_types, float eps, int* status,
                        cudaStream_t stream);
int ab200_pool_normalize(const void* h, long long ld, const void* starts, void* out, int n_seqs,
                         int hidden, int mode, int normalize, cudaStream_t stream);
// kv_cache.cu
int ab200_kv_bulk_write(const void* kv, long long ld, const void* positions, const void* slots,
                        const void* inv_freq, const void* k_ptrs, const void* v_ptrs,
                        const void* k_scales, const void* v_scales, long long T, int L, int Hkv,
                        int D, int block_size, long long num_slots, int fp8, int* status,
                        cudaStream_t stream);
int ab200_kv_write_fp4(const void* k, long long ldk, const void* v, long long ldv,
                       const void* slots, void* k_codes, void* v_codes, void* k_scales,
                       void* v_scales, long long T, int Hkv, int D, int block_size,
                       long long num_slots, int* status, cudaStream_t stream);
int ab200_kv_read_fp4(const void* codes, const void* scales, const void* slots, void* out,
                      long long ldo, long long R, int Hkv, int D, int block_size,
                      cudaStream_t stream);
int ab200_patch_ids(void* ids, const void* src_rows, const void* prev_ids, long long n,
                    long long n_prev, cudaStream_t stream);
int ab200_argmax_sample(const void* logits, int dtype, long long ld, long long B, int V,
                        const void* temperature, const void* seeds, void* out_ids, void* out_vals,
                        long long index_offset, cudaStream_t stream);

// ---- attention.cu
int ab200_attention(const void* q, long long ldq, const void* k, const void* v, long long ld_kv,
                    long long num_blocks, int block_size, const void* block_tables, int max_blocks,
                    const void* work, int num_work, const void* tok_splits, int max_splits,
                    long long T, int Hq, int Hkv, int D, int causal, float scale, void* out,
                    long long ldo, void* o_part, void* lse_part, void* lse_out, int tile_keys,
                    int* status, cudaStream_t stream);
int ab200_attention_scatter(const void* q, long long ldq, const void* k, const void* v,
                            long long num_blocks, int block_size, const void* block_tables,
                            int max_blocks, const void* work, int num_work,
                            const void* tok_splits, int max_splits, long long T, int Hq, int Hkv,
                            int D, float scale, const void* const* peer_ptrs, int world,
                            int peer_tokens, long long ldo, void* o_part, void* lse_part,
                            int tile_keys, int* status, cudaStream_t stream);
int ab200_linear_bf16_scatter(const void* x, long long ldx, const void* w, long long ldw,
                              const void* const* peer_ptrs, int world, int peer_cols,
                              long long peer_row_off, long long ldo, int M, int N, int K,
                              int* status, cudaStream_t stream);

// ---- gemm_bf16.cu, fp8 operands with per-token / per-feature scales
int ab200_linear_fp8_row(const void* xq, long long ldx, const void* sx, const void* wq,
                         long long ldw, const void* sw, void* out, long long ldo, int M, int N,
                         int K, const void* bias, const void* residual, long long ldr, int act,
                         void* workspace, size_t workspace_bytes, int force_splits,
                         const void* const* peer_ptrs, int world, int peer_cols,
                         long long peer_row_off, int* status, cudaStream_t stream);

// ---- quant_row.cu
int ab200_quant_fp8_row(const void* x, long long ldx, void* xq, long long ldq, void* sx,
                        long long M, int K, cudaStream_t stream);
int ab200_rmsnorm_quant(const void* x, long long ldx, void* residual, const void* weight,
                        void* yq, long long ldq, void* sy, void* y, long long ldy, long long T,
                        int hidden, float eps, cudaStream_t stream);
int ab200_silu_mul_quant(const void* x, void* outq, long long ldq, void* so, long long T,
                         int inter, int nblk, cudaStream_t stream);

// ---- gemm_fp8.cu
int ab200_quant_fp8(const void* x, long long ldx, void* xq, long long ldq, void* sx_t,
                    long long ld_sx, long long M, int K, cudaStream_t stream);
int ab200_dequant_fp8(const void* wq, long long ldw, const void* sw, long long ld_sw, void* out,
                      long long ldo, long long N, int K, cudaStream_t stream);
int ab200_linear_w8a16(const void* x, long long ldx, const void* wq, long long ldw, const void* sw,
                       long long ld_sw, void* out, long long ldo, int M, int N, int K,
                       void* workspace, size_t workspace_bytes, int force_splits,
                       const void* const* peer_ptrs, int world, int peer_cols,
                       long long peer_row_off, int* status, cudaStream_t stream);
size_t ab200_linear_fp8_workspace_bytes(int M, int N, int K);
int ab200_linear_fp8(const void* xq, long long ldxq, const void* sx_t, long long ld_sx,
                     const void* wq, long long ldw, const void* sw, long long ld_sw, void* out,
                     long long ldo, int M, int N, int K, void* workspace, size_t workspace_bytes,
                     int force_splits, const void* const* peer_ptrs, int world, int peer_cols,
                     long long peer_row_off, int* status, cudaStream_t stream);

// ---- speculator.cu
int ab200_spec_ln(const void* x, long long ldx, const void* w, const void* b, void* y,
                  long long ldy, long long rows, int hidden, float eps, float out_scale,
                  cudaStream_t stream);
int ab200_mlp_spec_step(const void* proj, long long ldp, const void* emb, const void* tok,
                        float emb_scale, const void* ln_w, const void* ln_b, void* out,
                        long long ldo, long long rows, int dim, float eps, int tanh_approx,
                        cudaStream_t stream);
int ab200_sum_lstm(const void* gates, long long ldg, const void* emb, int emb_cols,
                   const void* tok, float alpha, const void* prev_c, long long ldc,
                   const void* w_cell, const void* b_cell, const void* w_state,
                   const void* b_state, void* c_out, void* h_out, long long ldo, long long rows,
                   int D, float eps, int tanh_approx, cudaStream_t stream);
int ab200_verify_greedy(const void* input_ids, const void* target, const void* row_start,
                        const void* num_draft, int R, int max_draft, void* accepted,
                        void* next_tok, void* sel_row, void* out_tokens, cudaStream_t stream);

// ---- comm.cu (pointer arrays are host arrays of `world` device pointers)
int ab200_barrier(const void* const* flag_ptrs, int my_rank, int world, void* epoch_ctr,
                  int* status, cudaStream_t stream);
int ab200_barrier_timed(const void* const* flag_ptrs, int my_rank, int world, void* epoch_ctr,
                        int limit_ms, int* status, cudaStream_t stream);
int ab200_allreduce(const void* const* part_ptrs, int world, void* out, const void* residual,
                    long long n_elems, cudaStream_t stream);
// Two-shot all-reduce in one launch (reduce-scatter by peer loads, all-gather by peer stores,
// flag exchanges inside the kernel); the result lands in every rank's result buffer.
long long ab200_allreduce2_flag_bytes();
int ab200_allreduce2(const void* const* part_ptrs, const void* const* res_ptrs,
                     const void* const* flag_ptrs, void* epochs, int my_rank, int world,
                     long long n_elems, int* status, cudaStream_t stream);
// ---- variants with cross-rank ordering built in (see Ab200PeerSync)
int ab200_attention_scatter_sync(const void* q, long long ldq, const void* k, const void* v,
                                 long long num_blocks, int block_size, const void* block_tables,
                                 int max_blocks, const void* work, int num_work,
                                 const void* tok_splits, int max_splits, long long T, int Hq,
                                 int Hkv, int D, float scale, const void* const* peer_ptrs,
                                 int world, int peer_tokens, long long ldo, void* o_part,
                                 void* lse_part, int tile_keys, const Ab200PeerSync* sync,
                                 int* status, cudaStream_t stream);
int ab200_rope_cache_wait(void* qkv, long long ld, const void* positions, const void* slots,
                          const void* inv_freq, void* k_cache, void* v_cache, long long T, int Hq,
                          int Hkv, int D, int block_size, long long num_slots, int rotate_q,
                          const Ab200PeerSync* sync, int* status, cudaStream_t stream);
// ---- sampling.cu: y = x / temperature restricted to the top-k / top-p set, -inf elsewhere
int ab200_topk_topp_mask(const void* logits, long long ld_in, void* out, long long ld_out, int B,
                         int V, const void* temperature, const void* top_k, const void* top_p,
                         cudaStream_t stream);
// ---- qk_norm.cu: in-place RMSNorm over head_dim of the Hq query and Hkv key heads of every row
int ab200_qk_norm(void* qkv, long long ld, const void* wq, const void* wk, long long T, int Hq,
                  int Hkv, int D, float eps, const Ab200PeerSync* sync, int* status,
                  cudaStream_t stream);
int ab200_quant_fp8_row_wait(const void* x, long long ldx, void* xq, long long ldq, void* sx,
                             long long M, int K, const Ab200PeerSync* sync, int* status,
                             cudaStream_t stream);

// ---- comm_fused.cu
int ab200_push_rows(const void* src_a, long long ld_a, const void* src_b, long long ld_b,
                    long long rows_per_rank, int my_rank, int world, const void* idx,
                    const void* const* dst_a, const void* const* dst_b, long long R, int hidden,
                    cudaStream_t stream);
int ab200_rmsnorm_allgather(const void* x, long long ldx, void* residual, const void* weight,
                            const void* const* dst, long long row_off, int my_rank, int world,
                            long long T, int hidden, float eps, cudaStream_t stream);
int ab200_reduce_rmsnorm(const void* const* part_ptrs, int world, long long ld_part, void* residual,
                         const void* weight, void* y, long long ldy, void* yq, long long ldq,
                         void* sy, void* h_out, long long ldh, long long rows, int hidden,
                         float eps, const Ab200PeerSync* sync, int* status, cudaStream_t stream);
size_t ab200_argmax_exchange_slot_bytes(int world, int max_rows);
int ab200_argmax_exchange(const void* ids, const void* vals, int B, int max_rows,
                          const void* const* slot_ptrs, const void* const* flag_ptrs, int my_rank,
                          int world, void* epoch_ctr, void* out_ids, void* out_vals, int* status,
                          cudaStream_t stream);

#ifdef __cplusplus
}
#endif
