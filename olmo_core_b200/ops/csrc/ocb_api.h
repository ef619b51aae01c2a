// C entry points of the sm_100a kernel library. Every launcher is asynchronous on `stream`, returns 0
// on success and a negative value on a host-side failure (bad argument / launch error). Kernels that
// can wait on the device additionally report through an `int* status` device word (see common.cuh).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// dtype codes for activation tensors
#define OCB_BF16 0
#define OCB_F32 1

// ---- GEMM (gemm_sm100.cu) ---------------------------------------------------------------------------
// epilogue: 0 = bf16 store, 1 = fp32 accumulate (C += AB), 2 = fp32 store, 3 = bf16 accumulate.
int ocb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb,
                  long long ldc, int a_mn_major, int b_mn_major, int epilogue, int* status, cudaStream_t stream);

// Grouped GEMM over rows sorted by group; offsets: int32 [num_groups + 1] device array of row prefix sums.
// mode 1: C[r, :N] = A[r, :K] * op(B_g) for the rows r of group g (B: groups stacked along the outer dimension).
// mode 2: C_g[M, N] (=|+=) A[rows of g, :M]^T * B[rows of g, :N] (both operands MN-major; C: [G*M, N]).
int ocb_grouped_gemm_bf16(const void* A, const void* B, void* C, const int* offsets, int num_groups, int mode,
                          int total_rows, int M, int N, int K, long long lda, long long ldb, long long ldc, int b_mn_major,
                          int epilogue, int* status, cudaStream_t stream);

// Tensor-parallel GEMMs with the collective inside the kernel (m_local % 128 == 0, world <= 8):
// gather_a: C[world*m_local, N] = [A_0; ...; A_{world-1}] * op(B), A_r read from a_ptrs[r] (peer memory) tile by tile.
// scatter_c: rows of rank r of A * op(B) are added into c_ptrs[r] (fp32 [m_local, N]) with reductions over NVLink.
int ocb_gemm_bf16_tp(const void* const* a_ptrs, const void* B, void* const* c_ptrs, int m_local, int N, int K,
                     long long lda, long long ldb, long long ldc, int world, int rank, int gather_a, int scatter_c,
                     int b_mn_major, int epilogue, int* status, cudaStream_t stream);

// ---- 8-bit floating point (gemm_sm100.cu, fp8_sm100.cu) -----------------------------------------------
// C[M, N] = (A_q * B_q^T) .* (scale_a[m] * scale_b[n]); A_q [M, K], B_q [N, K] e4m3 bytes, K-major.
// epilogue: 0 = bf16 store, 1 = fp32 accumulate, 2 = fp32 store.
int ocb_gemm_fp8(const void* A, const void* B, void* C, const float* scale_a, const float* scale_b, int M, int N, int K,
                 long long lda, long long ldb, long long ldc, int epilogue, int* status, cudaStream_t stream);
// q[r, :] = e4m3(x[r, :] / scale[r]), scale[r] = amax(x[r, :]) / 448   (x bf16, cols % 8 == 0)
// pow2 != 0 rounds every scale up to a power of two.
int ocb_quantize_e4m3_rowwise(const void* x, void* q, float* scale, int rows, int cols, long long ldx, long long ldq,
                              int pow2, cudaStream_t stream);
// q_t[c, :] = e4m3(x[:, c] / scale[c]): the transposed operand, scaled per column of x. scratch: fp32 [cols].
int ocb_quantize_e4m3_colwise_t(const void* x, void* q_t, float* scale, float* scratch, int rows, int cols, long long ldx,
                                long long ldq, int pow2, cudaStream_t stream);

// ---- mixture of experts (moe_sm100.cu) --------------------------------------------------------------
// scores = softmax (mode 0) or sigmoid (mode 1) of logits [n_tokens, n_experts]; weights / experts: [n_tokens, top_k];
// counts: int32 [n_experts] tokens per expert (may be null); scores may be null.
int ocb_moe_router_topk(const void* logits, float* scores, float* weights, int* experts, int* counts, int n_tokens,
                        int n_experts, int top_k, int mode, int normalize, long long ld, int act_dtype,
                        cudaStream_t stream);
// Stable counting sort of n routed copies by expert id. dest[j]: row of copy j in the sorted layout; src: its inverse;
// sorted_experts (may be null): expert of every row; offsets: int32 [n_experts + 1] prefix sums.
long long ocb_moe_sort_scratch_ints(int n, int n_experts);
int ocb_moe_sort(const int* experts, int* dest, int* src, int* sorted_experts, int* offsets, int* scratch, int n,
                 int n_experts, cudaStream_t stream);
// out[r] = (w[src[r]] *) x[src[r] / top_k]   (bf16 rows, cols % 8 == 0; w fp32 or null)
int ocb_moe_gather(const void* x, const int* src, const float* w, void* out, int n_rows, int cols, int top_k,
                   long long ldx, long long ldo, cudaStream_t stream);
// y[t] = sum_j w[t*top_k + j] * ys[dest[t*top_k + j]]   (fp32 accumulation in a fixed order)
int ocb_moe_scatter(const void* ys, const int* dest, const float* w, void* y, int n_tokens, int cols, int top_k,
                    long long lds, long long ldy, cudaStream_t stream);
// dw[j] = <ys[dest[j]], dy[j / top_k]>
int ocb_moe_rowdot(const void* ys, const int* dest, const void* dy, float* dw, int n_copies, int cols, int top_k,
                   long long lds, long long ldd, cudaStream_t stream);
// Expert-parallel exchange over peer memory (moe_peer_sm100.cu): segment s moves rows [src_start[s], +count[s]) of src
// (row i read from gather_idx[i] / gather_div when gather_idx is given) to rows dst_start[s]... of rank dst_rank[s]'s
// buffer peer_ptrs[dst_rank[s]]. Rows that would land beyond dst_capacity_rows are skipped and reported in *status.
int ocb_moe_push_rows(const void* src, const int* gather_idx, int gather_div, const int* seg_src_start,
                      const int* seg_count, const int* seg_dst_rank, const long long* seg_dst_start, int num_segments,
                      void* const* peer_ptrs, int world, long long dst_capacity_rows, int cols, long long ld_src,
                      long long ld_dst, int* status, cudaStream_t stream);
// Same, for row slices: segment s copies `cols` elements from 16-byte vector seg_src_col_vec[s] of its source rows to vector
// seg_dst_col_vec[s] of its destination rows (the Ulysses sequence <-> head exchange).
// out rows [seg_dst_start[s], +seg_count[s]) = sum over the ranks in seg_peer_mask[s] of rows [seg_src_start[s], ...) of
// peer_ptrs[rank]; bf16 rows of `cols` elements, fp32 accumulation in rank order.
int ocb_peer_reduce_rows(void* const* peer_ptrs, int world, void* out, const long long* seg_src_start,
                         const long long* seg_dst_start, const int* seg_count, const int* seg_peer_mask, int num_segments,
                         int cols, long long ld_src, long long ld_dst, cudaStream_t stream);
int ocb_push_row_slices(const void* src, const int* seg_src_start, const int* seg_count, const int* seg_dst_rank,
                        const long long* seg_dst_start, const int* seg_src_col_vec, const int* seg_dst_col_vec,
                        int num_segments, void* const* peer_ptrs, int world, long long dst_capacity_rows, int cols,
                        long long ld_src, long long ld_dst, int* status, cudaStream_t stream);

// ---- normalisation / rotary / activation (elementwise.cu) -------------------------------------------
// y = rmsnorm(x) * w  (+ resid).  x,y,resid: [rows, cols] with row strides ldx/ldy/ldr. w: [cols].
// group = width of one normalisation group (cols for a full-row norm, head_dim for a per-head norm).
int ocb_rmsnorm_fwd(const void* x, const void* w, const void* resid, void* y, float* rstd, int rows, int cols,
                    int group, long long ldx, long long ldy, long long ldr, float eps, int act_dtype, int w_dtype,
                    cudaStream_t stream);
// dx = d rmsnorm; dw_partial: [n_partial, cols] fp32 scratch (n_partial returned by ocb_norm_bwd_partials()).
int ocb_norm_bwd_partials();
int ocb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_partial,
                    int rows, int cols, int group, long long lddy, long long ldx, long long lddx, int act_dtype,
                    int w_dtype, cudaStream_t stream);
// out[c] (+)= sum_p partial[p, c]; out is fp32 or bf16.
int ocb_reduce_partials(const float* partial, void* out, int n_partial, int cols, int accumulate, int out_dtype,
                        cudaStream_t stream);

// Fused (optional) RMSNorm + rotary embedding over [rows, n_heads*head_dim] rows.
// norm_mode: 0 = none, 1 = full-row norm, 2 = per-head norm. sin/cos: [max_pos, head_dim] fp32.
// pos_ids: optional int32 [rows]; when null the position is (row % seq_len) + pos_offset.
int ocb_norm_rope_fwd(const void* x, const void* w, void* y, float* rstd, const float* sin_t, const float* cos_t,
                      const int* pos_ids, int rows, int n_heads, int head_dim, int seq_len, int pos_offset,
                      int norm_mode, long long ldx, long long ldy, float eps, int act_dtype, int w_dtype,
                      cudaStream_t stream);
int ocb_norm_rope_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_partial,
                      const float* sin_t, const float* cos_t, const int* pos_ids, int rows, int n_heads, int head_dim,
                      int seq_len, int pos_offset, int norm_mode, long long lddy, long long ldx, long long lddx,
                      int act_dtype, int w_dtype, cudaStream_t stream);

// out = silu(a) * b ; (da, db) = d/d(a,b) given dout.
int ocb_swiglu_fwd(const void* a, const void* b, void* out, long long rows, int cols, long long lda, long long ldb,
                   long long ldo, int act_dtype, cudaStream_t stream);
int ocb_swiglu_bwd(const void* dout, const void* a, const void* b, void* da, void* db, long long rows, int cols,
                   long long lddo, long long lda, long long ldb, long long ldda, long long lddb, int act_dtype,
                   cudaStream_t stream);

// ---- loss (elementwise.cu) -------------------------------------------------------------------------
// Row-wise cross entropy + z-loss over logits [rows, vocab] (bf16 or fp32, row stride ld).
// Writes ce[row], z[row] (0 for ignored rows) and, when dlogits != null, the gradient
//   grad_scale * ((softmax - onehot) + 2*z_mult*lse*softmax)   (may alias logits).
int ocb_cross_entropy_fwd_bwd(const void* logits, const long long* labels, float* ce, float* z, void* dlogits,
                              int rows, int vocab, long long ld, long long ldd, long long ignore_index, float z_mult,
                              const float* grad_scale, int act_dtype, cudaStream_t stream);

// ---- embedding --------------------------------------------------------------------------------------
int ocb_embedding_fwd(const long long* ids, const void* table, void* out, int rows, int dim, long long vocab,
                      int act_dtype, cudaStream_t stream);
// dtable[ids[r]] += dout[r]  (fp32 atomics)
int ocb_embedding_bwd(const long long* ids, const void* dout, float* dtable, int rows, int dim, long long vocab,
                      int act_dtype, cudaStream_t stream);

// ---- optimiser --------------------------------------------------------------------------------------
// SkipStep-AdamW over a flat fp32 range. step / step_factor / grad_scale are device scalars (fp32);
// grad_scale and step_factor may be null (=1). p_lowp (bf16 copy of the updated parameters) may be null.
int ocb_adamw_step(float* p, float* m, float* v, const void* g, void* p_lowp, long long n, float lr, float beta1,
                   float beta2, float eps, float weight_decay, const float* step, const float* step_factor,
                   const float* grad_scale, int grad_dtype, cudaStream_t stream);
// out[0] (+)= sum(x^2). scratch: fp32 [ocb_sumsq_partials()] device buffer.
int ocb_sumsq_partials();
int ocb_sumsq(const void* x, long long n, float* scratch, float* out, int accumulate, int dtype, cudaStream_t stream);
// y = bf16(x * scale) / generic cast helpers
int ocb_cast_f32_to_bf16(const float* x, void* y, long long n, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
