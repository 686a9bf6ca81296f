// C launch interface of the CUDA kernels.  Everything takes raw device pointers
// and a stream; the PyTorch bindings (bindings.cpp) and any other host can call
// these directly.  All functions return 0 on success or a negative error code.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ------------------------------------------------------------------ tcgen05 GEMM
// C[M,N] = alpha * A[M,K] * B[N,K]^T (+ beta * D), bf16 operands, fp32 accumulation in TMEM.
enum { KMOE_GEMM_DENSE = 0, KMOE_GEMM_GROUPED_M = 1, KMOE_GEMM_BATCHED = 2 };
enum { KMOE_EPI_STORE = 0, KMOE_EPI_SWIGLU = 1 };
enum { KMOE_MAJOR_K = 0, KMOE_MAJOR_MN = 1 };

typedef struct KmoeGemmDesc {
  const void* A;        // bf16. K-major: [rows, K] (lda); MN-major: [K, rows] (lda)
  const void* B;        // bf16. K-major: [N, K] (ldb);    MN-major: [K, N] (ldb)
  const void* B2;       // SWIGLU epilogue only: second weight (same layout as B)
  void* C;              // bf16 or fp32 output, row-major [M, N] (ldc)
  const void* D;        // optional addend with C's type and ldd
  const void* D2;       // optional second addend (bf16 output, CTA-pair kernel): C = alpha A B + beta D + beta2 D2
  void* G_out;          // SWIGLU only, optional: pre-activation gate, [M, N] bf16 (ldc)
  void* U_out;          // SWIGLU only, optional: up projection
  int mode;             // KMOE_GEMM_*
  int epilogue;         // KMOE_EPI_*
  int M, N, K;          // per-group dims. GROUPED_M: M = rows of the whole padded buffer
  int groups;           // GROUPED_M: number of B groups; BATCHED: number of independent GEMMs
  int a_major, b_major;
  long long lda, ldb, ldc, ldd;
  long long a_gstride, b_gstride, c_gstride;  // elements between groups (0 = shared)
  // GROUPED_M: m-tile i covers rows [128 i, 128 i + 128) of A and C and uses B group tile_group[i];
  // *num_m_tiles (device) tiles are live.
  const int* tile_group;
  const int* num_m_tiles;
  // BATCHED, optional ragged reduction range per group, in elements of K (multiples of 64).
  const int* k_begin;
  const int* k_len;
  int out_f32;
  float alpha, beta, beta2;
  const float* row_scale;  // optional per-row multiplier applied to the product
  // optional (STORE epilogue): device array with the address of every output row, which may lie in a
  // peer GPU's memory; 0 skips the row.  Replaces C + row * ldc; D is still read at its usual place.
  const long long* c_row_ptr;
  // optional device arrays, one entry per group of a BATCHED GEMM (entry 0 otherwise): alpha and beta are
  // multiplied by them, so scalars computed on the device (e.g. 1 / norm) need no separate pass.
  const float* alpha_dev;
  const float* beta_dev;
  // Symmetric products (M == N, bf16 output; A A^T, or two commuting symmetric operands): tiles entirely below
  // the diagonal are not computed but mirrored from the upper part.  Addends must be symmetric too.
  int sym_upper;
  // added to the elements on the main diagonal of every (group's) output after alpha is applied (STORE
  // epilogue, bf16 output): C = alpha * A B + diag_add * I, e.g. the 1.5 I - 0.5 X X^T factor of Newton-Schulz
  float diag_add;
  // STORE epilogue, optional: the reduction is the concatenation of two B operands, elements [0, k_split) from
  // B and [k_split, K) from B2 (same layout, ldb and group stride; k_split a multiple of 64), while A is one
  // [M, K] operand.  C = A[:, :k_split] B^T + A[:, k_split:] B2^T in one pass, e.g. dX = [dG | dU] [W1 ; W2].
  int k_split;
  int* status;             // device int; non-zero after the launch = a bounded wait expired
  int num_sms;             // 0 = query
} KmoeGemmDesc;

int kmoe_gemm(const KmoeGemmDesc* d, cudaStream_t stream);
void kmoe_gemm_clear_tensormap_cache(void);

// ------------------------------------------------------------ Muon elementwise passes
// `n_mat` matrices of `numel` bf16 elements each.  buf: stacked momentum (n_mat, numel); grad_ptrs / param_ptrs:
// device arrays with the address of each matrix's gradient / parameter.
//   momentum: buf = mu * buf + grad ; sumsq[i] += sum(buf_i^2)      (sumsq zeroed by the caller)
//   apply   : param = param * (1 - lr * wd) - lr * (nesterov ? grad + mu * ortho : ortho) ; buf = ortho
// gcoef (optional device float): the gradients are read as bf16(g * bf16(*gcoef)) - a clip coefficient applied on
// the fly instead of by a pass over the gradients in memory.
int kmoe_muon_momentum(void* buf, const long long* grad_ptrs, float* sumsq, int n_mat, long long numel, float mu,
                       const float* gcoef, cudaStream_t st);
int kmoe_muon_apply(void* buf, const void* ortho, const long long* grad_ptrs, const long long* param_ptrs, int n_mat,
                    long long numel, float lr, float mu, float wd, int nesterov, const float* gcoef, cudaStream_t st);

// int8 momentum of Muon8bit: blocks of `block` elements, q = rint(x / s * 127) with s = max(absmax, 1e-8).
// x / g / out are fp32 or bf16 (is_bf16); q holds ceil(n / block) * block bytes, scales one float per block.
//   quant   : x -> (q, scales)
//   momentum: out = mu * dequant(q, scales) + g
int kmoe_q8_quant(const void* x, int is_bf16, signed char* q, float* scales, long long n, int block, cudaStream_t st);
int kmoe_q8_momentum(const signed char* q, const float* scales, const void* g, int is_bf16, void* out, long long n,
                     int block, float mu, cudaStream_t st);

// ------------------------------------------------------------ MXFP8 (e4m3 + e8m0 1x32 block scales)
// Scale factors live in 512-byte chunks, one per (128 operand rows, 128 reduction elements):
//   chunk = (row / 128) * (K / 128) + k / 128,  byte = (row % 32) * 16 + ((row % 128) / 32) * 4 + (k % 128) / 32
// which is the arrangement the block-scaled tensor-core instruction expects in tensor memory.
long long kmoe_mx_sf_bytes(long long rows, long long K);
// x (rows, C) bf16 -> q (rows, C) e4m3, reduction along C (C % 128 == 0).  x2 != NULL: quantise silu(x) * x2.
// live_rows (device, optional): only the first *live_rows rows are processed.
int kmoe_mx_quant_rows(const void* x, const void* x2, long long rows, int C, long long ld, void* q, void* sf,
                       const int* live_rows, cudaStream_t st);
// x (groups, R, C) bf16 -> q (groups, C, R) e4m3, reduction along R (R % 128 == 0); scale rows are (group, c).
int kmoe_mx_quant_cols(const void* x, int groups, long long R, int C, long long ld, long long g_stride, void* q,
                       void* sf, const int* live_rows, cudaStream_t st);

typedef struct KmoeMxGemmDesc {
  const void* A;        // e4m3 [M, K] (or [groups, M, K] when a_grouped), K contiguous
  const void* B;        // e4m3 [N, K] (or [groups, N, K] when b_grouped)
  const void* sfa;      // scale chunks of A / B in the arrangement above
  const void* sfb;
  void* C;              // bf16 or fp32 [M, N] (ldc)
  const void* D;        // optional addend (C's type, ldd)
  int mode;             // KMOE_GEMM_DENSE / GROUPED_M / BATCHED
  int M, N, K, groups;  // K % 128 == 0
  int a_grouped, b_grouped;
  long long ldc, ldd, c_gstride;
  const int* tile_group;
  const int* num_m_tiles;
  const int* k_begin;   // BATCHED: optional ragged reduction range per group (multiples of 128)
  const int* k_len;
  int out_f32;
  float alpha, beta;
  int* status;
  int num_sms;
} KmoeMxGemmDesc;
int kmoe_gemm_mxfp8(const KmoeMxGemmDesc* d, cudaStream_t stream);
void kmoe_mxfp8_clear_tensormap_cache(void);

// ------------------------------------------------------------ row kernels (bf16 data, fp32 math)
int kmoe_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int d, float eps, cudaStream_t st);
/* residual add + norm in one pass: sum_out = x + addend, y = rmsnorm(sum_out) (addend / sum_out both or neither) */
int kmoe_add_rmsnorm_fwd(const void* x, const void* addend, const void* w, void* sum_out, void* y, float* rstd,
                         int rows, int d, float eps, cudaStream_t st);
/* kmoe_rmsnorm_bwd plus the gradient of the residual branch (dres, bf16 [rows, d], optional) added into dx */
int kmoe_rmsnorm_bwd_res(const void* x, const void* w, const void* dy, const float* rstd, const void* dres, void* dx,
                         void* dw_bf16, float* dw_f32, float* partial, int rows, int d, cudaStream_t st);
int kmoe_rmsnorm_bwd_num_partials(int rows);
// sum of squares of n bf16 values (16-byte aligned) in fp32, summed in a fixed order; partial = scratch of
// kmoe_sumsq_num_partials() floats
int kmoe_sumsq_num_partials(void);
int kmoe_sumsq_bf16(const void* x, long long n, float* partial, float* out, cudaStream_t st);
// dst = bf16(src * *scale) over n bf16 values (both 16-byte aligned; scale is a device float)
int kmoe_scale_copy(const void* src, void* dst, long long n, const float* scale, cudaStream_t st);
// out (bf16, n values) = sum of nparts fp32 vectors of n values stored back to back; n % 4 == 0
int kmoe_sum_partials(const float* partial, void* out, int nparts, long long n, cudaStream_t st);
/* nn.Linear(d, 1): y[row] = x[row, :] . w ; backward gives dx (optional) and dw (bf16 and/or fp32). */
int kmoe_rowdot_fwd(const void* x, const void* w, void* y, int rows, int d, cudaStream_t st);
int kmoe_rowdot_bwd(const void* x, const void* w, const void* dy, void* dx, void* dw_bf16, float* dw_f32,
                    float* partial, int rows, int d, cudaStream_t st);
int kmoe_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx, void* dw_bf16,
                     float* dw_f32, float* partial, int rows, int d, cudaStream_t st);
int kmoe_rope(const void* x, const float* cs, const float* sn, void* out, int B, int S, int H, int D,
              long long cs_bstride, int transpose, cudaStream_t st);
// live_rows (device, optional): only the first min(rows, *live_rows) rows are processed.
int kmoe_swiglu_fwd(const void* g, const void* u, void* h, long long rows, int cols, long long ldg, long long ldu,
                    const int* live_rows, cudaStream_t st);
int kmoe_swiglu_bwd(const void* g, const void* u, const void* dh, void* dg, void* du, long long rows, int cols,
                    long long ldg, long long ldu, long long ldo, const int* live_rows, cudaStream_t st);

// --------------------------------------------------------------------------- Mamba
// groups: number of parameter sets stacked along the first dimension of w / bias (A, D, dt_bias for the scan);
// batch entries [g * B / groups, (g + 1) * B / groups) use set g.  1 = one set for the whole batch.
int kmoe_conv1d_fwd(const void* x, const float* w, const float* bias, void* y, int B, int S, int C, long long ldx,
                    int act, int groups, cudaStream_t st);
int kmoe_conv1d_bwd(const void* x, const float* w, const float* bias, const void* dy, void* dx, float* dw,
                    float* dbias, int B, int S, int C, long long ldx, int act, int groups, cudaStream_t st);
// Selective scan.  The sequence is processed in kmoe_scan_segments(B, S, C) parallel segments.
//   ckpt (forward, optional): [B, ceil(S / kmoe_scan_chunk()), N, C] floats, the state before every chunk.
//   seg  (required when there is more than one segment): [B, segments, N + 1, C] floats of scratch that the
//        backward pass reads again;  gseg: [B, segments, N, C] floats of scratch for the backward pass.
//   C % 8 == 0, N == 16.
int kmoe_scan_chunk(void);
int kmoe_scan_segments(int B, int S, int C);
int kmoe_scan_fwd(const void* u, const void* delta, const void* z, const float* A, const float* Bm, const float* Cm,
                  const float* D, const float* dt_bias, void* out, float* ckpt, float* seg, int B, int S, int C,
                  int N, long long ldz, int softplus, int groups, cudaStream_t st);
int kmoe_scan_bwd(const void* u, const void* delta, const void* z, const float* A, const float* Bm, const float* Cm,
                  const float* D, const float* dt_bias, const void* dout, const float* ckpt, const float* seg,
                  float* gseg, void* du, void* ddelta, void* dz, long long lddz, float* dA, float* dB, float* dC,
                  float* dD, float* dbias, int B, int S, int C, int N, long long ldz, int softplus, int groups,
                  cudaStream_t st);

// ------------------------------------------------------------------- MoE bookkeeping
int kmoe_moe_max_rows(int n_assign, int E);
int kmoe_moe_plan(const long long* idx, const unsigned char* keep, int n, int E, int max_rows, int expert_base,
                  int* pos, int* row_src, int* counts, int* offsets, int* tile_group, int* meta, cudaStream_t st);
// keep[i] = assignment i is among the first `cap` of its expert in flat (token, slot) order
int kmoe_moe_capacity_mask(const long long* idx, int n, int E, int cap, unsigned char* keep, cudaStream_t st);
// greedy balanced top-k assignment, slot by slot (probs [T, E] fp32, taken [T, E] zeroed, counts [k + 1, E] zeroed,
// sel [T, k] int64 out): see moe_balanced_slot_kernel
int kmoe_moe_balanced_assign(const float* probs, unsigned char* taken, int* counts, long long* sel, int T, int E,
                             int k, int cap, cudaStream_t st);
int kmoe_moe_gather_rows(const void* src, const int* row_src, const float* assign_scale, const int* meta, void* dst,
                         int max_rows, int d, int div, cudaStream_t st);
int kmoe_moe_combine(const void* Y, const int* pos, const float* w, void* out, int T, int k, int d, cudaStream_t st);
int kmoe_moe_combine_dw(const void* Y, const void* dout, const int* pos, float* dw, int n, int k, int d,
                        cudaStream_t st);

// ----------------------------------------------------------------------- attention
// Causal GQA flash attention. q/out/dq [B,S,H,D], k/v/dk/dv [B,S,Hkv,D] bf16; lse, delta [B,H,S] fp32; D in {64,128}.
// doc_start (optional, (B, S) int32): first position of the packed document containing each position; a query
// then attends to keys doc_start[q] <= k <= q only (causal attention that does not cross document boundaries).
int kmoe_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int H, int Hkv,
                  int D, float scale, const int* doc_start, int* status, cudaStream_t st);
int kmoe_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                  float* delta, void* dq, void* dk, void* dv, int B, int S, int H, int Hkv, int D, float scale,
                  const int* doc_start, int* status, cudaStream_t st);

// ------------------------------------------- collectives over NVLink peer pointers
// `*_ptrs`: device addresses (as integers) of the same symmetric buffer on every rank, indexed by rank.
int kmoe_p2p_barrier(const long long* flag_ptrs, int rank, int world, int epoch, double timeout_s, int* status,
                     cudaStream_t st);
// mc_ptr: multicast (NVLink switch) address of the same symmetric buffer, or 0 to use plain peer accesses.
int kmoe_p2p_reduce_scatter(const long long* grad_ptrs, int rank, int world, long long off, long long n,
                            float* sq_out, long long mc_ptr, int max_blocks /*0 = whole device*/, cudaStream_t st);
int kmoe_p2p_adamw_allgather(const long long* param_ptrs, const void* grad, float* m, float* v, int rank, int world,
                             long long off, long long n, float lr, float beta1, float beta2, float eps, float wd,
                             int step, const float* clip_coef, long long mc_ptr, cudaStream_t st);
// src (optional): read the n elements from there instead of this rank's own buffer, and store them into it too.
int kmoe_p2p_allgather(const long long* buf_ptrs, int rank, int world, long long off, long long n, long long mc_ptr,
                       const void* src, int max_blocks /*0 = whole device*/, cudaStream_t st);

// Expert-parallel token exchange.  E experts are split evenly over `world` ranks (expert e lives on rank
// e / (E / world)).  The receive buffer of a rank holds (E / world) * world slots of `cap` rows; slot
// (e_local, src) belongs to source rank src.  `meta` holds (count, source row offset) per slot.
//   dispatch : rows of `src` selected by the local plan (row_src, offsets, counts over all E experts) are
//              stored into the owners' receive buffers; div > 0: source row = assignment / div (token
//              matrix), div == 0: source row = padded row; assign_scale (optional) multiplies each row.
//   recv_plan: counts -> padded expert-major layout of the received rows (offsets, tile_group, out_meta).
//   move     : dir 0 gathers the slots into that layout; dir 1 stores layout rows back into the source
//              ranks' return buffers at the rows their own plan assigned.
int kmoe_ep_dispatch(const void* src, const int* row_src, const float* assign_scale, const int* offsets,
                     const int* counts, const long long* recv_ptrs, const long long* meta_ptrs, int rank, int world,
                     int E, long long cap, int d, int div, int max_rows, cudaStream_t st);
int kmoe_ep_recv_plan(const int* meta_in, int n_local, int world, int max_rows, int* slot_dst, int* offsets,
                      int* tile_group, int* out_meta, cudaStream_t st);
// row_ptr_out (optional, dir 0): for every packed row the address of its place in the source rank's return
// buffer (0 for padding) - the table a GEMM epilogue uses to store its rows straight to the peers.
int kmoe_ep_move(const void* slots, void* packed, const int* meta_in, const int* slot_dst, const int* offsets,
                 const long long* ret_ptrs, int rank, int n_local, int world, long long cap, int d, int max_rows,
                 int dir, long long* row_ptr_out, cudaStream_t st);

// ---------------------------------------------------------------------------- routing decisions
// Token choice: softmax over E experts -> top-k -> renormalise; also accumulates (atomically, into
// zero-initialised buffers) sum_t p[t, e], the number of assignments per expert and sum_t lse_t^2.
int kmoe_route_topk_fwd(const float* logits, int T, int E, int k, float* w, long long* idx, float* lse, float* p_sum,
                        float* counts, float* z_sum, cudaStream_t st);
int kmoe_route_topk_bwd(const float* logits, const float* lse, const long long* idx, const float* w, const float* dw,
                        const float* counts, const float* d_aux, float w_lb, float w_z, int T, int E, int k,
                        float* dlogits, cudaStream_t st);
// Per-row top-k of a strided score matrix; row r starts at (r / rows_inner) * outer_stride +
// (r % rows_inner) * row_stride and its S entries are col_stride apart.  mode 0: k largest scores,
// indices ascending, softmax over the kept scores.  mode 1: softmax over the row, k largest
// probabilities (descending), renormalised; stat (rows, 3) keeps (max, denominator, kept mass).
int kmoe_seq_topk_fwd(const float* scores, long long row_stride, long long col_stride, int rows_inner,
                      long long outer_stride, int rows, int S, int k, int mode, long long* idx, float* w, float* stat,
                      cudaStream_t st);
int kmoe_seq_topk_bwd(const float* scores, long long row_stride, long long col_stride, int rows_inner,
                      long long outer_stride, int rows, int S, int k, int mode, const long long* idx, const float* w,
                      const float* dw, const float* stat, float* dscores, cudaStream_t st);

// ---------------------------------------------------------------------------- mixture-of-depths rows
// idx (B, k) int64, ascending per row, unique.  src/res/out/dout (B, S, d), proc/dproc (B, k, d), w/dw (B, k).
int kmoe_rows_gather(const void* src, const long long* idx, void* out, int B, int S, int k, int d, cudaStream_t st);
int kmoe_rows_scatter(const void* src, const long long* idx, void* out, int B, int S, int k, int d, cudaStream_t st);
// mean binary cross-entropy of bf16 logits [B, S] against "position is among the ascending kept indices idx [B, k]";
// dlogits (bf16 [B, S]) = gradient for an upstream gradient of 1; partial = scratch of kmoe_mod_bce_num_partials floats
int kmoe_mod_bce_num_partials(int B, int S);
int kmoe_mod_bce(const void* logits, const long long* idx, float* partial, float* loss, void* dlogits, int B, int S,
                 int k, cudaStream_t st);
// the same plus coef[b, t] * wvec[:] on every row (coef bf16 [B * S], wvec bf16 [d])
int kmoe_rows_scatter_rank1(const void* src, const long long* idx, const void* coef, const void* wvec, void* out,
                            int B, int S, int k, int d, cudaStream_t st);
int kmoe_mod_combine_fwd(const void* res, const void* proc, const float* w, const long long* idx, void* out, int B,
                         int S, int k, int d, cudaStream_t st);
int kmoe_mod_combine_bwd(const void* dout, const void* proc, const float* w, const long long* idx, void* dproc,
                         float* dw, int B, int S, int k, int d, cudaStream_t st);

// ---------------------------------------------------------------------------- loss
int kmoe_ce_fwd_bwd(void* logits, const long long* labels, float* loss_rows, const float* grad_scale, int R, int V,
                    long long ld, long long ignore_index, int write_grad, cudaStream_t st);

#ifdef __cplusplus
}
#endif
