// C entry points of the sm_100a kernels (called from bindings.cpp; no torch types here so the
// kernels compile in seconds).  dtype codes: 0 = fp32, 1 = bf16.  All launches are asynchronous
// on `stream`; a non-zero return value is a host-side launch / argument error.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// D = alpha·op(A)·op(B) (+beta·C).  mode 0: A[M,K]·B[N,K]ᵀ, 1: A[M,K]·B[K,N], 2: A[K,M]ᵀ·B[K,N].
int b200_gemm_bf16(int mode, const void* A, const void* B, void* out, const void* cin, int M, int N, int K, int lda,
                   int ldb, int ldc, float alpha, float beta, int out_f32, int accumulate, int num_sms, int* status,
                   cudaStream_t stream);

int b200_gemm_bf16_batched(int mode, const void* A, const void* B, void* out, const void* cin, int batch, int M, int N,
                           int K, float alpha, float beta, int num_sms, int* status, cudaStream_t stream);

// RMSNorm over the last dim.  x:[rows,cols] (fp32|bf16), w:[cols] or null, out dtype chosen by out_dtype.
int b200_rmsnorm_fwd(const void* x, int x_dtype, const void* w, int w_dtype, void* out, int out_dtype, float* rstd,
                     int rows, int cols, float eps, cudaStream_t stream);
// dx (dtype of x) and per-CTA partial dw [n_partials, cols] fp32 (n_partials = return of b200_rmsnorm_bwd_partials).
int b200_rmsnorm_bwd_partials(int rows, int cols);
int b200_rmsnorm_bwd(const void* dy, int dy_dtype, const void* x, int x_dtype, const void* w, int w_dtype,
                     const float* rstd, void* dx, float* dw_partial, float* dw, int rows, int cols, cudaStream_t stream);

// Fused residual add + RMSNorm: x = res + h_scale·h (stored to res_out when h != null; out_dtype 0: fp32 stream, 1: bf16 stream,
// which needs bf16 res), n = rmsnorm(x)·w (bf16).
int b200_add_rmsnorm_fwd(const void* res, int res_dtype, const void* h, float h_scale, const void* w, int w_dtype,
                         void* res_out, void* n_out, float* rstd, int rows, int cols, float eps, cudaStream_t stream,
                         int out_dtype = 0);
// d_res = g_res + rmsnorm_bwd(g_n), d_h = bf16(h_scale·d_res) (optional); g_dtype: type of g_res and d_res (0 fp32, 1 bf16 with bf16 x);
// cols: a multiple of 8 up to 4096.
int b200_add_rmsnorm_bwd(const void* g_res, const void* g_n, const void* x, int x_dtype, const void* w, int w_dtype,
                         const float* rstd, void* d_res, void* d_h, float h_scale, float* dw_partial, float* dw,
                         int rows, int cols, cudaStream_t stream, int g_dtype = 0);

// SwiGLU: y = silu(g)·u.  Packed variant reads g = x[:, :I], u = x[:, I:] from a [rows, 2I] bf16 tensor.
int b200_swiglu_fwd(const void* g, const void* u, void* y, int64_t n, cudaStream_t stream);
int b200_swiglu_bwd(const void* g, const void* u, const void* dy, void* dg, void* du, int64_t n, cudaStream_t stream);
int b200_swiglu_packed_fwd(const void* x, void* y, int64_t rows, int I, cudaStream_t stream);
int b200_swiglu_packed_bwd(const void* x, const void* dy, void* dx, int64_t rows, int I, cudaStream_t stream);

// Cross-entropy over a logits chunk, in place: logits ← d(Σ loss)/d logits, loss[row] fp32.
int b200_cross_entropy_fwd_bwd(void* logits, int dtype, const int64_t* target, float* loss, int rows, int vocab,
                               int64_t row_stride, int ignore_index, float label_smoothing, float lse_square_scale,
                               cudaStream_t stream);

// Per-head RMSNorm (optional) + NeoX RoPE (optional) on q:[N,H,D] and k:[N,G,D] bf16; T = positions per batch row.
int b200_qknorm_rope_fwd(const void* q, const void* k, const void* qw, const void* kw, int w_dtype, const void* cos,
                         const void* sin, void* qo, void* ko, float* q_rstd, float* k_rstd, int64_t n_tokens, int T,
                         int H, int G, int D, float eps, int64_t q_token_stride, int64_t k_token_stride, cudaStream_t stream);
int b200_qknorm_rope_bwd(const void* dqo, const void* dko, const void* q, const void* k, const void* qw, const void* kw,
                         int w_dtype, const void* cos, const void* sin, const float* q_rstd, const float* k_rstd,
                         void* dq, void* dk, float* dqw, float* dkw, float* dw_partial /* [grid, 2, D] */,
                         int64_t n_tokens, int T, int H, int G, int D, int64_t q_token_stride, int64_t k_token_stride,
                         cudaStream_t stream);
// The same on heads addressed through a group layout: query head h of a token sits at (h / q_hpg)·q_gs + (h % q_hpg)·D from the
// token's query base, key (value) head g at g·k_gs from its base.  Dense rows: q_hpg = H, k_gs = D.  The per-group interleaved
// output of a fused QKV projection: q_hpg = q_per_kv, q_gs = k_gs = (q_per_kv + 2)·D.  Forward can also copy the value heads to
// dense rows (v, vo); backward writes dq / dk in a layout of its own (o_*) and can copy a dense dv into that layout (dvo, dv_dst),
// so the gradient of the fused projection is assembled without a concatenation.
int b200_qknorm_rope_fwd_ex(const void* q, const void* k, const void* v, const void* qw, const void* kw, int w_dtype, const void* cos,
                            const void* sin, void* qo, void* ko, void* vo, float* q_rstd, float* k_rstd, int64_t n_tokens, int T,
                            int H, int G, int D, float eps, int64_t q_ts, int64_t k_ts, int q_hpg, int64_t q_gs, int64_t k_gs,
                            cudaStream_t stream);
int b200_qknorm_rope_bwd_ex(const void* dqo, const void* dko, const void* dvo, const void* q, const void* k, const void* qw,
                            const void* kw, int w_dtype, const void* cos, const void* sin, const float* q_rstd, const float* k_rstd,
                            void* dq, void* dk, void* dv_dst, float* dqw, float* dkw, float* dw_partial, int64_t n_tokens, int T,
                            int H, int G, int D, int64_t q_ts, int64_t k_ts, int q_hpg, int64_t q_gs, int64_t k_gs, int64_t o_q_ts,
                            int64_t o_k_ts, int o_q_hpg, int64_t o_q_gs, int64_t o_k_gs, cudaStream_t stream);
int b200_qknorm_rope_grid();

// ---- mixture of experts (moe_routing.cu, gemm_bf16.cu)
int b200_topk_indices(const float* logits, int* idx, int N, int E, int K, cudaStream_t stream);
int b200_routing_chunks(int n_pairs);
int b200_routing_capacity(int n_pairs, int E);
int b200_routing_layout(const int* expert_of_pair, int n_pairs, int E, int* counts, int* offsets, int* slot_pair,
                        int* pair_slot, int capacity, int* scratch, cudaStream_t stream);
// The three row kernels check every index they read against its table (pair < n_pairs, 0 <= slot < capacity): an index
// outside is reported as STATUS_INDEX_RANGE in the status word and its access is skipped.
int b200_gather_rows(const void* x, const int* slot_pair, const float* pair_scale, void* xs, int capacity, int C, int K,
                     const int* offsets, int E, cudaStream_t stream, int n_pairs, int* status);
int b200_combine_rows(const void* y, const int* pair_slot, const float* w, void* out, int N, int C, int K, const void* add,
                      float alpha, cudaStream_t stream, int capacity, int* status);
int b200_pair_dots(const void* y, const void* g, const int* pair_slot, float* dots, int n_pairs, int C, int K, cudaStream_t stream,
                   int capacity, int* status);
int b200_grouped_gemm_bf16(int kind, const void* A, const void* B, void* out, const int* offsets, int E, int capacity, int M,
                           int N, int K, int out_f32, int accumulate, int num_sms, int* status, cudaStream_t stream);

// Attention forward (attention_fwd.cu).  q:[B,T,H,D] k,v:[B,T,G,D] bf16 → out bf16, lse fp32 [B,H,T].
// row_start: optional int32 [B*T], first key each query row may see (packed documents).
int b200_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, const int* row_start, int B, int T,
                  int H, int G, int D, int window_left, float scale, int* status, cudaStream_t stream);

// Two-stream variant of the forward kernel (attention_fwd2s.cu); same contract.  ARCHSCALE_B200_ATTN_FWD=2stream routes
// b200_attn_fwd to it.  set_trace: development aid, 16×64 int64 clock stamps of the first CTA, null = off.
int b200_attn_fwd_2s(const void* q, const void* k, const void* v, void* out, float* lse, const int* row_start, int B, int T,
                     int H, int G, int D, int window_left, float scale, int* status, cudaStream_t stream);
void b200_attn_fwd_2s_set_trace(long long* buf);
// Single-kernel backward (attention_bwd1.cu): five products per tile pair, dQ summed in fp32 through `dq_acc` [B,T,H,D]
// with reductions in memory (fast, not bitwise reproducible).  ARCHSCALE_B200_ATTN_BWD=split selects the two-kernel form.
int b200_attn_bwd1(const void* d_out, const void* q, const void* k, const void* v, const void* out, const float* lse, float* delta,
                   float* dq_acc, const int* row_start, const int* doc_end, void* dq, void* dk, void* dv, int B, int T, int H,
                   int G, int D, int window_left, float scale, int* status, cudaStream_t stream);
int b200_attn_bwd_delta(const void* out, const void* d_out, float* delta, int B, int T, int H, int D, cudaStream_t stream);
void b200_attn_bwd_set_trace(long long* buf);       // same aid for the dK/dV kernel: 8×64 stamps

// Attention backward (attention_bwd.cu): δ preprocess + dK/dV kernel + dQ kernel, deterministic.
// delta: fp32 scratch [B,H,T]; doc_end: optional int32 [B*T] (exclusive end of each position's document).
int b200_attn_bwd(const void* d_out, const void* q, const void* k, const void* v, const void* out, const float* lse,
                  float* delta, const int* row_start, const int* doc_end, void* dq, void* dk, void* dv, int B, int T,
                  int H, int G, int D, int window_left, float scale, int* status, cudaStream_t stream);

// ---- peer-memory collectives (comm.cu).  `bases[p]` = local mapping of rank p's symmetric heap.
// Forward GEMM with the FSDP all-gather of the whole flat parameter group fused in (gemm_bf16.cu).
int b200_ag_gemm_bf16(const void* A, void* out, int M, int N, int K, int lda, int ldc, const void* const* bases,
                      size_t src_off, void* dst, size_t shard_bytes, size_t b_off, uint32_t* flags, uint32_t epoch,
                      int rank, int world, int n_copy, int num_sms, int* status, cudaStream_t stream);
void b200_set_peer_wait_limit_cycles(long long cycles);
int b200_symm_barrier(const void* const* bases, size_t signal_off, int channel, int rank, int world, uint32_t epoch,
                      int* status, cudaStream_t stream);
int b200_symm_post(const void* const* bases, size_t signal_off, int channel, int rank, int world, uint32_t epoch,
                   cudaStream_t stream);
int b200_symm_wait(const void* const* bases, size_t signal_off, int channel, int rank, int world, uint32_t epoch,
                   int* status, cudaStream_t stream);
int b200_pull_pieces(const void* const* bases, size_t obj_off, void* dst, const void* table, int n_pieces, int world,
                     int max_ctas, cudaStream_t st);
int b200_allgather_pull(const void* const* bases, size_t src_off, void* dst, size_t shard_bytes, int rank, int world,
                        int max_ctas, cudaStream_t stream);
int b200_reduce_scatter_pull(const void* const* bases, size_t full_off, float* out, size_t shard_elems, int rank,
                             int world, float scale, int accumulate, int max_ctas, cudaStream_t stream);
int b200_reduce_scatter_pull_bf16(const void* const* bases, size_t full_off, void* out, size_t shard_elems, int rank,
                                  int world, int max_ctas, cudaStream_t stream);

// Expert-parallel dispatch (owners pull their experts' rows from every rank's send buffer) and return.
int b200_ep_plan(const void* const* bases, size_t off_counts, size_t off_table, int rank, int world, int e_local,
                 int recv_cap, int* recv_offsets, int* status, cudaStream_t stream);
int b200_ep_pull(const void* const* bases, size_t off_counts, size_t off_offsets, size_t off_table, size_t off_send,
                 void* recv_local, int rank, int world, int e_local, int C, int recv_cap, const int* recv_offsets,
                 cudaStream_t stream);
int b200_ep_return(const void* const* bases, size_t off_counts, size_t off_offsets, size_t off_table, size_t off_result,
                   void* dst, int rank, int world, int e_local, int C, cudaStream_t stream);

// Depthwise causal conv1d (+SiLU) on token-major rows (conv1d.cu); dw [C,W], db [C] fp32 must be zero on entry.
int b200_conv1d_fwd(const void* x, int dtype, const float* w, const float* bias, const int* seq_idx, void* y, int B, int L, int C,
                    int W, int silu, int xs, cudaStream_t st);
int b200_conv1d_bwd(const void* dy, const void* x, int dtype, const float* w, const float* bias, const int* seq_idx, void* dx,
                    float* dw, float* db, int B, int L, int C, int W, int silu, int xs, int dys, cudaStream_t st);
// Mamba-1 selective scan (selective_scan.cu), 16 states per channel, token-major.
int b200_selective_scan_ckpt_segments(int L);
int b200_selective_scan_fwd(const void* u, int su, const void* delta, int sd, const float* A, const void* Bm, int sB,
                            const void* Cm, int sC, const float* D, const void* z, int sz, const float* dbias, const int* reset,
                            void* y, float* ckpt, int dtype, int B, int L, int Di, int softplus, cudaStream_t st);
int b200_selective_scan_bwd(const void* dy, int sdy, const void* u, int su, const void* delta, int sd, const float* A,
                            const void* Bm, int sB, const void* Cm, int sC, const float* D, const void* z, int sz,
                            const float* dbias, const int* reset, const float* ckpt, void* du, void* ddelta, void* dz, float* dA,
                            float* partB, float* partC, void* dB, void* dC, float* dD, float* ddbias, int dtype, int B, int L,
                            int Di, int softplus, cudaStream_t st);
int b200_selective_scan_channel_blocks(int Di);

// Block-scaled MXFP8 (gemm_mxfp8.cu): quantisers and the tcgen05 block-scaled GEMM.
size_t b200_mxfp8_sf_bytes(int rows, int K);
int b200_mxfp8_quantize(const void* x, int ld, void* q, void* sf, int R, int C, int colwise, cudaStream_t st,
                        void* qT = nullptr, void* sfT = nullptr);   // colwise 2: both orientations from one read
int b200_gemm_mxfp8(const void* A, const void* sfa, const void* B, const void* sfb, void* out, int M, int N, int K, int lda,
                    int ldb, int ldc, float alpha, int out_f32, int accumulate, int num_sms, int* status, cudaStream_t stream);
// NVFP4 (gemm_mxfp8.cu): packed e2m1 elements, E4M3 scales per 16 elements, one fp32 scale per tensor derived on the device
// from the tensor's largest magnitude (amax: fp32 [1] in device memory, zeroed before b200_nvfp4_amax).
size_t b200_nvfp4_sf_bytes(int rows, int K);
int b200_nvfp4_amax(const void* x, int ld, float* amax, int R, int C, cudaStream_t st);
int b200_nvfp4_quantize(const void* x, int ld, void* q, void* sf, void* qT, void* sfT, const float* amax, int R, int C, int mode,
                        cudaStream_t st, int stochastic = 0, unsigned seed = 0, int rht = 0, unsigned sign_mask = 0);
int b200_gemm_nvfp4(const void* A, const void* sfa, const void* B, const void* sfb, const float* amax_a, const float* amax_b,
                    void* out, int M, int N, int K, int lda, int ldb, int ldc, float alpha, int out_f32, int accumulate,
                    int num_sms, int* status, cudaStream_t stream);

// LayerNorm (layernorm.cu)
int b200_layernorm_bwd_partials(int rows);
int b200_layernorm_fwd(const void* x, int dtype, const float* w, const float* bias, void* y, float* mean, float* rstd, int rows,
                       int cols, float eps, cudaStream_t st);
int b200_layernorm_bwd(const void* dy, const void* x, int dtype, const float* w, const float* mean, const float* rstd, void* dx,
                       float* part, float* dw, float* db, int rows, int cols, cudaStream_t st);

// Tensor-parallel fused layers (gemm_bf16.cu): activation all-gather → GEMM, and GEMM → reduce-scatter over peer memory.
int b200_ag_a_gemm_bf16(const void* const* bases, size_t src_off, void* dst, size_t shard_bytes, const void* B, void* out, int M,
                        int N, int K, int ldb, int ldc, uint32_t* flags, uint32_t epoch, int rank, int world, int n_copy,
                        int num_sms, int* status, cudaStream_t stream);
int b200_gemm_rs_bf16(const void* A, const void* B, int M, int N, int K, int lda, int ldb, const void* const* bases,
                      size_t part_off, size_t cnt_off, uint32_t expect, void* out_local, int rank, int world, int num_sms,
                      int* status, cudaStream_t stream);

// Optimizer kernels on flat fp32 shards (optim.cu)
int b200_muon_momentum(const float* g, float* m, void* u, long long n, float mu, int nesterov, const float* gscale, cudaStream_t st);
int b200_seg_update(int mode, float* x, const void* u, long long n, const long long* bounds, const int* kidx, int nseg,
                    const float* coef, float* acc, cudaStream_t st);
int b200_adamw_fused(int mode, float* x, const float* g, float* m, float* v, float* u_out, long long n, float lr, float beta1,
                     float beta2, float eps, float wd, float bc1, float bc2, const float* gscale, float* acc, cudaStream_t st);

// Gated RMSNorm with groups (gated_norm.cu)
int b200_gated_rmsnorm_fwd(const void* x, const void* z, const float* w, void* y, float* rstd, int dtype, long long rows, int cols,
                           int gsize, float eps, int norm_before_gate, cudaStream_t st);
int b200_gated_rmsnorm_bwd(const void* dy, const void* x, const void* z, const float* w, const float* rstd, void* dx, void* dz, float* dw,
                           int dtype, long long rows, int cols, int gsize, int norm_before_gate, cudaStream_t st);

// Differential-attention combine (diff_attn.cu)
int b200_diff_combine_fwd(const void* a1, const void* a2, const float* lam, const float* w, float c, void* y, float* rstd, long long rows,
                          int width, float eps, cudaStream_t st);
int b200_diff_combine_bwd(const void* dy, const void* a1, const void* a2, const float* lam, const float* w, float c, const float* rstd,
                          void* da1, void* da2, float* dlam, float* dw, long long rows, int width, cudaStream_t st);

// 2-CTA (cta_group::2) variant of b200_gemm_bf16: one 256×256 tile per pair of SMs (gemm2_bf16.cu)
int b200_gemm2_bf16(int mode, const void* A, const void* B, void* out, const void* cin, int M, int N, int K,
                    int lda, int ldb, int ldc, float alpha, float beta, int out_f32, int accumulate,
                    int num_sms, int* status, cudaStream_t stream);

int b200_grouped_gemm2_bf16(int kind, const void* A, const void* B, void* out, const int* offsets, int E,
                            int capacity, int M, int N, int K, int out_f32, int accumulate, int num_sms,
                            int* status, cudaStream_t stream);
int b200_gemm2_bf16_batched(int mode, const void* A, const void* B, void* out, const void* cin, int batch, int M,
                            int N, int K, float alpha, float beta, const float* alpha_vec, const float* beta_vec, int symmetric,
                            int num_sms, int* status, cudaStream_t stream);

// Chunk-to-chunk state recurrence of the SSD scan and its backward (ssd_scan.cu); PN = head_dim · state, a multiple of 1024
int b200_ssd_state_fwd(const float* add, const float* keep, float* s_in, int B, int nC, int H, int PN, cudaStream_t st);
int b200_ssd_state_bwd(const float* d_s_in, const float* s_in, const float* keep, float* d_add, float* d_keep_part,
                       int B, int nC, int H, int PN, cudaStream_t st);
// NT product with SwiGLU in the epilogue on the SM-pair kernel (gemm2_bf16.cu): act = silu(A·B_gateᵀ)∘(A·B_upᵀ), h optional
int b200_gemm2_swiglu_bf16(const void* A, const void* B, void* h, void* act, int M, int I, int K, int lda, int ldb, int num_sms,
                           int* status, cudaStream_t stream);
int b200_grouped_gemm2_swiglu_bf16(const void* A, const void* B, void* h, void* act, const int* offsets, int E, int capacity,
                                   int I, int K, int num_sms, int* status, cudaStream_t stream);
// Row-wise "prepare" stage of the chunked gated delta rule and its backward (gdn_prepare.cu)
int b200_gdn_prepare_fwd(const void* q, const void* k, const void* v, const float* gc, void* qn, void* kn, void* vc, void* kd,
                         void* qg, int B, int T, int Tp, int H, int Dk, int Dv, float scale, float eps, cudaStream_t st);
int b200_gdn_prepare_bwd(const void* q, const void* k, const float* gc, const void* dqn, const void* dkn, const void* dvc,
                         const void* dkd, const void* dqg, void* dq, void* dk, void* dv, float* a_row, float* s_row, int B, int T,
                         int Tp, int H, int Dk, int Dv, float scale, float eps, cudaStream_t st);
// Intra-chunk part of the SSD scan and its backward (ssd_intra.cu); x_dtype 0 fp32 / 1 bf16
int b200_ssd_intra_fwd(const void* x, int x_dtype, const float* dt, const float* cs, const float* CB, const int* bc, float* y,
                       int B, int nC, int H, int G, int P, cudaStream_t st);
int b200_ssd_intra_bwd(const void* x, int x_dtype, const float* dt, const float* cs, const float* CB, const int* bc, const float* dy,
                       float* dx, float* ddt, float* dcs, float* dCB, int B, int nC, int H, int G, int P, int hsplit, cudaStream_t st);
// (I + A)^-1 for [n_mat, 64, 64] strictly lower-triangular fp32 matrices (tri_inverse.cu)
int b200_tri_inverse64(const float* A, float* T, int n_mat, cudaStream_t st);
// One pass of the chunked gated-delta-rule recurrence (gdn_chunk.cu)
int b200_gdn_state(const void* a_op, const void* c_add, const void* bm_op, const void* e_op, const void* f_op,
                   const float* decay, void* v_out, void* x_all, float* x_final, int BH, int Tp, int DK, int DV,
                   float sgn_p, float sgn_v, int reverse, int* status, cudaStream_t stream);

void b200_gemm_set_splitk_workspace(uint32_t* sem, int n);

#ifdef __cplusplus
}
#endif
