/* C ABI of the sm_100a kernel library (libceo_b200.so).
 *
 * Every entry point takes raw device pointers and a stream, allocates nothing
 * (callers pass outputs and scratch), and returns 0 on success, a positive
 * cudaError_t value when a launch failed, or a negative code for rejected
 * arguments (-2 alignment, -3/-4 tensor-map encoding, -5 shape/dtype).
 * bf16 tensors are row-major with the stated leading dimension in elements.
 *
 * This plays the role of the reference's kernels/cuda/include/kernels.h:35-421
 * (26 prototypes); the Python shims in ceo_b200/ops bind it through ctypes the
 * way src/kernels/*_kernels.zig bind the reference's.
 */
#ifndef CEO_KERNELS_H
#define CEO_KERNELS_H

#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CEO_NORM_BWD_MAX_BLOCKS 592  /* 148 SMs x 4 */
#define CEO_SUMSQ_MAX_BLOCKS 1184    /* 148 SMs x 8 */

/* ---- GEMM (tcgen05 / TMEM / TMA) -------------------------------------------
 * C[b] (M x N) = alpha * A[b] (M x K) * B[b]^T (N x K)  (+bias[n]) (+residual) (+C if accumulate)
 * a_mn_major = 0: A stored (M rows, K contiguous, lda); 1: A stored (K rows, M contiguous, lda)
 * b_mn_major = 0: B stored (N rows, K contiguous, ldb); 1: B stored (K rows, N contiguous, ldb)
 * out_f32: C is fp32 (else bf16).  residual is bf16.  `status` is a device int that the
 * kernel sets non-zero if one of its bounded waits ran out (it then returns normally).
 * max_ctas > 0 caps the persistent grid (leaves SMs free for a concurrent kernel). */
int ceo_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                  long long ldb, long long ldc, int a_mn_major, int b_mn_major, int batch,
                  long long batch_stride_a, long long batch_stride_b, long long batch_stride_c,
                  int out_f32, int accumulate, float alpha, const float* bias,
                  const void* residual, long long ldr, long long batch_stride_r, int* status,
                  int max_ctas, cudaStream_t stream);

/* 1: weight-gradient GEMMs never split K (split-K accumulates with fp32 atomics, whose order
 * varies from run to run).  Default 0. */
int ceo_set_deterministic(int on);

/* ---- EFLA (chunked delta rule), chunk = 64, D in {64, 128}, T % 64 == 0 -------------
 * q,k,v: bf16 (B,T,H,D) with a token stride in elements (slices of a fused QKV output are
 * fine); alpha fp32 (B,T,H); s0 / s_final / ds_final / ds0 fp32 (B,H,D,D) (s0, ds_final may
 * be NULL).  Saved for backward: w, up (bf16 (B,T,H,D)), states (bf16 (B,H,T/64,D,D)), xinv (bf16
 * (B,H,T/64,64,64): the inverse of each chunk's 64x64 triangular system).
 * resets (optional): bytes (B,T/64); non-zero marks a chunk that starts a new document, i.e.
 * the state entering it is zero (packed sequences aligned to the chunk length).
 * Backward workspaces: dloc, dup (bf16 (B,T,H,D)), dstates (bf16 (B,H,T/64,D,D)). */
int ceo_efla_fwd(const void* q, const void* k, const void* v, const float* alpha, const float* s0,
                 void* w, void* up, void* states, void* xinv, void* o, float* s_final,
                 const unsigned char* resets, int B, int T, int H, int D, long long q_stride,
                 long long k_stride, long long v_stride, int* status, cudaStream_t stream);
int ceo_efla_bwd(const void* q, const void* k, const void* v, const float* alpha, const void* w,
                 const void* up, const void* states, const void* xinv, const void* dO,
                 const float* ds_final, void* dloc, void* dup, void* dstates, void* dq, void* dk,
                 void* dv, float* dalpha, float* ds0, const unsigned char* resets, int B, int T,
                 int H, int D, long long q_stride, long long k_stride,
                 long long v_stride, long long dq_stride, long long dk_stride,
                 long long dv_stride, int* status, cudaStream_t stream);
/* 1: compute the chunk outputs with the tcgen05 kernel (chunk pairs, D = 128, even chunk count;
 * other shapes keep the warp-MMA kernel).  Default 0: it is the slower of the two today. */
int ceo_efla_set_tcgen05(int on);
/* One of the six EFLA kernels at a time (0 wy, 1 state_fwd, 2 out, 3 bwd_local, 4 state_bwd,
 * 5 bwd_final).  ptrs (host array of 25 device pointers): 0 q, 1 k, 2 v, 3 alpha, 4 w, 5 u,
 * 6 up, 7 states, 8 o, 9 s0, 10 s_final, 11 dO, 12 dloc, 13 dup, 14 dstates, 15 ds_final,
 * 16 ds0, 17 dq, 18 dk, 19 dv, 20 dalpha, 21 p_final (optional, stage 1: also returns the
 * span's transfer matrix P with S_out = P S_in + R), 22 status word (optional), 23 xinv, 24 resets (optional);
 * strides (host array of 6): q, k, v, dq, dk, dv. */
int ceo_efla_stage(int stage, void* const* ptrs, const long long* strides, int B, int T, int H,
                   int D, cudaStream_t stream);
/* q/k L2 normalisation (optional) + alpha = c(beta, |k|^2); one launch each way.
 * beta: fp32 (rows*H) or one scalar (beta_scalar = 1).  qn, kn: bf16 (rows, H, D) dense. */
int ceo_efla_prep_fwd(const void* q, const void* k, const float* beta, int beta_scalar, void* qn,
                      void* kn, float* rq, float* rk, float* alpha, long long rows, int H, int D,
                      long long q_stride, long long k_stride, int normalize, cudaStream_t stream);
int ceo_efla_prep_bwd(const void* dqn, const void* dkn, const void* qn, const void* kn,
                      const float* rq, const float* rk, const float* beta, int beta_scalar,
                      const float* dalpha, void* dq, void* dk, float* dbeta, long long rows, int H,
                      int D, long long dq_stride, long long dk_stride, int normalize,
                      cudaStream_t stream);

/* ---- normalisation ---------------------------------------------------------- */
int ceo_norm_bwd_blocks(int rows); /* rows of the partial scratch the bwd kernels need */
int ceo_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* h_out,
                    float* rstd, int rows, int D, float eps, cudaStream_t stream);
/* partial_scratch: fp32 [ceo_norm_bwd_blocks(rows)][D] */
int ceo_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                    const void* dres, void* dx, float* dw, int dw_accumulate,
                    float* partial_scratch, int rows, int D, cudaStream_t stream);
int ceo_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean,
                      float* rstd, int rows, int D, float eps, cudaStream_t stream);
/* partial_scratch: fp32 [ceo_norm_bwd_blocks(rows)][2*D] */
int ceo_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean,
                      const float* rstd, void* dx, float* dw, float* db, int accumulate,
                      float* partial_scratch, int rows, int D, cudaStream_t stream);

/* ---- activations ------------------------------------------------------------ */
int ceo_swiglu_fwd(const void* gate_up, void* out, long long rows, int F, cudaStream_t stream);
int ceo_swiglu_bwd(const void* dout, const void* gate_up, void* dgate_up, long long rows, int F,
                   cudaStream_t stream);
/* mode 0 tanh-GELU, 1 erf-GELU, 2 SiLU, 3 ReLU */
/* SwiGLU on a (rows, 2F) gate/up tensor whose gate and up columns alternate (interleaved = 1:
 * column 2j = gate_j, 2j+1 = up_j, the layout of the fused GEMM epilogue) or sit in two
 * halves (interleaved = 0). */
int ceo_swiglu_il_fwd(const void* gate_up, void* out, long long rows, int F, int interleaved,
                      cudaStream_t stream);
int ceo_swiglu_il_bwd(const void* dout, const void* gate_up, void* dgate_up, long long rows, int F,
                      int interleaved, cudaStream_t stream);
int ceo_act_fwd(const void* x, void* y, long long n, int mode, cudaStream_t stream);
int ceo_act_bwd(const void* dy, const void* x, void* dx, long long n, int mode,
                cudaStream_t stream);
int ceo_softmax_fwd(const float* x, float* y, int rows, int n, cudaStream_t stream);
/* Inverted dropout on bf16: y = keep ? x / (1 - p) : 0, keep from a stateless hash of
 * (element index, seed); the backward pass is the same call on dy with the same seed. */
int ceo_dropout(const void* x, void* y, long long n, float p, unsigned int seed,
                cudaStream_t stream);

/* ---- causal depthwise short convolution: x,y (B,T,D) bf16, weight (D,Wn) bf16 ------- */
int ceo_shortconv_fwd(const void* x, const void* weight, void* y, int B, int T, int D, int Wn,
                      cudaStream_t stream);
int ceo_shortconv_bwd_input(const void* dy, const void* weight, void* dx, int B, int T, int D,
                            int Wn, cudaStream_t stream);
int ceo_shortconv_bwd_weight(const void* dy, const void* x, float* dw, int B, int T, int D, int Wn,
                             int accumulate, cudaStream_t stream);

/* ---- loss ------------------------------------------------------------------- */
int ceo_cross_entropy(const void* logits, int logits_f32, const long long* targets, float* loss,
                      void* dlogits_bf16, int rows, int V, long long ld, long long ldd,
                      float label_smoothing, const float* scale_ptr, float scale,
                      long long ignore_index, cudaStream_t stream);

/* ---- embedding -------------------------------------------------------------- */
int ceo_embedding_fwd(const long long* ids, const void* table, void* out, long long n, int D,
                      long long vocab, int* oob_count, cudaStream_t stream);
int ceo_embedding_bwd(const long long* ids, const void* dy, float* dtable, long long n, int D,
                      long long vocab, cudaStream_t stream);

/* ---- optimizers / clipping ---------------------------------------------------- */
int ceo_sumsq_blocks(long long n); /* floats of partial scratch ceo_sumsq / ceo_muon_momentum need */
int ceo_sumsq(const void* x, int is_f32, long long n, float* out, int accumulate,
              float* partial_scratch, cudaStream_t stream);
int ceo_clip_scale(const float* sumsq, float max_norm, float* scale_out, float* norm_out,
                   cudaStream_t stream);
int ceo_scale(void* x, int is_f32, long long n, const float* scale_ptr, float scale,
              cudaStream_t stream);
int ceo_clip_value(float* x, long long n, float clip, cudaStream_t stream);
int ceo_adamw_step(float* master, float* m, float* v, void* grad, int grad_f32, void* shadow_bf16,
                   long long n, float lr, float beta1, float beta2, float eps, float weight_decay,
                   int step, const float* gscale_ptr, float gscale, int zero_grad,
                   cudaStream_t stream);
int ceo_lion_step(float* master, float* m, void* grad, int grad_f32, void* shadow_bf16,
                  long long n, float lr, float beta1, float beta2, float weight_decay,
                  const float* gscale_ptr, float gscale, int zero_grad, cudaStream_t stream);
int ceo_muon_momentum(float* m, void* grad, int grad_f32, long long n, float beta,
                      const float* gscale_ptr, float gscale, int zero_grad, float* sumsq_out,
                      float* partial_scratch, cudaStream_t stream);
int ceo_muon_normalize(const float* m, const float* sumsq, void* y_bf16, long long n, float eps,
                       cudaStream_t stream);
int ceo_ns_poly(void* g_bf16, const void* g2_bf16, int n, float a, float b, float c,
                cudaStream_t stream);
/* gscale_ptr (optional): the device clip scale of the step; exactly 0 marks a step whose
 * gradient norm was not finite, which every update kernel above and this one then skip. */
int ceo_muon_apply(float* master, const void* y_bf16, void* shadow_bf16, long long n, float lr,
                   float weight_decay, float scale, const float* gscale_ptr,
                   cudaStream_t stream);

/* ---- PRISM refinement (one iteration in the head_dim-wide proxy space) -------------------
 * gate: bd = sigmoid(bt) * gelu_tanh(p * rp), all (n) bf16, n a multiple of 8; the backward
 * returns d(rp), d(p), d(bt) from d(bd).  update: r_out = r_in - c, out_out = out_in +
 * scale * c in one pass (outputs may alias their inputs).  state: the recurrent state
 * S_t = alpha S_{t-1} (I - b k^T) + sum_l bd^l k^l^T with b = sigmoid(bt1) * k^1 over T tokens;
 * bd, k: (L, B, T, hd) bf16 (L <= 4), bt1: (B, T, hd) beta logits of iteration 1, s_in (may
 * be null = zero) / s_out: (B, hd, hd) fp32, hd in {32, 64, 128}. */
int ceo_prism_gate_fwd(const void* rp, const void* p, const void* bt, void* bd, long long n,
                       cudaStream_t stream);
int ceo_prism_gate_bwd(const void* dbd, const void* rp, const void* p, const void* bt, void* drp,
                       void* dp, void* dbt, long long n, cudaStream_t stream);
int ceo_prism_update(const void* c, const void* r_in, const void* out_in, void* r_out,
                     void* out_out, long long n, float scale, cudaStream_t stream);
int ceo_prism_state(const void* bd, const void* k, const void* bt1, const float* s_in,
                    float* s_out, int B, int T, int hd, int L, float alpha, cudaStream_t stream);

/* Bounds-checked debug build only (-DCEO_BOUNDS_CHECK; -1 otherwise): out[4] = {violations,
 * site, index, extent} of the first out-of-range index recorded since the last reset. */
int ceo_bounds_status(long long* out, int reset);
/* Checked build only: indexes buf[0 .. n + extra) through the checked accessor (the `extra`
 * indices are recorded and redirected, nothing outside buf is touched); buf holds n + 1
 * floats, the sum is added to buf[n]. */
int ceo_bounds_selftest(float* buf, int n, int extra, cudaStream_t stream);

/* ---- fill / cast / copy / reduce / fp8 (dtype: 0 fp32, 1 fp16, 2 bf16) ---------- */
int ceo_fill(void* x, int dtype, long long n, float value, cudaStream_t stream);
int ceo_cast(const void* src, int src_dtype, void* dst, int dst_dtype, long long n,
             cudaStream_t stream);
int ceo_copy(const void* src, void* dst, long long bytes, cudaStream_t stream);
int ceo_axpby_f32(float* y, const float* x, long long n, float a, float b, cudaStream_t stream);
int ceo_reduce_blocks(long long n);
int ceo_reduce(const void* x, int dtype, long long n, int mode, float* out, float* partial_scratch,
               cudaStream_t stream);
int ceo_fp8_quantize(const void* x_bf16, void* q, long long n, const float* scale, float* amax_out,
                     int kind, cudaStream_t stream);
/* codes of x (rows, cols; both multiples of 16) written transposed, qt (cols, rows), and, when q
 * is not null, in the order of x as well; one read of x. */
int ceo_fp8_quantize_t(const void* x_bf16, void* q, void* qt, int rows, int cols, long long ldx,
                       const float* scale, float* amax_out, int kind, cudaStream_t stream);
int ceo_fp8_dequantize(const void* q, void* x_bf16, long long n, const float* scale, int kind,
                       cudaStream_t stream);
int ceo_fp8_update_scale(float* history, int hist_len, int* cursor, float* amax, float* scale,
                         float fp8_max, float margin_pow2, cudaStream_t stream);

/* ---- scan / gather / scatter / memory utilities --------------------------------------
 * cumsum: fp32 rows of n elements, inclusive or exclusive, optionally from the end of the row;
 * `scratch` must hold ceo_cumsum_scratch_floats(rows, n) floats (0 for many short rows).
 * gather / scatter move rows of row_bytes (multiple of 16) by 64-bit row indices; indices out
 * of range give zero rows (gather) or are skipped (scatter).  transpose16 works on any 2-byte
 * element type. */
int ceo_cumsum_scratch_floats(long long rows, long long n);
int ceo_cumsum_f32(const float* x, float* y, long long rows, long long n, int exclusive,
                   int reverse, float* scratch, cudaStream_t stream);
int ceo_gather_rows(const long long* idx, const void* src, void* dst, long long n,
                    long long row_bytes, long long src_rows, cudaStream_t stream);
int ceo_scatter_rows(const long long* idx, const void* src, void* dst, long long n,
                     long long row_bytes, long long dst_rows, cudaStream_t stream);
int ceo_scatter_add_f32(const long long* idx, const float* src, float* dst, long long n, int D,
                        long long dst_rows, cudaStream_t stream);
int ceo_copy2d(const void* src, long long src_pitch, void* dst, long long dst_pitch,
               long long rows, long long row_bytes, cudaStream_t stream);
int ceo_transpose16(const void* src, void* dst, int rows, int cols, long long lds, long long ldd,
                    cudaStream_t stream);
int ceo_memset32(void* x, long long n, unsigned int value, cudaStream_t stream);

/* bf16 GEMM with SwiGLU in the epilogue.  mode 1: C (M x N) = A B^T holds gate/up in
 * interleaved columns (2j gate, 2j+1 up) and aux (M x N/2) receives silu(gate) * up; N a
 * multiple of 64.  mode 2: A B^T is d(act) (M x N, N a multiple of 32), aux is the saved
 * interleaved gate/up (M x 2N) and C (M x 2N) receives the interleaved d(gate/up). */
int ceo_gemm_bf16_swiglu(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                         long long ldb, long long ldc, int a_mn_major, int b_mn_major, float alpha,
                         int mode, void* aux, long long ld_aux, int* status, cudaStream_t stream);

/* C = alpha / (scale_a * scale_b) * A[M,K] @ B[N,K]^T (+ bias) (+ residual): 8-bit float
 * operands (kind 0 e4m3, 1 e5m2), both K-major, strides multiples of 16; scale_a / scale_b
 * are the device-side quantisation scales (both null: no rescaling). */
int ceo_gemm_fp8(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                 long long ldb, long long ldc, int kind_a, int kind_b, int out_f32,
                 int accumulate, float alpha, const float* scale_a, const float* scale_b,
                 const float* bias, const void* residual, long long ldr, int* status,
                 cudaStream_t stream);

/* ---- peer-memory collectives (NVLink), fused with their compute --------------------------
 * Buffers are plain cudaMalloc allocations mapped into every rank through CUDA IPC; the
 * `void* const*` arguments are host arrays of `world` device pointers indexed by rank (this
 * rank's own entry is its local pointer).  flags: 8 slots x 8 unsigned per rank, zeroed once;
 * `epoch` must grow by at least 2 between uses of the same slot set.  world <= 8. */
int ceo_dev_malloc(void** out, long long bytes);
int ceo_dev_free(void* p);
int ceo_dev_memset(void* p, int value, long long bytes, cudaStream_t stream);
int ceo_ipc_get_handle(void* p, void* handle64);
int ceo_ipc_open(const void* handle64, void** out);
int ceo_ipc_close(void* p);
int ceo_symm_barrier(void* const* flags, int rank, int world, int slot, unsigned int epoch,
                     int* status, cudaStream_t stream);
int ceo_symm_allreduce(void* const* bufs, void* const* flags, float* out, int n, int rank,
                       int world, unsigned int epoch, int* status, cudaStream_t stream);
/* All-gather fused into the consuming GEMM (copy CTAs pull peer shards through shared memory
 * with bulk async copies while the other CTAs compute, local rows first; the TMA producer
 * waits on per-row-block flags).  gathered[r] = rank r's (rows x K) bf16 buffer whose own
 * shard is already in place; operand 1 = A (M rows), 2 = B (N rows).  flags: local
 * unsigned[rows / blk_rows], zeroed once; target grows by 1 per call.  blk_rows: rows per
 * flag, a divisor of rows / world (0 = 128 for A, 256 for B).  extra (optional): per-rank
 * buffers of a second tensor sharded into extra_shard_bytes per rank that the copy CTAs
 * gather after the operand (complete when the kernel ends).
 * copy_ctas: number of copy CTAs (0 = 8); -1 = copy-first mode: every CTA of the grid first
 * moves its round-robin share of 32 KB chunks of the peers' shards (operand and extra tensor),
 * then computes; flags[0] is then the launch's counter (zeroed in stream by the call) and
 * blk_rows / target are not used.  Right for weights (a gather much shorter than the GEMM).
 * Call ceo_symm_barrier first so every rank's shard is complete. */
int ceo_ag_gemm_bf16(void* const* gathered, int operand, const void* other, void* C, int M, int N,
                     int K, long long ld_other, long long ldc, int other_mn_major, int out_f32,
                     int accumulate, float alpha, const void* residual, long long ldr, void* flags,
                     unsigned int target, int rank, int world, int copy_ctas, int blk_rows,
                     void* const* extra, long long extra_shard_bytes, int* status,
                     cudaStream_t stream);
/* GEMM fused with the reduce-scatter of its output over M (epilogue stores partial tiles
 * into the owner's staging area over NVLink and bumps its counters; each rank then reduces
 * its own rows, adding an optional bf16 residual).  stage[r]: [world][M/world][N] bf16;
 * counters[r]: unsigned[world][M/world/128], zeroed once and never reset: target is the value
 * they reach when this call's tiles have all arrived (+ 4*ceil(N/256) per call with the same
 * M).  rs_ctas CTAs (0 = 32) only reduce, stripe by stripe, while the others compute.
 * Successive calls alternate between two staging buffers instead of a barrier between them. */
int ceo_gemm_rs_bf16(const void* A, const void* B, int M, int N, int K, long long lda,
                     long long ldb, int a_mn_major, int b_mn_major, float alpha,
                     void* const* stage, void* const* counters, unsigned int target, void* out,
                     const void* residual, long long ldo, int rank, int world, int rs_ctas,
                     int* status, cudaStream_t stream);
/* Context-parallel exchange: store `n` floats into slot `rank` of every rank's gather buffer
 * (n floats per slot) and barrier, in one launch.  done_counter: local unsigned, zero. */
int ceo_cp_exchange(const float* src, void* const* gather, void* const* flags, long long n,
                    int rank, int world, unsigned int epoch, unsigned int* done_counter,
                    int* status, cudaStream_t stream);
/* out[b] = P[b] s[b] + R[b] (transpose: P[b]^T) for nb d x d fp32 matrices, d a multiple of 16:
 * one step of composing a rank's affine state map in context parallelism. */
int ceo_fold_affine(const float* P, const float* s, const float* R, float* out, int nb, int d,
                    int transpose, cudaStream_t stream);
/* One cooperative launch per rank: reduce-scatter of the fp32 gradients (peer loads) ->
 * global-norm clip -> AdamW (kind 0) or Lion (kind 1; v unused) on the rank's fp32 master
 * shard -> bf16 parameters stored into every rank's buffer -> this rank's gradient buffer
 * zeroed.  `ranges`: device array of nranges records {long long goff, len, loff; int gather,
 * pad}: rank r owns flat elements [goff + r*len, goff + (r+1)*len), its master weights and
 * moments for them sit at [loff, loff + len) of master / m / v; gather = 0 keeps the updated
 * bf16 values local (a later fused all-gather moves them).  do_reduce = 0: the gradients
 * were already reduced by ceo_zero_bucket_reduce launches, whose squared norms are in
 * local_acc[0].  local_acc: 2 floats.  clip_out receives the clip scale used; 0 means the
 * gradient norm was not finite and the step was skipped (states and parameters untouched,
 * gradients zeroed).  When a peer barrier's bounded wait runs out the kernel writes the
 * status word and returns without touching any state. */
int ceo_zero_step(void* const* grads, void* const* params, void* const* flags, void* const* slots,
                  float* master, float* m, float* v, float* local_acc, float* norm_out,
                  float* clip_out, int* status, const void* ranges, int nranges, long long total,
                  long long decay_end, int rank, int world, unsigned int epoch, int kind,
                  int do_reduce, float lr, float beta1, float beta2, float eps,
                  float weight_decay, int step, float gscale, float max_norm, int max_ctas,
                  cudaStream_t stream);
/* Flag barrier (slot 4) + reduce-scatter of ranges [r0, r1) on `stream`, for overlap with the
 * rest of the backward pass: the sums stay in this rank's gradient buffer, their squared norm
 * is added to local_acc[0].  ctas bounds the grid (0 = 32). */
int ceo_zero_bucket_reduce(void* const* grads, void* const* flags, const void* ranges, int r0,
                           int r1, int rank, int world, unsigned int epoch, float* local_acc,
                           int* status, int ctas, cudaStream_t stream);
/* Run-time override of the iteration limit of every bounded wait in the library (0 = the
 * compile-time defaults).  For tests that make a wait run out; not for production use. */
int ceo_set_wait_limit(unsigned int iterations);
int ceo_gemm_set_wait_limit(unsigned int iterations);
int ceo_efla_set_wait_limit(unsigned int iterations);

#ifdef __cplusplus
}
#endif
#endif /* CEO_KERNELS_H */
