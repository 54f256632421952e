/*
 * C ABI of libcoda_b200.so: B200 (sm_100a) kernels behind the fused-linear
 * operators of coda.kernels.functional.
 *
 * Conventions
 *  - Every pointer is a device pointer unless stated otherwise; the library
 *    allocates no device memory and never synchronises the device.  Work is enqueued on
 *    `stream` (a cudaStream_t passed as void*; NULL = legacy default stream) of
 *    the current device.
 *  - Matrices are bf16 unless stated otherwise.  An operand is described by its
 *    two element strides, exactly one of which must be 1, so transposed views
 *    (`w.mT`, `g.mT`) are consumed in place.  Base addresses must be 16-byte
 *    aligned and leading dimensions multiples of 8 elements.
 *  - Functions return 0 on success or a negative code (CODA_B200_E*) for
 *    arguments rejected on the host; coda_b200_last_error() then describes the
 *    problem.  Device-side trouble (a bounded wait that expired) is reported
 *    asynchronously through `dev_status`, an int32 the device can write that
 *    stays 0 on success and receives a positive code otherwise.  It may be
 *    device memory (read it back, or use coda_b200_status_poll) or pinned host
 *    memory, which the device maps at the same address: the kernels write it
 *    with a plain system-scope store, only on the failure path, and the host
 *    then sees the code by reading the word, with no copy and no CUDA call.
 *
 * Each entry point names the reference interface it stands in for, as
 * file:line inside the coda-kernels project.
 */
#ifndef CODA_B200_H_
#define CODA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CODA_B200_OK 0
#define CODA_B200_EARG (-1)    /* bad shape / alignment / stride */
#define CODA_B200_ELAYOUT (-2) /* operand not contiguous along either dimension */
#define CODA_B200_ECUDA (-3)   /* CUDA runtime error */
#define CODA_B200_EDRIVER (-4) /* tensor-map encoder not available */

/* Library version (major * 100 + minor). */
int coda_b200_version(void);

/* Message for the last non-zero return code on the calling thread. */
const char* coda_b200_last_error(void);

/* Tuning switches: "cta_group" (1 or 2), "group_m", "max_ctas", "tile_n"
 * (0 = automatic, 64, 128, 256; plain and sigmoid GEMMs only), "epi_tma"
 * (1 = epilogues stage output tiles in shared memory and write them with TMA
 * stores, the default; 0 = per-thread 16-byte stores), "split_tail" (1 = a plain
 * GEMM that is given a workspace may cut the tiles of its last round along K, the
 * default; 0 = never: see coda_b200_gemm_ws).  Options are
 * process-wide atomics: a launch reads them once at its start, so changing one
 * from another host thread is safe and affects later launches only.
 * "probe_ld_kb" / "probe_st_kb" (0 = off) are a measurement aid: KB of extra
 * global loads / shared-memory stores per k-block and CTA that the epilogue
 * warps issue while a GEMM's mainloop runs, to measure what the load/store
 * traffic of an operand-transforming prologue would cost; results are unchanged.
 * Returns 0, or CODA_B200_EARG for an unknown name or value. */
int coda_b200_set_option(const char* name, int value);

/* Failure-path self-test (no counterpart in the reference).  Launches one warp
 * that waits, with the same bounded wait every kernel role uses, on a barrier
 * that nothing arrives at; after `timeout_us` (1 us .. 1 s) the wait gives up,
 * the kernel returns normally and dev_status receives a positive code.
 * waited_us (device int32, may be NULL) receives the time the wait took. */
int coda_b200_selftest_wait_timeout(int* dev_status, int64_t timeout_us, int* waited_us, void* stream);

/* Non-blocking look at a `dev_status` that lives in device memory (no counterpart in the reference; a status word in
 * pinned host memory needs no call at all).  Each call first checks the snapshot the
 * previous call took: if that 4-byte copy has landed (an event query, never a wait) and holds a code, the code
 * (> 0) is returned once and the device word is cleared by an asynchronous memset on `stream`.  Otherwise it enqueues a
 * fresh copy of the word into pinned host memory on `stream` and returns 0.  So the call after the one that follows a
 * failed launch's completion reports it.  Returns 0 without enqueuing anything while `stream` is capturing; negative on
 * a CUDA error.  The one piece of state the library owns: a pinned host word and an event per device, created by
 * the first poll on that device. */
int coda_b200_status_poll(int* dev_status, void* stream);

/* D[M,N] = alpha * (A[M,K] @ B[K,N]); D row-major with leading dimension ldd,
 * bf16 (d_is_fp32 = 0) or fp32 (1); alpha = device fp32 scalar or NULL.
 * Replaces `coda::_gemm` and `coda::_gemm_scalar_scale_epi`
 * (coda/core/gemm/functional.py:35-51, 94-113; epilogue coda/core/gemm/epilogues.py:34-36). */
int coda_b200_gemm(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                   int64_t b_stride_n, void* D, int64_t ldd, int d_is_fp32, int M, int N, int K, const float* alpha,
                   int* dev_status, void* stream);

/* D[M,N] = alpha * (A @ B) + C in one kernel: C[M,N] row-major, bf16
 * (c_is_fp32 = 0) or fp32 (1), leading dimension ldc, may alias D; C = NULL
 * gives coda_b200_gemm.  Replaces the `C=` form of `gemm`, i.e. quack's
 * `gemm_add` (coda/core/gemm/functional.py:54-69). */
int coda_b200_gemm_add(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                       int64_t b_stride_n, const void* C, int64_t ldc, int c_is_fp32, void* D, int64_t ldd, int d_is_fp32,
                       int M, int N, int K, const float* alpha, int* dev_status, void* stream);

/* The same product as coda_b200_gemm with a caller-provided workspace that lets the library shorten the last round of
 * its persistent grid.  Tiles are dealt to the CTA pairs round-robin, so the `tiles mod pairs` tiles of the last
 * round keep that many pairs busy for a whole contraction while the rest idle.  With a workspace each of those tiles
 * is cut into equal ranges of k-blocks that run as separate work items; their fp32 partial accumulators go to
 * `workspace` and a follow-up kernel adds them in a fixed order, scales, converts and writes the tile (reproducible run
 * to run; the last bit may differ from the uncut product).  coda_b200_gemm_workspace_bytes(M, N, K) says how much
 * workspace such a launch wants under the current options: 0 when the schedule would be left alone (the cut must save
 * at least 15 % of the last round; option "split_tail" = 0 switches it off), in which case workspace may be NULL and
 * the call equals coda_b200_gemm.  A smaller workspace than asked for is not an error: the launch then runs whole tiles.
 * No counterpart in the reference (quack's persistent tile scheduler, coda/core/gemm/gemm_interface.py:103-143). */
int64_t coda_b200_gemm_workspace_bytes(int M, int N, int K);
int coda_b200_gemm_ws(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                      int64_t b_stride_n, void* D, int64_t ldd, int d_is_fp32, int M, int N, int K, const float* alpha,
                      void* workspace, int64_t workspace_bytes, int* dev_status, void* stream);

/* Input gradient of linear_sigmoid with the activation gradient fused into the
 * GEMM's A-operand path: dx[M, K] = G[M, N] @ W[N, K] where G = dout * out *
 * (1 - out) is formed tile by tile by the kernel's transform warps (packed bf16
 * math) instead of being read from memory; G is also written once, for the
 * weight-gradient GEMM.  out, dout, G: bf16 [M, N]; W: bf16 [N, K] row-major.
 * Replaces the `sigmoid_backward` pass + dgrad GEMM of
 * coda/kernels/functional/sigmoid.py:33-38 by one launch.  CTA-pair build only. */
int coda_b200_gemm_dsigmoid_dgrad(const void* out, int64_t ld_out, const void* dout, int64_t ld_dout, const void* W, int64_t ldw,
                                  void* G, int64_t ld_g, void* dx, int64_t ld_dx, int M, int N, int K, int* dev_status,
                                  void* stream);

/* D = sigmoid(A @ B).  For N <= 64 (one gate per attention head, the shape
 * the reference benchmarks) a 64-column tile is used.  Replaces `coda::_gemm_sigmoid_epi`
 * (coda/core/gemm/functional.py:199-217; epilogue coda/core/gemm/epilogues.py:39-41). */
int coda_b200_gemm_sigmoid(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                           int64_t b_stride_n, void* D, int64_t ldd, int d_is_fp32, int M, int N, int K, int* dev_status,
                           void* stream);

/* preact[M,N] = bf16(A @ B); postact[M,N/2][:, j] = silu(acc[:, 2j]) * acc[:, 2j+1]
 * (gate / up columns interleaved).  N must be a multiple of 16.  Replaces
 * `coda::_gemm_swiglu_epi` (coda/core/gemm/functional.py:237-258; epilogues.py:44-47). */
int coda_b200_gemm_swiglu(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                          int64_t b_stride_n, void* preact, int64_t ld_pre, void* postact, int64_t ld_post, int M, int N,
                          int K, int* dev_status, void* stream);

/* Extension (no counterpart in the reference): the sigmoid-gated projection
 * sigmoid(x @ W_gate^T) * (x @ W_val^T) with gate / value rows interleaved like the
 * SwiGLU weight: preact = bf16(A @ B) [M,N], postact[:, j] = sigmoid(acc[:, 2j]) *
 * acc[:, 2j+1] [M,N/2]; coda_b200_dsigmoid_glu is its backward element-wise pass
 * (dgate = dout*val*s*(1-s), dval = dout*s). */
int coda_b200_gemm_sigmoid_glu(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                               int64_t b_stride_n, void* preact, int64_t ld_pre, void* postact, int64_t ld_post, int M, int N,
                               int K, int* dev_status, void* stream);
int coda_b200_dsigmoid_glu(const void* preact, int64_t ld_pre, const void* dout, int64_t ld_dout, void* grad_pre, int64_t ld_grad,
                           int M, int F, void* stream);

/* Number of column tiles the LSE epilogue produces for N columns
 * (= second extent of part_max / part_sum). */
int coda_b200_lse_tiles(int N);

/* Log-sum-exp partials of A @ B per (row, column tile): part_max, part_sum
 * fp32 [M, coda_b200_lse_tiles(N)]; target_logit fp32 [M] receives
 * acc[i, target[i]] for rows whose int32 target lies in [0, N) (other rows are
 * left untouched).  If P != NULL, P[M,N] (bf16, leading dimension ldp)
 * receives exp(acc - tile max): the logits themselves are never stored.
 * Replaces `coda::_gemm_lse_epi` and `coda::_lse_select_logits_epi`
 * (coda/core/gemm/functional.py:342-368, 453-493). */
int coda_b200_gemm_lse(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                       int64_t b_stride_n, void* P, int64_t ldp, float* part_max, float* part_sum, const int32_t* target,
                       float* target_logit, int M, int N, int K, int* dev_status, void* stream);

/* Per row: lse = logsumexp over the tile partials; losses[i] = lse[i] -
 * target_logit[i], or 0 where target[i] == ignore_index.  lse, losses fp32 [M].
 * Replaces the `logsumexp(partials)` step and quack `cross_entropy_fwd_out`
 * call (coda/core/gemm/functional.py:337-339, 484-493). */
int coda_b200_lse_finalize(const float* part_max, const float* part_sum, int tiles_n, const int32_t* target,
                           const float* target_logit, int ignore_index, float* lse, float* losses, int M, void* stream);

/* In place: P[i,j] <- exp(tile max - lse[i]) * P[i,j] - (j == target[i]), or +0
 * for ignored rows; turns the stored probabilities into d(loss_i)/d(logits).
 * Replaces `cross_entropy_fwd_bwd_kernel`
 * (coda/core/elementwise/cross_entropy.py:18-131; wrapper coda/core/elementwise/functional.py:221-311). */
int coda_b200_ce_grad_fixup(void* P, int64_t ldp, const float* part_max, int tiles_n, const float* lse,
                            const int32_t* target, int ignore_index, int M, int N, void* stream);

/* Fused [q | k | v] projection.  N = (hq + hk + hv) * head_dim columns; q and k
 * heads get per-head RMSNorm (gamma = [gamma_q | gamma_k], bf16 [2*head_dim])
 * and interleaved-pair RoPE from `positions` (int32 or fp32 [M]) and
 * `frequencies` (fp32 [(hq+hk)*head_dim], (hi, lo) turns per pair); v heads are
 * stored as they are.  Outputs: qk, preact bf16 [M, (hq+hk)*head_dim];
 * v bf16 [M, hv*head_dim] (may be NULL when N has no v columns);
 * mean_sq fp32 [M, hq+hk].  head_dim is 64 or 128.  Replaces
 * `coda::_gemm_qknorm_rope_epi` plus the separate v GEMM
 * (coda/core/gemm/functional.py:1079-1200; coda/kernels/functional/qknorm_rope.py:27-42). */
int coda_b200_gemm_qknorm_rope(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                               int64_t b_stride_n, void* qk, int64_t ld_qk, void* preact, int64_t ld_pre, void* v,
                               int64_t ld_v, float* mean_sq, const void* gamma, const void* positions, int pos_is_float,
                               const float* frequencies, int head_dim, int hq, int hk, float eps, int M, int N, int K,
                               int* dev_status, void* stream);

/* grad_pre[M,2F] from preact[M,2F] (interleaved gate/up) and dout[M,F]:
 * dgate = dout*up*(s + g*s*(1-s)), dup = dout*g*s, s = sigmoid(g).
 * Replaces `dswiglu_backward` (coda/core/elementwise/functional.py:181-218). */
int coda_b200_dswiglu(const void* preact, int64_t ld_pre, const void* dout, int64_t ld_dout, void* grad_pre, int64_t ld_grad,
                      int M, int F, void* stream);

/* grad_pre = dout * out * (1 - out), bf16 result; out is bf16 (out_is_fp32 = 0)
 * or fp32.  Replaces the `aten.sigmoid_backward(...).to(x.dtype)` step of
 * coda/kernels/functional/sigmoid.py:35. */
int coda_b200_dsigmoid(const void* out, int64_t ld_out, int out_is_fp32, const void* dout, int64_t ld_dout, void* grad_pre,
                       int64_t ld_grad, int M, int N, void* stream);

/* Deferred-RMSNorm variants: the same three fused GEMMs with the accumulator
 * multiplied by a per-row fp32 scale `rstd[M]` before the epilogue math, i.e.
 * the result of feeding rmsnorm(x) (without its weight) instead of x.
 *   swiglu:      preact = bf16(acc * rstd), postact from the scaled pairs
 *   lse:         logits = acc * rstd everywhere (partials, probabilities, target logit)
 *   qknorm_rope: q, k (statistic and output) and v use acc * rstd; preact keeps
 *                the unscaled acc, mean_sq is that of the scaled head
 * Replace `coda::_gemm_rmsnorm_swiglu_epi`, `coda::_gemm_rmsnorm_lse_epi` and the
 * `rstd_qknorm_rope_epi` program (coda/core/gemm/functional.py:283-334, 392-450;
 * coda/core/gemm/epilogues.py:50-58, 262-303).  rstd == NULL gives the plain ops. */
int coda_b200_gemm_rmsnorm_swiglu(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                                  int64_t b_stride_n, const float* rstd, void* preact, int64_t ld_pre, void* postact,
                                  int64_t ld_post, int M, int N, int K, int* dev_status, void* stream);
int coda_b200_gemm_rmsnorm_lse(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                               int64_t b_stride_n, const float* rstd, void* P, int64_t ldp, float* part_max, float* part_sum,
                               const int32_t* target, float* target_logit, int M, int N, int K, int* dev_status, void* stream);
int coda_b200_gemm_rmsnorm_qknorm_rope(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                       int64_t b_stride_k, int64_t b_stride_n, const float* rstd, void* qk, int64_t ld_qk,
                                       void* preact, int64_t ld_pre, void* v, int64_t ld_v, float* mean_sq, const void* gamma,
                                       const void* positions, int pos_is_float, const float* frequencies, int head_dim, int hq,
                                       int hk, float eps, int M, int N, int K, int* dev_status, void* stream);

/* The reference's own cross-entropy dataflow, for callers that want the logits:
 * coda_b200_gemm_lse_logits stores logits = bf16(acc * rstd) (rstd may be NULL)
 * plus the LSE partials; coda_b200_lse_reduce folds the partials into lse[M];
 * coda_b200_cross_entropy_fwd_bwd then overwrites the logits in place with
 * exp(logit - lse) - onehot (+0 for ignored rows) and writes losses[M] = lse -
 * logit[target] (0 if ignored; targets outside [0, N) leave losses untouched).
 * Replace `coda::_gemm_lse_epi` + `logsumexp(partials)` and
 * `cross_entropy_fwd_bwd` (coda/core/gemm/functional.py:337-389;
 * coda/core/elementwise/functional.py:221-311, kernel coda/core/elementwise/cross_entropy.py:18-131). */
int coda_b200_gemm_lse_logits(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                              int64_t b_stride_n, const float* rstd, void* logits, int64_t ld_logits, float* part_max,
                              float* part_sum, int M, int N, int K, int* dev_status, void* stream);
int coda_b200_lse_reduce(const float* part_max, const float* part_sum, int tiles_n, float* lse, int M, void* stream);
int coda_b200_cross_entropy_fwd_bwd(void* logits, int64_t ld, const float* lse, const int32_t* target, int ignore_index,
                                    float* losses, int M, int N, void* stream);

/* GEMMs that sit between the fused-linear operators inside a transformer layer.
 *
 * coda_b200_gemm_residual_partial_rmsnorm: pre = A @ B + C, post = pre * weight[col],
 * rstd[M] = rsqrt(mean_col(pre^2) + eps) from the unrounded sum; C may alias pre or
 * post.  part_sq is fp32 scratch [M, ceil(N / 256)].  Replaces
 * `coda::_gemm_residual_partial_rmsnorm_epi` (coda/core/gemm/functional.py:573-652).
 *
 * coda_b200_gemm_swiglu_bwd_zdz: acc = A @ B is d(postact) [M, N]; Z is the stored
 * SwiGLU preact [M, 2N] (gate, up interleaved; may alias dZ).  Writes dZ =
 * dswiglu(Z, acc) [M, 2N], postact = silu(gate) * up [M, N] and zdz[M] = scale *
 * sum_col(Z * dZ).  part_zdz is fp32 scratch [M, ceil(N / 256)].  Replaces
 * `coda::_gemm_swiglu_bwd_zdz_epi(_scaled)` (coda/core/gemm/functional.py:827-952).
 *
 * coda_b200_gemm_residual_partial_rmsnorm_bwd: y = alpha * (A @ B) (alpha: device
 * scalar or NULL), n = pre * rstd[row]; dX = (y * weight[col] - n * zdz[row]) *
 * rstd[row], added to dX's contents if accumulate != 0; normed = n * weight[col]
 * (may alias pre); dW[N] fp32 = sum_row(y * n).  part_dw is fp32 scratch
 * [ceil(M / 32), N].  Replaces `coda::_gemm_residual_partial_rmsnorm_bwd_epi_{store,accum}`
 * (coda/core/gemm/functional.py:655-824). */
int coda_b200_gemm_residual_partial_rmsnorm(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                            int64_t b_stride_k, int64_t b_stride_n, const void* C, int64_t ldc,
                                            const void* weight, float eps, void* pre, int64_t ld_pre, void* post,
                                            int64_t ld_post, float* rstd, float* part_sq, int M, int N, int K, int* dev_status,
                                            void* stream);
int coda_b200_gemm_swiglu_bwd_zdz(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                                  int64_t b_stride_n, const void* Z, int64_t ldz, void* dZ, int64_t ld_dz, void* postact,
                                  int64_t ld_post, float* zdz, float scale, float* part_zdz, int M, int N, int K,
                                  int* dev_status, void* stream);
int coda_b200_gemm_residual_partial_rmsnorm_bwd(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                                int64_t b_stride_k, int64_t b_stride_n, const void* weight, const void* pre,
                                                int64_t ld_pre, const float* zdz, const float* rstd, const float* alpha,
                                                void* dX, int64_t ld_dx, int accumulate, float* dW, void* normed,
                                                int64_t ld_normed, float* part_dw, int M, int N, int K, int* dev_status,
                                                void* stream);

/* Pieces the fused Llama-3 layer blocks add on top of the GEMMs above.
 *
 * coda_b200_partial_rmsnorm: h = x * weight[col], rstd[M] = rsqrt(mean(x^2) + eps) and,
 * if residual != NULL, a copy of x, from one read of x [M, N].  Replaces
 * `partial_rmsnorm` (imported by coda/kernels/blocks/llama3.py:10-13).
 *
 * coda_b200_gemm_rmsnorm_rope: D = rotate((A @ B) * rstd[row]) over every adjacent
 * column pair with `frequencies` fp32 [N] ((hi, lo) turns; zero for v columns) and
 * `positions` [M]; rstd may be NULL.  Replaces `coda::_gemm_rope_epi` /
 * `coda::_gemm_rmsnorm_rope_epi` (coda/core/gemm/functional.py:955-1062).
 *
 * coda_b200_rope_bwd_zdz: dz = R^T dy for the same angles and zdz[M] = scale *
 * sum_col(y * dy).  Replaces `rope_bwd_zdz` (coda/core/elementwise/zdz.py:21).
 *
 * coda_b200_gemm_rmsnorm_lse_zdz / coda_b200_lse_finalize_zdz: the LSE GEMM and its
 * per-row reduction with one more partial, from which zdz[M] = sum_col(logit *
 * dlogit) (0 for ignored rows) is formed without touching the [M, N] buffer.
 * Replace `gemm_rmsnorm_cross_entropy_fwd_bwd(..., return_zdz=True)`
 * (imported by coda/kernels/blocks/llama3.py:23-26). */
int coda_b200_partial_rmsnorm(const void* x, int64_t ldx, const void* weight, float eps, void* residual, int64_t ld_res, void* h,
                              int64_t ld_h, float* rstd, int M, int N, void* stream);
int coda_b200_gemm_rmsnorm_rope(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                                int64_t b_stride_n, const float* rstd, void* D, int64_t ldd, const void* positions,
                                int pos_is_float, const float* frequencies, int M, int N, int K, int* dev_status, void* stream);
int coda_b200_rope_bwd_zdz(const void* y, int64_t ldy, const void* dy, int64_t ld_dy, const void* positions, int pos_is_float,
                           const float* frequencies, float scale, void* dz, int64_t ld_dz, float* zdz, int M, int N, void* stream);
int coda_b200_gemm_rmsnorm_lse_zdz(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                                   int64_t b_stride_n, const float* rstd, void* P, int64_t ldp, float* part_max, float* part_sum,
                                   float* part_sz, const int32_t* target, float* target_logit, int M, int N, int K,
                                   int* dev_status, void* stream);
int coda_b200_lse_finalize_zdz(const float* part_max, const float* part_sum, const float* part_sz, int tiles_n,
                               const int32_t* target, const float* target_logit, int ignore_index, float* lse, float* losses,
                               float* zdz, int M, void* stream);

/* Size in bytes of the scratch buffer coda_b200_qknorm_rope_bwd needs. */
int64_t coda_b200_qknorm_rope_bwd_scratch_bytes(int M, int head_dim);

/* Backward of the q,k epilogue.  dq [M, hq*d], dk [M, hk*d] (row strides ld_dq,
 * ld_dk); preact, mean_sq as saved by the forward.  Writes grad_pre into
 * grad[:, :(hq+hk)*d] and, if dv != NULL, copies dv [M, nv] into
 * grad[:, (hq+hk)*d:], so that one GEMM over `grad` yields dx and one yields
 * dW.  dgamma fp32 [2*d].  `scratch` holds per-block partial sums of dgamma.
 * Every leading dimension must cover its row (ld_dq >= hq*d, ld_dk >= hk*d,
 * ld_dv >= nv, ld_pre >= (hq+hk)*d, ld_grad >= (hq+hk)*d + nv): rows are read
 * and written with 16-byte accesses, a short stride returns CODA_B200_EARG.
 * Replaces `qknorm_rope_bwd` (coda/core/elementwise/functional.py:314-456;
 * kernel coda/core/elementwise/rope.py:19-253). */
int coda_b200_qknorm_rope_bwd(const void* dq, int64_t ld_dq, const void* dk, int64_t ld_dk, const void* dv, int64_t ld_dv,
                              int nv, const void* preact, int64_t ld_pre, const float* mean_sq, const void* gamma,
                              const void* positions, int pos_is_float, const float* frequencies, int head_dim, int hq,
                              int hk, float eps, void* grad, int64_t ld_grad, float* dgamma, void* scratch,
                              int64_t scratch_bytes, int M, void* stream);

/* Same computation and arguments as coda_b200_qknorm_rope_bwd, minus the
 * scratch buffer.  This entry point has no counterpart in the reference; it
 * exists for hosts that cannot supply a workspace: a bare C / ctypes caller
 * that owns only its input and output arrays, or a process that took all of
 * its device memory at start-up and may not call cudaMalloc afterwards.  The
 * per-block dgamma partials go to a 1 MiB array built into the library (held by
 * every GPU that loads it until the process exits), so
 *   - M may be at most 16384 rows per call; larger M returns CODA_B200_EARG;
 *   - it calls no cudaMalloc / cudaFree or any other allocating routine;
 *   - the first call on each device looks up the array's device address (with
 *     that device current); make that first call before any stream capture;
 *   - all calls share the array, which keeps the previous call's contents (each
 *     call overwrites every entry it later reads, so nothing needs clearing);
 *     two calls that overlap on the GPU (different streams) race on it;
 *   - the array used is the current device's: a call whose `grad` buffer lives
 *     on another GPU returns CODA_B200_EARG instead of launching. */
int coda_b200_qknorm_rope_bwd_noalloc(const void* dq, int64_t ld_dq, const void* dk, int64_t ld_dk, const void* dv,
                                      int64_t ld_dv, int nv, const void* preact, int64_t ld_pre, const float* mean_sq,
                                      const void* gamma, const void* positions, int pos_is_float, const float* frequencies,
                                      int head_dim, int hq, int hk, float eps, void* grad, int64_t ld_grad, float* dgamma,
                                      int M, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CODA_B200_H_ */
