// C-ABI entry points for the GEMMs with fused SwiGLU, log-sum-exp and
// QK-norm + RoPE epilogues.  See include/coda_b200.h for the contract.
#include "../../include/coda_b200.h"
#include "gemm_host.cuh"

using namespace cb;

namespace {
constexpr int kTileN = 256;  // column-tile width of every fused GEMM in this file

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
}  // namespace

namespace {
template <class Epi>
int run_gated(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k, int64_t b_stride_n,
              const float* rstd, void* preact, int64_t ld_pre, void* postact, int64_t ld_post, int M, int N, int K, int* dev_status,
              void* stream) {
  if (!A || !B || !preact || !postact) return fail(kBadArgument, "NULL matrix pointer");
  if (N % 16 != 0) return fail(kBadArgument, "the gated GEMM needs N (= 2F) to be a multiple of 16");
  if (ld_pre % 8 != 0 || ld_post % 8 != 0 || ld_pre < N || ld_post < N / 2)
    return fail(kBadArgument, "output leading dimensions must be multiples of 8 and cover the row");
  if (!aligned16(preact) || !aligned16(postact)) return fail(kBadArgument, "outputs must be 16-byte aligned");
  typename Epi::Params ep;
  ep.preact = static_cast<__nv_bfloat16*>(preact);
  ep.ld_pre = ld_pre;
  ep.postact = static_cast<__nv_bfloat16*>(postact);
  ep.ld_post = ld_post;
  ep.row_scale = rstd;
  int rc = make_tmap_out(&ep.tm_pre, ep.preact, N, M, ld_pre, 32);
  if (rc == kOk) rc = make_tmap_out(&ep.tm_post, ep.postact, N / 2, M, ld_post, 16);
  if (rc != kOk) return rc;
  Operand a{A, a_stride_m, a_stride_k};
  Operand b{B, b_stride_n, b_stride_k};
  return launch_gemm<Epi, 0>(a, b, M, N, K, ep, dev_status, static_cast<cudaStream_t>(stream));
}
}  // namespace

extern "C" int coda_b200_gemm_rmsnorm_swiglu(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                             int64_t b_stride_k, int64_t b_stride_n, const float* rstd, void* preact,
                                             int64_t ld_pre, void* postact, int64_t ld_post, int M, int N, int K,
                                             int* dev_status, void* stream) {
  return run_gated<EpiSwiGLU>(A, a_stride_m, a_stride_k, B, b_stride_k, b_stride_n, rstd, preact, ld_pre, postact, ld_post, M, N, K,
                              dev_status, stream);
}

extern "C" int coda_b200_gemm_sigmoid_glu(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                                          int64_t b_stride_n, void* preact, int64_t ld_pre, void* postact, int64_t ld_post, int M,
                                          int N, int K, int* dev_status, void* stream) {
  return run_gated<EpiSigmoidGLU>(A, a_stride_m, a_stride_k, B, b_stride_k, b_stride_n, nullptr, preact, ld_pre, postact, ld_post, M,
                                  N, K, dev_status, stream);
}

extern "C" int coda_b200_gemm_swiglu(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                     int64_t b_stride_k, int64_t b_stride_n, void* preact, int64_t ld_pre, void* postact,
                                     int64_t ld_post, int M, int N, int K, int* dev_status, void* stream) {
  return coda_b200_gemm_rmsnorm_swiglu(A, a_stride_m, a_stride_k, B, b_stride_k, b_stride_n, nullptr, preact, ld_pre, postact,
                                       ld_post, M, N, K, dev_status, stream);
}

extern "C" int coda_b200_lse_tiles(int N) { return (N + kTileN - 1) / kTileN; }

extern "C" int coda_b200_gemm_rmsnorm_lse_zdz(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                              int64_t b_stride_k, int64_t b_stride_n, const float* rstd, void* P, int64_t ldp,
                                              float* part_max, float* part_sum, float* part_sz, const int32_t* target,
                                              float* target_logit, int M, int N, int K, int* dev_status, void* stream) {
  if (!A || !B || !part_max || !part_sum || !target || !target_logit) return fail(kBadArgument, "NULL pointer");
  if (N % 8 != 0) return fail(kBadArgument, "N must be a multiple of 8");
  Operand a{A, a_stride_m, a_stride_k};
  Operand b{B, b_stride_n, b_stride_k};
  const int tiles_n = coda_b200_lse_tiles(N);
  if (P != nullptr) {
    if (!aligned16(P) || ldp % 8 != 0 || ldp < N) return fail(kBadArgument, "P must be 16-byte aligned with ldp % 8 == 0, ldp >= N");
    EpiLse<kLseStoreProbs>::Params ep;
    ep.P = static_cast<__nv_bfloat16*>(P);
    ep.ldp = ldp;
    ep.part_max = part_max;
    ep.part_sum = part_sum;
    ep.tiles_n = tiles_n;
    ep.target = target;
    ep.target_logit = target_logit;
    ep.row_scale = rstd;
    ep.part_sz = part_sz;
    const int rc = make_tmap_out(&ep.tm_p, ep.P, N, M, ldp);
    if (rc != kOk) return rc;
    return launch_gemm<EpiLse<kLseStoreProbs>, 0>(a, b, M, N, K, ep, dev_status, static_cast<cudaStream_t>(stream));
  }
  EpiLse<kLseStoreNone>::Params ep;
  memset(&ep.tm_p, 0, sizeof(ep.tm_p));
  ep.P = nullptr;
  ep.ldp = 0;
  ep.part_max = part_max;
  ep.part_sum = part_sum;
  ep.tiles_n = tiles_n;
  ep.target = target;
  ep.target_logit = target_logit;
  ep.row_scale = rstd;
  ep.part_sz = part_sz;
  return launch_gemm<EpiLse<kLseStoreNone>, 0>(a, b, M, N, K, ep, dev_status, static_cast<cudaStream_t>(stream));
}

extern "C" int coda_b200_gemm_rmsnorm_lse(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                          int64_t b_stride_k, int64_t b_stride_n, const float* rstd, void* P, int64_t ldp,
                                          float* part_max, float* part_sum, const int32_t* target, float* target_logit, int M,
                                          int N, int K, int* dev_status, void* stream) {
  return coda_b200_gemm_rmsnorm_lse_zdz(A, a_stride_m, a_stride_k, B, b_stride_k, b_stride_n, rstd, P, ldp, part_max, part_sum,
                                        nullptr, target, target_logit, M, N, K, dev_status, stream);
}

extern "C" int coda_b200_gemm_lse(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                                  int64_t b_stride_n, void* P, int64_t ldp, float* part_max, float* part_sum,
                                  const int32_t* target, float* target_logit, int M, int N, int K, int* dev_status,
                                  void* stream) {
  return coda_b200_gemm_rmsnorm_lse(A, a_stride_m, a_stride_k, B, b_stride_k, b_stride_n, nullptr, P, ldp, part_max, part_sum,
                                    target, target_logit, M, N, K, dev_status, stream);
}

extern "C" int coda_b200_gemm_lse_logits(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                         int64_t b_stride_k, int64_t b_stride_n, const float* rstd, void* logits, int64_t ld_logits,
                                         float* part_max, float* part_sum, int M, int N, int K, int* dev_status, void* stream) {
  if (!A || !B || !logits || !part_max || !part_sum) return fail(kBadArgument, "NULL pointer");
  if (N % 8 != 0) return fail(kBadArgument, "N must be a multiple of 8");
  if (!aligned16(logits) || ld_logits % 8 != 0 || ld_logits < N)
    return fail(kBadArgument, "logits must be 16-byte aligned with ld % 8 == 0, ld >= N");
  EpiLse<kLseStoreLogits>::Params ep;
  ep.P = static_cast<__nv_bfloat16*>(logits);
  ep.ldp = ld_logits;
  ep.part_max = part_max;
  ep.part_sum = part_sum;
  ep.tiles_n = coda_b200_lse_tiles(N);
  ep.target = nullptr;
  ep.target_logit = nullptr;
  ep.row_scale = rstd;
  ep.part_sz = nullptr;
  const int rc = make_tmap_out(&ep.tm_p, ep.P, N, M, ld_logits);
  if (rc != kOk) return rc;
  Operand a{A, a_stride_m, a_stride_k};
  Operand b{B, b_stride_n, b_stride_k};
  return launch_gemm<EpiLse<kLseStoreLogits>, 0>(a, b, M, N, K, ep, dev_status, static_cast<cudaStream_t>(stream));
}

namespace {
template <int kHD>
int run_qknorm(const Operand& a, const Operand& b, void* qk, int64_t ld_qk, void* preact, int64_t ld_pre, void* v, int64_t ld_v,
               float* mean_sq, const void* gamma, const void* positions, int pos_is_float, const float* frequencies, int hq,
               int hk, float eps, const float* rstd, int M, int N, int K, int* dev_status, void* stream) {
  typename EpiQKNormRope<kHD>::Params ep;
  ep.qk = static_cast<__nv_bfloat16*>(qk);
  ep.ld_qk = ld_qk;
  ep.preact = static_cast<__nv_bfloat16*>(preact);
  ep.ld_pre = ld_pre;
  ep.v = static_cast<__nv_bfloat16*>(v);
  ep.ld_v = ld_v;
  ep.mean_sq = mean_sq;
  ep.gamma = static_cast<const __nv_bfloat16*>(gamma);
  ep.positions = positions;
  ep.pos_is_float = pos_is_float;
  ep.freq = frequencies;
  ep.hq = hq;
  ep.hk = hk;
  ep.eps = eps;
  ep.row_scale = rstd;
  const long long size_qk = static_cast<long long>(hq + hk) * kHD;
  int rc = make_tmap_out(&ep.tm_qk, ep.qk, size_qk, M, ld_qk);
  if (rc == kOk) rc = make_tmap_out(&ep.tm_pre, ep.preact, size_qk, M, ld_pre);
  if (rc == kOk && N > size_qk) rc = make_tmap_out(&ep.tm_v, ep.v, N - size_qk, M, ld_v);
  else if (rc == kOk) memset(&ep.tm_v, 0, sizeof(ep.tm_v));
  if (rc != kOk) return rc;
  return launch_gemm<EpiQKNormRope<kHD>, 0>(a, b, M, N, K, ep, dev_status, static_cast<cudaStream_t>(stream));
}
}  // namespace

extern "C" int coda_b200_gemm_rmsnorm_qknorm_rope(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                                  int64_t b_stride_k, int64_t b_stride_n, const float* rstd, void* qk,
                                                  int64_t ld_qk, void* preact, int64_t ld_pre, void* v, int64_t ld_v,
                                                  float* mean_sq, const void* gamma, const void* positions, int pos_is_float,
                                                  const float* frequencies, int head_dim, int hq, int hk, float eps, int M,
                                                  int N, int K, int* dev_status, void* stream) {
  if (!A || !B || !qk || !preact || !mean_sq || !gamma || !positions || !frequencies)
    return fail(kBadArgument, "NULL pointer");
  if (head_dim != 64 && head_dim != 128) return fail(kBadArgument, "head_dim must be 64 or 128");
  if (hq < 0 || hk < 0 || hq + hk <= 0) return fail(kBadArgument, "bad head counts");
  const long long size_qk = static_cast<long long>(hq + hk) * head_dim;
  if (N < size_qk || N % head_dim != 0) return fail(kBadArgument, "N must hold the q and k heads and be a multiple of head_dim");
  if (N > size_qk && v == nullptr) return fail(kBadArgument, "v output required when N has v columns");
  if (ld_qk % 8 || ld_pre % 8 || ld_qk < size_qk || ld_pre < size_qk) return fail(kBadArgument, "bad qk / preact leading dimension");
  if (v != nullptr && (ld_v % 8 || ld_v < N - size_qk || !aligned16(v))) return fail(kBadArgument, "bad v leading dimension / alignment");
  if (!aligned16(qk) || !aligned16(preact)) return fail(kBadArgument, "outputs must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(frequencies) & 15u) || (reinterpret_cast<uintptr_t>(gamma) & 15u))
    return fail(kBadArgument, "frequencies and gamma must be 16-byte aligned");
  Operand a{A, a_stride_m, a_stride_k};
  Operand b{B, b_stride_n, b_stride_k};
  if (head_dim == 128)
    return run_qknorm<128>(a, b, qk, ld_qk, preact, ld_pre, v, ld_v, mean_sq, gamma, positions, pos_is_float, frequencies, hq,
                           hk, eps, rstd, M, N, K, dev_status, stream);
  return run_qknorm<64>(a, b, qk, ld_qk, preact, ld_pre, v, ld_v, mean_sq, gamma, positions, pos_is_float, frequencies, hq, hk,
                        eps, rstd, M, N, K, dev_status, stream);
}

extern "C" int coda_b200_gemm_qknorm_rope(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                          int64_t b_stride_k, int64_t b_stride_n, void* qk, int64_t ld_qk, void* preact,
                                          int64_t ld_pre, void* v, int64_t ld_v, float* mean_sq, const void* gamma,
                                          const void* positions, int pos_is_float, const float* frequencies, int head_dim,
                                          int hq, int hk, float eps, int M, int N, int K, int* dev_status, void* stream) {
  return coda_b200_gemm_rmsnorm_qknorm_rope(A, a_stride_m, a_stride_k, B, b_stride_k, b_stride_n, nullptr, qk, ld_qk, preact,
                                            ld_pre, v, ld_v, mean_sq, gamma, positions, pos_is_float, frequencies, head_dim, hq,
                                            hk, eps, M, N, K, dev_status, stream);
}
