// C-ABI entry points for the plain and sigmoid GEMMs, plus library-wide
// option / error plumbing.  See include/coda_b200.h for the contract.
#include "../../include/coda_b200.h"
#include "gemm_host.cuh"

using namespace cb;

extern "C" int coda_b200_version(void) { return 1; }

extern "C" const char* coda_b200_last_error(void) { return g_last_error.c_str(); }

extern "C" int coda_b200_set_option(const char* name, int value) {
  if (name == nullptr) return fail(kBadArgument, "option name is NULL");
  Options& o = options();
  if (!strcmp(name, "cta_group")) {
    if (value != 1 && value != 2) return fail(kBadArgument, "cta_group must be 1 or 2");
    o.cta_group = value;
  } else if (!strcmp(name, "group_m")) {
    if (value < 0) return fail(kBadArgument, "group_m must be >= 0");
    o.group_m = value;
  } else if (!strcmp(name, "max_ctas")) {
    if (value < 0) return fail(kBadArgument, "max_ctas must be >= 0");
    o.max_ctas = value;
  } else if (!strcmp(name, "tile_n")) {
    if (value != 0 && value != 64 && value != 128 && value != 256) return fail(kBadArgument, "tile_n must be 0, 64, 128 or 256");
    o.tile_n = value;
  } else if (!strcmp(name, "epi_tma")) {
    if (value != 0 && value != 1) return fail(kBadArgument, "epi_tma must be 0 or 1");
    o.epi_tma = value;
  } else if (!strcmp(name, "split_tail")) {
    if (value != 0 && value != 1) return fail(kBadArgument, "split_tail must be 0 or 1");
    o.split_tail = value;
  } else if (!strcmp(name, "probe_ld_kb") || !strcmp(name, "probe_st_kb")) {
    if (value < 0 || value > 256) return fail(kBadArgument, "probe traffic must be between 0 and 256 KB per k-block");
    (name[6] == 'l' ? o.probe_ld_kb : o.probe_st_kb) = value;
  } else {
    return fail(kBadArgument, std::string("unknown option: ") + name);
  }
  return kOk;
}

namespace {
template <typename OutT, Act kAct>
int run_store(const void* A, int64_t asm_, int64_t ask, const void* B, int64_t bsk, int64_t bsn, const void* C, int64_t ldc,
              int c_is_fp32, void* D, int64_t ldd, int M, int N, int K, const float* alpha, int* dev_status, void* stream,
              void* workspace = nullptr, int64_t workspace_bytes = 0) {
  if (D == nullptr || A == nullptr || B == nullptr) return fail(kBadArgument, "NULL matrix pointer");
  if ((reinterpret_cast<uintptr_t>(D) & 15u) != 0) return fail(kBadArgument, "D must be 16-byte aligned");
  if (N % 8 != 0 || ldd % 8 != 0 || ldd < N) return fail(kBadArgument, "N and ldd must be multiples of 8 with ldd >= N");
  if (C != nullptr && ((reinterpret_cast<uintptr_t>(C) & 15u) != 0 || ldc % 8 != 0 || ldc < N))
    return fail(kBadArgument, "C must be 16-byte aligned with ldc a multiple of 8 and >= N");
  typename EpiStore<OutT, kAct>::Params ep;
  ep.D = static_cast<OutT*>(D);
  ep.ldd = ldd;
  ep.alpha = alpha;
  ep.C = C;
  ep.ldc = ldc;
  ep.c_is_fp32 = c_is_fp32;
  if (kAct == Act::kNone && C == nullptr && workspace != nullptr) {  // a plain GEMM may be split along K
    if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return fail(kBadArgument, "workspace must be 16-byte aligned");
    ep.ws = static_cast<float*>(workspace);
    ep.ws_bytes = workspace_bytes;
  }
  int rc = make_tmap_out(&ep.tm_d, ep.D, N, M, ldd);
  if (rc != kOk) return rc;
  Operand a{A, asm_, ask};
  Operand b{B, bsn, bsk};
  return launch_gemm<EpiStore<OutT, kAct>, 3, 2>(a, b, M, N, K, ep, dev_status, static_cast<cudaStream_t>(stream));
}
}  // namespace

extern "C" int coda_b200_gemm_add(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                                  int64_t b_stride_n, const void* C, int64_t ldc, int c_is_fp32, void* D, int64_t ldd,
                                  int d_is_fp32, int M, int N, int K, const float* alpha, int* dev_status, void* stream) {
  if (d_is_fp32)
    return run_store<float, Act::kNone>(A, a_stride_m, a_stride_k, B, b_stride_k, b_stride_n, C, ldc, c_is_fp32, D, ldd, M, N, K,
                                        alpha, dev_status, stream);
  return run_store<__nv_bfloat16, Act::kNone>(A, a_stride_m, a_stride_k, B, b_stride_k, b_stride_n, C, ldc, c_is_fp32, D, ldd, M, N,
                                              K, alpha, dev_status, stream);
}

extern "C" int64_t coda_b200_gemm_workspace_bytes(int M, int N, int K) {
  if (M <= 0 || N <= 128 || K <= 0) return 0;  // narrow outputs keep their narrow tiles
  const LaunchOptions opt = launch_options();
  if (opt.split_tail == 0) return 0;
  const int group = opt.cta_group == 2 ? 2 : 1;
  const int tile_m = kBlockM * group, clusters = full_clusters(opt, group);
  const long long tiles = static_cast<long long>((M + tile_m - 1) / tile_m) * ((N + 255) / 256);
  int tail = 0;
  if (plan_tail_split(tiles, (K + kBlockK - 1) / kBlockK, clusters, &tail) <= 1) return 0;
  return split_workspace_bytes(clusters, tile_m, 256);
}

extern "C" int coda_b200_gemm_ws(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                                 int64_t b_stride_n, void* D, int64_t ldd, int d_is_fp32, int M, int N, int K, const float* alpha,
                                 void* workspace, int64_t workspace_bytes, int* dev_status, void* stream) {
  if (workspace_bytes < 0) return fail(kBadArgument, "workspace_bytes must not be negative");
  if (d_is_fp32)
    return run_store<float, Act::kNone>(A, a_stride_m, a_stride_k, B, b_stride_k, b_stride_n, nullptr, 0, 0, D, ldd, M, N, K, alpha,
                                        dev_status, stream, workspace, workspace_bytes);
  return run_store<__nv_bfloat16, Act::kNone>(A, a_stride_m, a_stride_k, B, b_stride_k, b_stride_n, nullptr, 0, 0, D, ldd, M, N, K,
                                              alpha, dev_status, stream, workspace, workspace_bytes);
}

extern "C" int coda_b200_gemm(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                              int64_t b_stride_n, void* D, int64_t ldd, int d_is_fp32, int M, int N, int K,
                              const float* alpha, int* dev_status, void* stream) {
  return coda_b200_gemm_add(A, a_stride_m, a_stride_k, B, b_stride_k, b_stride_n, nullptr, 0, 0, D, ldd, d_is_fp32, M, N, K, alpha,
                            dev_status, stream);
}

extern "C" int coda_b200_gemm_sigmoid(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                      int64_t b_stride_k, int64_t b_stride_n, void* D, int64_t ldd, int d_is_fp32, int M,
                                      int N, int K, int* dev_status, void* stream) {
  if (d_is_fp32)
    return run_store<float, Act::kSigmoid>(A, a_stride_m, a_stride_k, B, b_stride_k, b_stride_n, nullptr, 0, 0, D, ldd, M, N, K,
                                           nullptr, dev_status, stream);
  return run_store<__nv_bfloat16, Act::kSigmoid>(A, a_stride_m, a_stride_k, B, b_stride_k, b_stride_n, nullptr, 0, 0, D, ldd, M, N,
                                                 K, nullptr, dev_status, stream);
}

extern "C" int coda_b200_gemm_dsigmoid_dgrad(const void* out, int64_t ld_out, const void* dout, int64_t ld_dout, const void* W,
                                             int64_t ldw, void* G, int64_t ld_g, void* dx, int64_t ld_dx, int M, int N, int K,
                                             int* dev_status, void* stream) {
  // dx[M, K] = G[M, N] @ W[N, K] with G = dout * out * (1 - out) formed by the GEMM's own transform warps.
  if (!out || !dout || !W || !G || !dx) return fail(kBadArgument, "NULL pointer");
  if (M <= 0 || N <= 0 || K <= 0) return fail(kBadArgument, "extents must be positive");
  if (dev_status == nullptr) return fail(kBadArgument, "device status word is required");
  if (N % 8 || K % 8 || ld_out % 8 || ld_dout % 8 || ld_g % 8 || ld_dx % 8 || ldw % 8)
    return fail(kBadArgument, "extents and leading dimensions must be multiples of 8");
  if (ld_out < N || ld_dout < N || ld_g < N || ld_dx < K || ldw < K) return fail(kBadArgument, "a leading dimension is smaller than its row");
  for (const void* p : {out, dout, W, static_cast<const void*>(G), static_cast<const void*>(dx)})
    if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) return fail(kBadArgument, "pointers must be 16-byte aligned");
  const LaunchOptions opt = launch_options();
  if (opt.cta_group != 2) return fail(kBadArgument, "the fused sigmoid-gradient GEMM is built for CTA pairs only (cta_group = 2)");
  using Epi = EpiStore<__nv_bfloat16, Act::kNone>;
  Epi::Params ep;
  ep.D = static_cast<__nv_bfloat16*>(dx);
  ep.ldd = ld_dx;
  ep.alpha = nullptr;
  ep.C = nullptr;
  ep.ldc = 0;
  ep.c_is_fp32 = 0;
  ep.use_tma = opt.epi_tma;
  int rc = make_tmap_out(&ep.tm_d, ep.D, K, M, ld_dx);
  if (rc != kOk) return rc;
  ProDSigmoid::Params pp;
  rc = make_tmap_bf16(&pp.tm_dout, dout, N, M, ld_dout, kBlockM);  // same geometry as the A operand (`out`)
  if (rc != kOk) return rc;
  pp.G = static_cast<__nv_bfloat16*>(G);
  pp.ld_g = ld_g;
  // A slot <- `out` [M, N] by TMA, rewritten in place; operand B = W[N, K] read MN-major (contiguous along the output
  // dimension K); the contraction runs over N
  return launch_gemm_cfg<2, 256, false, true, Epi, ProDSigmoid>(out, ld_out, W, ldw, M, /*N=*/K, /*K=*/N, ep, dev_status,
                                                                static_cast<cudaStream_t>(stream), opt, pp);
}
