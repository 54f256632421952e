// C-ABI entry points for the GEMMs between the fused-linear operators of a transformer layer: residual add with
// deferred RMSNorm (forward and backward) and the down-projection dgrad through SwiGLU.  See include/coda_b200.h.
#include "../../include/coda_b200.h"
#include "epilogues_block.cuh"
#include "gemm_host.cuh"

using namespace cb;

namespace {
constexpr int kTileN = 256;
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int launch_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(kCudaError, std::string(what) + ": " + cudaGetErrorString(e));
  return kOk;
}

// out[row] = f(sum_t partials[row, t]): one warp per row.  mode 0: scale * sum;  mode 1: rsqrt(scale * sum + eps).
__global__ void __launch_bounds__(256) row_reduce_kernel(const float* __restrict__ partials, int tiles, float* __restrict__ out,
                                                         int M, float scale, float eps, int mode) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= M) return;
  float s = 0.f;
  for (int t = lane; t < tiles; t += 32) s += partials[static_cast<long long>(row) * tiles + t];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) out[row] = mode == 0 ? s * scale : rsqrtf(s * scale + eps);
}

// out[c] = sum_b partials[b, c]: 32 columns x 8 row-lanes per block.
__global__ void __launch_bounds__(256) col_reduce_kernel(const float* __restrict__ partials, int nrows, int width,
                                                         float* __restrict__ out) {
  __shared__ float red[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (c < width)
    for (int b = ry; b < nrows; b += 8) s += partials[static_cast<long long>(b) * width + c];
  red[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && c < width) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) t += red[j][cx];
    out[c] = t;
  }
}
}  // namespace

extern "C" int coda_b200_gemm_residual_partial_rmsnorm(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                                       int64_t b_stride_k, int64_t b_stride_n, const void* C, int64_t ldc,
                                                       const void* weight, float eps, void* pre, int64_t ld_pre, void* post,
                                                       int64_t ld_post, float* rstd, float* part_sq, int M, int N, int K,
                                                       int* dev_status, void* stream) {
  if (!A || !B || !C || !weight || !pre || !post || !rstd || !part_sq) return fail(kBadArgument, "NULL pointer");
  if (N % 8 || ldc % 8 || ld_pre % 8 || ld_post % 8 || ldc < N || ld_pre < N || ld_post < N)
    return fail(kBadArgument, "N and leading dimensions must be multiples of 8 and cover the row");
  if (!aligned16(C) || !aligned16(pre) || !aligned16(post) || !aligned16(weight)) return fail(kBadArgument, "pointers must be 16-byte aligned");
  EpiResidualNorm::Params ep;
  ep.C = static_cast<const __nv_bfloat16*>(C);
  ep.ldc = ldc;
  ep.pre = static_cast<__nv_bfloat16*>(pre);
  ep.ld_pre = ld_pre;
  ep.post = static_cast<__nv_bfloat16*>(post);
  ep.ld_post = ld_post;
  ep.weight = static_cast<const __nv_bfloat16*>(weight);
  ep.part_sq = part_sq;
  ep.tiles_n = (N + kTileN - 1) / kTileN;
  int rc = make_tmap_out(&ep.tm_pre, ep.pre, N, M, ld_pre);
  if (rc == kOk) rc = make_tmap_out(&ep.tm_post, ep.post, N, M, ld_post);
  if (rc == kOk) rc = make_tmap_out(&ep.tm_c, ep.C, N, M, ldc);
  if (rc != kOk) return rc;
  Operand a{A, a_stride_m, a_stride_k};
  Operand b{B, b_stride_n, b_stride_k};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = launch_gemm<EpiResidualNorm, 3>(a, b, M, N, K, ep, dev_status, st);
  if (rc != kOk) return rc;
  row_reduce_kernel<<<(M + 7) / 8, 256, 0, st>>>(part_sq, ep.tiles_n, rstd, M, 1.0f / static_cast<float>(N), eps, 1);
  return launch_check("rstd reduce launch");
}

extern "C" int coda_b200_gemm_rmsnorm_rope(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B, int64_t b_stride_k,
                                           int64_t b_stride_n, const float* rstd, void* D, int64_t ldd, const void* positions,
                                           int pos_is_float, const float* frequencies, int M, int N, int K, int* dev_status,
                                           void* stream) {
  if (!A || !B || !D || !positions || !frequencies) return fail(kBadArgument, "NULL pointer");
  if (N % 8 || ldd % 8 || ldd < N || !aligned16(D)) return fail(kBadArgument, "D must be 16-byte aligned, N and ldd multiples of 8");
  if (reinterpret_cast<uintptr_t>(frequencies) & 7u) return fail(kBadArgument, "frequencies must be 8-byte aligned");
  EpiRope::Params ep;
  ep.D = static_cast<__nv_bfloat16*>(D);
  ep.ldd = ldd;
  ep.row_scale = rstd;
  ep.positions = positions;
  ep.pos_is_float = pos_is_float;
  ep.freq = frequencies;
  const int rc = make_tmap_out(&ep.tm_d, ep.D, N, M, ldd);
  if (rc != kOk) return rc;
  Operand a{A, a_stride_m, a_stride_k};
  Operand b{B, b_stride_n, b_stride_k};
  return launch_gemm<EpiRope, 0>(a, b, M, N, K, ep, dev_status, static_cast<cudaStream_t>(stream));
}

extern "C" int coda_b200_gemm_swiglu_bwd_zdz(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                             int64_t b_stride_k, int64_t b_stride_n, const void* Z, int64_t ldz, void* dZ,
                                             int64_t ld_dz, void* postact, int64_t ld_post, float* zdz, float scale,
                                             float* part_zdz, int M, int N, int K, int* dev_status, void* stream) {
  if (!A || !B || !Z || !dZ || !postact || !zdz || !part_zdz) return fail(kBadArgument, "NULL pointer");
  if (N % 8 || ldz % 8 || ld_dz % 8 || ld_post % 8 || ldz < 2 * N || ld_dz < 2 * N || ld_post < N)
    return fail(kBadArgument, "N and leading dimensions must be multiples of 8 and cover the row");
  if (!aligned16(Z) || !aligned16(dZ) || !aligned16(postact)) return fail(kBadArgument, "pointers must be 16-byte aligned");
  EpiSwigluBwdZdz::Params ep;
  ep.Z = static_cast<const __nv_bfloat16*>(Z);
  ep.ldz = ldz;
  ep.dZ = static_cast<__nv_bfloat16*>(dZ);
  ep.ld_dz = ld_dz;
  ep.postact = static_cast<__nv_bfloat16*>(postact);
  ep.ld_post = ld_post;
  ep.part_zdz = part_zdz;
  ep.tiles_n = (N + kTileN - 1) / kTileN;
  int rc = make_tmap_out(&ep.tm_dz, ep.dZ, 2LL * N, M, ld_dz);
  if (rc == kOk) rc = make_tmap_out(&ep.tm_post, ep.postact, N, M, ld_post);
  if (rc == kOk) rc = make_tmap_out(&ep.tm_z, ep.Z, 2LL * N, M, ldz);
  if (rc != kOk) return rc;
  Operand a{A, a_stride_m, a_stride_k};
  Operand b{B, b_stride_n, b_stride_k};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = launch_gemm<EpiSwigluBwdZdz, 3>(a, b, M, N, K, ep, dev_status, st);
  if (rc != kOk) return rc;
  row_reduce_kernel<<<(M + 7) / 8, 256, 0, st>>>(part_zdz, ep.tiles_n, zdz, M, scale, 0.f, 0);
  return launch_check("zdz reduce launch");
}

extern "C" int coda_b200_gemm_residual_partial_rmsnorm_bwd(const void* A, int64_t a_stride_m, int64_t a_stride_k, const void* B,
                                                           int64_t b_stride_k, int64_t b_stride_n, const void* weight,
                                                           const void* pre, int64_t ld_pre, const float* zdz, const float* rstd,
                                                           const float* alpha, void* dX, int64_t ld_dx, int accumulate, float* dW,
                                                           void* normed, int64_t ld_normed, float* part_dw, int M, int N, int K,
                                                           int* dev_status, void* stream) {
  if (!A || !B || !weight || !pre || !zdz || !rstd || !dX || !dW || !normed || !part_dw) return fail(kBadArgument, "NULL pointer");
  if (N % 8 || ld_pre % 8 || ld_dx % 8 || ld_normed % 8 || ld_pre < N || ld_dx < N || ld_normed < N)
    return fail(kBadArgument, "N and leading dimensions must be multiples of 8 and cover the row");
  if (!aligned16(pre) || !aligned16(dX) || !aligned16(normed) || !aligned16(weight)) return fail(kBadArgument, "pointers must be 16-byte aligned");
  EpiRmsnormBwd::Params ep;
  ep.pre = static_cast<const __nv_bfloat16*>(pre);
  ep.ld_pre = ld_pre;
  ep.dX = static_cast<__nv_bfloat16*>(dX);
  ep.ld_dx = ld_dx;
  ep.normed = static_cast<__nv_bfloat16*>(normed);
  ep.ld_normed = ld_normed;
  ep.weight = static_cast<const __nv_bfloat16*>(weight);
  ep.rstd = rstd;
  ep.zdz = zdz;
  ep.alpha = alpha;
  ep.part_dw = part_dw;
  ep.accumulate = accumulate;
  int rc = make_tmap_out(&ep.tm_dx, ep.dX, N, M, ld_dx);
  if (rc == kOk) rc = make_tmap_out(&ep.tm_normed, ep.normed, N, M, ld_normed);
  if (rc == kOk) rc = make_tmap_out(&ep.tm_pre, ep.pre, N, M, ld_pre);
  if (rc != kOk) return rc;
  Operand a{A, a_stride_m, a_stride_k};
  Operand b{B, b_stride_n, b_stride_k};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  rc = launch_gemm<EpiRmsnormBwd, 3>(a, b, M, N, K, ep, dev_status, st);
  if (rc != kOk) return rc;
  const int slabs = (M + 31) / 32;
  col_reduce_kernel<<<(N + 31) / 32, 256, 0, st>>>(part_dw, slabs, N, dW);
  return launch_check("dweight reduce launch");
}
