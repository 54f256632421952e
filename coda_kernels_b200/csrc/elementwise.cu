// HBM-bound side kernels of the fused-linear operators: the activation
// gradients that feed the backward GEMMs, the log-sum-exp reduction and the
// in-place softmax-gradient pass.  All of them move 16 bytes per thread per
// access and keep their math in fp32.  See include/coda_b200.h for the contract.
#include "../../include/coda_b200.h"
#include "gemm_host.cuh"

using namespace cb;

namespace {

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int launch_check(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(kCudaError, std::string(what) + ": " + cudaGetErrorString(e));
  return kOk;
}

// ------------------------------------------------------------------ dSwiGLU
// One thread: 8 outputs of dout <-> 16 interleaved (gate, up) values.
template <bool kSigmoidGate>
__global__ void __launch_bounds__(256) dswiglu_kernel(const __nv_bfloat16* __restrict__ preact, long long ld_pre,
                                                      const __nv_bfloat16* __restrict__ dout, long long ld_dout,
                                                      __nv_bfloat16* __restrict__ grad, long long ld_grad, int M, int F8) {
  const long long total = static_cast<long long>(M) * F8;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(idx / F8);
    const int g8 = static_cast<int>(idx - static_cast<long long>(row) * F8);
    const uint4 d4 = *reinterpret_cast<const uint4*>(dout + row * ld_dout + g8 * 8);
    const uint4* zp = reinterpret_cast<const uint4*>(preact + row * ld_pre + g8 * 16);
    const uint4 z0 = zp[0], z1 = zp[1];
    const uint32_t dw[4] = {d4.x, d4.y, d4.z, d4.w};
    const uint32_t zw[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
    uint32_t ow[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 dd = unpack_bf16x2(dw[j]);
      const float t[2] = {dd.x, dd.y};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float2 gu = unpack_bf16x2(zw[2 * j + h]);
        const float g = gu.x, u = gu.y;
        const float s = fast_sigmoid(g);
        // silu gate: d/dg [g s u] = u (s + g s (1 - s)), d/du = g s;  sigmoid gate: d/dg [s u] = u s (1 - s), d/du = s
        const float dg = kSigmoidGate ? t[h] * u * s * (1.0f - s) : t[h] * u * (s + g * s * (1.0f - s));
        const float du = kSigmoidGate ? t[h] * s : t[h] * g * s;
        ow[2 * j + h] = pack_bf16x2(dg, du);
      }
    }
    uint4* op = reinterpret_cast<uint4*>(grad + row * ld_grad + g8 * 16);
    op[0] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    op[1] = make_uint4(ow[4], ow[5], ow[6], ow[7]);
  }
}

// ------------------------------------------------------------------ dSigmoid
template <typename OutT>
__global__ void __launch_bounds__(256) dsigmoid_kernel(const OutT* __restrict__ out, long long ld_out,
                                                       const __nv_bfloat16* __restrict__ dout, long long ld_dout,
                                                       __nv_bfloat16* __restrict__ grad, long long ld_grad, int M, int N8) {
  const long long total = static_cast<long long>(M) * N8;
  for (long long idx = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int row = static_cast<int>(idx / N8);
    const int c8 = static_cast<int>(idx - static_cast<long long>(row) * N8);
    const uint4 d4 = *reinterpret_cast<const uint4*>(dout + row * ld_dout + c8 * 8);
    const uint32_t dw[4] = {d4.x, d4.y, d4.z, d4.w};
    float o[8];
    if constexpr (sizeof(OutT) == 2) {
      const uint4 o4 = *reinterpret_cast<const uint4*>(out + row * ld_out + c8 * 8);
      const uint32_t w[4] = {o4.x, o4.y, o4.z, o4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        o[2 * j] = f.x;
        o[2 * j + 1] = f.y;
      }
    } else {
      const float4* p = reinterpret_cast<const float4*>(out + row * ld_out + c8 * 8);
      const float4 a = p[0], b = p[1];
      o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
      o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
    }
    uint32_t r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 dd = unpack_bf16x2(dw[j]);
      r[j] = pack_bf16x2(dd.x * o[2 * j] * (1.0f - o[2 * j]), dd.y * o[2 * j + 1] * (1.0f - o[2 * j + 1]));
    }
    *reinterpret_cast<uint4*>(grad + row * ld_grad + c8 * 8) = make_uint4(r[0], r[1], r[2], r[3]);
  }
}

// ------------------------------------------------------------------ LSE finalize: one warp per row
__global__ void __launch_bounds__(256) lse_finalize_kernel(const float* __restrict__ part_max, const float* __restrict__ part_sum,
                                                           int tiles_n, const int* __restrict__ target,
                                                           const float* __restrict__ target_logit, int ignore_index,
                                                           float* __restrict__ lse, float* __restrict__ losses, int M,
                                                           const float* __restrict__ part_sz = nullptr,
                                                           float* __restrict__ zdz = nullptr) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= M) return;
  const float* pm = part_max + static_cast<long long>(row) * tiles_n;
  const float* ps = part_sum + static_cast<long long>(row) * tiles_n;
  float mx = -INFINITY;
  for (int t = lane; t < tiles_n; t += 32) mx = fmaxf(mx, pm[t]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  float s = 0.f;
  for (int t = lane; t < tiles_n; t += 32) s += ps[t] * __expf(pm[t] - mx);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) {
    const float l = mx + logf(s);
    lse[row] = l;
    if (target != nullptr) losses[row] = (target[row] != ignore_index) ? (l - target_logit[row]) : 0.0f;
  }
  if (zdz != nullptr) {
    // sum_j z_j * (softmax_j - onehot_j) = sum_t exp(m_t - lse) * sz_t - z_target; zero for ignored rows
    const float l = mx + logf(s);
    const float* pz = part_sz + static_cast<long long>(row) * tiles_n;
    float a = 0.f;
    for (int t = lane; t < tiles_n; t += 32) a += pz[t] * __expf(pm[t] - l);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (lane == 0) zdz[row] = (target[row] != ignore_index) ? (a - target_logit[row]) : 0.0f;
  }
}

// ------------------------------------------------------------------ partial RMSNorm: one warp per row
// h = x * weight[col], an optional copy of x, and rstd = rsqrt(mean(x^2) + eps), from one read of x.
__global__ void __launch_bounds__(256) partial_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, long long ldx,
                                                              const __nv_bfloat16* __restrict__ weight, float eps,
                                                              __nv_bfloat16* __restrict__ residual, long long ld_res,
                                                              __nv_bfloat16* __restrict__ h, long long ld_h,
                                                              float* __restrict__ rstd, int M, int N8) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= M) return;
  float sq = 0.f;
  for (int c8 = lane; c8 < N8; c8 += 32) {
    const uint4 xv = *reinterpret_cast<const uint4*>(x + row * ldx + c8 * 8);
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(weight + c8 * 8));
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
    uint32_t r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = unpack_bf16x2(xw[j]), b = unpack_bf16x2(ww[j]);
      sq = fmaf(a.x, a.x, fmaf(a.y, a.y, sq));
      r[j] = pack_bf16x2(a.x * b.x, a.y * b.y);
    }
    *reinterpret_cast<uint4*>(h + row * ld_h + c8 * 8) = make_uint4(r[0], r[1], r[2], r[3]);
    if (residual != nullptr) *reinterpret_cast<uint4*>(residual + row * ld_res + c8 * 8) = xv;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
  if (lane == 0) rstd[row] = rsqrtf(sq / static_cast<float>(N8 * 8) + eps);
}

// ------------------------------------------------------------------ RoPE backward with the row dot: one warp per row
// dz = R^T dy (pairs (a, b) -> (a c + b s, b c - a s) at the angle of their column), zdz = scale * sum(y * dy).
__global__ void __launch_bounds__(256) rope_bwd_zdz_kernel(const __nv_bfloat16* __restrict__ y, long long ldy,
                                                           const __nv_bfloat16* __restrict__ dy, long long ld_dy,
                                                           const void* __restrict__ positions, int pos_is_float,
                                                           const float* __restrict__ freq, float scale,
                                                           __nv_bfloat16* __restrict__ dz, long long ld_dz,
                                                           float* __restrict__ zdz, int M, int N8) {
  constexpr float kTwoPi = 6.283185307179586f;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= M) return;
  const float pos = pos_is_float ? reinterpret_cast<const float*>(positions)[row]
                                 : static_cast<float>(reinterpret_cast<const int*>(positions)[row]);
  float dot = 0.f;
  for (int c8 = lane; c8 < N8; c8 += 32) {
    const uint4 yv = *reinterpret_cast<const uint4*>(y + row * ldy + c8 * 8);
    const uint4 gv = *reinterpret_cast<const uint4*>(dy + row * ld_dy + c8 * 8);
    const float4 f0 = __ldg(reinterpret_cast<const float4*>(freq + c8 * 8));
    const float4 f1 = __ldg(reinterpret_cast<const float4*>(freq + c8 * 8 + 4));
    const float fr[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
    const uint32_t yw[4] = {yv.x, yv.y, yv.z, yv.w}, gw[4] = {gv.x, gv.y, gv.z, gv.w};
    uint32_t r[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float2 yy = unpack_bf16x2(yw[p]), g = unpack_bf16x2(gw[p]);
      dot = fmaf(yy.x, g.x, fmaf(yy.y, g.y, dot));
      const float hi = fr[2 * p], lo = fr[2 * p + 1];
      const float t = pos * hi;
      const float terr = fmaf(pos, hi, -t);
      const float l = fmaf(pos, lo, terr);
      const float frac = (t - rintf(t)) + l;
      float sn, cs;
      __sincosf(kTwoPi * frac, &sn, &cs);
      r[p] = pack_bf16x2(g.x * cs + g.y * sn, g.y * cs - g.x * sn);
    }
    *reinterpret_cast<uint4*>(dz + row * ld_dz + c8 * 8) = make_uint4(r[0], r[1], r[2], r[3]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  if (lane == 0) zdz[row] = dot * scale;
}

// ------------------------------------------------------------------ cross entropy from stored logits, in place
// logits[i,j] <- exp(logits[i,j] - lse[i]) - (j == target[i]), or +0 for ignored rows; the thread that holds the
// target column also writes losses[i] = lse[i] - logit (rows that are ignored get 0 from the thread of column 0).
__global__ void __launch_bounds__(256) ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, long long ld,
                                                         const float* __restrict__ lse, const int* __restrict__ target,
                                                         int ignore_index, float* __restrict__ losses, int N8) {
  const int row = blockIdx.x;
  const int c8 = blockIdx.y * blockDim.x + threadIdx.x;
  if (c8 >= N8) return;
  const int col = c8 * 8;
  uint4* ptr = reinterpret_cast<uint4*>(logits + row * ld + col);
  const int tgt = target[row];
  if (tgt == ignore_index) {
    *ptr = make_uint4(0u, 0u, 0u, 0u);
    if (c8 == 0) losses[row] = 0.0f;
    return;
  }
  const float l = lse[row];
  const uint4 p4 = *ptr;
  const uint32_t w[4] = {p4.x, p4.y, p4.z, p4.w};
  uint32_t r[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 v = unpack_bf16x2(w[j]);
    float d0 = __expf(v.x - l), d1 = __expf(v.y - l);
    if (col + 2 * j == tgt) {
      losses[row] = l - v.x;
      d0 -= 1.0f;
    }
    if (col + 2 * j + 1 == tgt) {
      losses[row] = l - v.y;
      d1 -= 1.0f;
    }
    r[j] = pack_bf16x2(d0, d1);
  }
  *ptr = make_uint4(r[0], r[1], r[2], r[3]);
}

// ------------------------------------------------------------------ softmax-gradient fix-up, in place
// Rows on grid.x (no 65535 limit), kFixPieces * 2048 columns per block: each thread owns kFixPieces 16-byte pieces
// 2048 columns apart and has all of their loads in flight before it computes (a pure streaming read-modify-write).
constexpr int kFixPieces = 4;
__global__ void __launch_bounds__(256) ce_grad_fixup_kernel(__nv_bfloat16* __restrict__ P, long long ldp,
                                                            const float* __restrict__ part_max, int tiles_n, int tile_w,
                                                            const float* __restrict__ lse, const int* __restrict__ target,
                                                            int ignore_index, int N8) {
  const int row = blockIdx.x;
  const int c8_0 = blockIdx.y * (256 * kFixPieces) + threadIdx.x;
  if (c8_0 >= N8) return;
  __nv_bfloat16* prow = P + row * ldp;
  const int tgt = target[row];
  if (tgt == ignore_index) {
#pragma unroll
    for (int k = 0; k < kFixPieces; ++k) {
      const int c8 = c8_0 + 256 * k;
      if (c8 < N8) *reinterpret_cast<uint4*>(prow + c8 * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    return;
  }
  uint4 v[kFixPieces];
#pragma unroll
  for (int k = 0; k < kFixPieces; ++k) {
    const int c8 = c8_0 + 256 * k;
    v[k] = (c8 < N8) ? *reinterpret_cast<const uint4*>(prow + c8 * 8) : make_uint4(0u, 0u, 0u, 0u);
  }
  const float l = lse[row];
  const float* pm = part_max + static_cast<long long>(row) * tiles_n;
#pragma unroll
  for (int k = 0; k < kFixPieces; ++k) {
    const int c8 = c8_0 + 256 * k;
    if (c8 >= N8) break;
    const int col = c8 * 8;
    const float f = __expf(pm[col / tile_w] - l);
    const uint32_t w[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
    uint32_t r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = unpack_bf16x2(w[j]);
      t.x = t.x * f - ((col + 2 * j) == tgt ? 1.0f : 0.0f);
      t.y = t.y * f - ((col + 2 * j + 1) == tgt ? 1.0f : 0.0f);
      r[j] = pack_bf16x2(t.x, t.y);
    }
    *reinterpret_cast<uint4*>(prow + c8 * 8) = make_uint4(r[0], r[1], r[2], r[3]);
  }
}

// ------------------------------------------------------------------ QK-norm + RoPE backward
constexpr int kQkRowsPerBlock = 16;  // unit of the dgamma workspace: one partial row per 16 input rows at most
constexpr int kQkWarps = 8;
constexpr int kQkBlocksPerSm = 3;  // what the kernel's register and shared-memory budget allows to be resident

// A group of kHD/8 lanes owns one ROW and walks over a run of its heads: each lane handles the same 8 consecutive
// elements (16-byte accesses) of every head, so a warp works on 2 (kHD = 128) or 4 (kHD = 64) rows at once and reads
// their heads as contiguous streams.  Work items are (row group, run of kQkHeadsPerItem heads), handed out to the
// warps of a persistent grid in order, which keeps every SM busy to the end.
//
// Memory pipeline: every thread streams its own (dy, preact, mean_sq) pieces through a private ring of kQkDepth
// slots in shared memory with cp.async, one commit group per (item, head), so kQkDepth heads are in flight per
// thread without holding registers: an HBM-bound pass needs tens of kilobytes in flight per SM, more than a
// register-resident prefetch can hold at this kernel's register count.
//
// The rotation angle depends on (row, element) and on the head's frequencies only: as long as a head carries the
// same frequencies as the one before it (the layout make_rope_frequencies produces), its sines and cosines are
// reused.  Per head: un-rotate dy, take the RMSNorm VJP at the saved statistic, accumulate the gamma gradient in
// registers; at the end the block folds its warps and writes one partial row of [gamma_q | gamma_k] sums.
constexpr int kQkHeadsPerItem = 8;
constexpr int kQkDepth = 6;
constexpr int kQkThreads = kQkWarps * 32;
constexpr int kQkRingBytes = kQkDepth * kQkThreads * (16 + 16 + 4);  // dy piece, preact piece, mean_sq per slot and thread

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

template <int kHD>
__global__ void __launch_bounds__(kQkThreads, kQkBlocksPerSm)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ dq, long long ld_dq, const __nv_bfloat16* __restrict__ dk,
                       long long ld_dk, const __nv_bfloat16* __restrict__ dv, long long ld_dv, int nv8,
                       const __nv_bfloat16* __restrict__ preact, long long ld_pre, const float* __restrict__ mean_sq,
                       const __nv_bfloat16* __restrict__ gamma, const void* __restrict__ positions, int pos_is_float,
                       const float* __restrict__ freq, int hq, int hk, float eps, __nv_bfloat16* __restrict__ grad,
                       long long ld_grad, float* __restrict__ partials, int M) {
  constexpr int kG = kHD / 8;    // lanes per row
  constexpr int kRPW = 32 / kG;  // rows per warp
  constexpr float kTwoPi = 6.283185307179586f;
  extern __shared__ __align__(16) uint8_t qk_smem[];
  float(*red)[2 * kHD] = reinterpret_cast<float(*)[2 * kHD]>(qk_smem + kQkRingBytes);  // [kQkWarps * kRPW][2 * kHD]
  const uint32_t ring = smem_u32(qk_smem);
  // slot i of this thread: dy piece at ring_a + i * stride16, preact piece at ring_b + ..., mean_sq at ring_m + ...
  const uint32_t ring_a = ring + threadIdx.x * 16;
  const uint32_t ring_b = ring + kQkDepth * kQkThreads * 16 + threadIdx.x * 16;
  const uint32_t ring_m = ring + 2 * kQkDepth * kQkThreads * 16 + threadIdx.x * 4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane % kG, grp = lane / kG;
  const int heads = hq + hk;
  const int e0 = sub * 8;
  // the lanes of one row reduce among themselves only: rows of a warp may be past the end independently
  const unsigned group_mask = (kG == 32 ? 0xffffffffu : ((1u << kG) - 1u)) << (grp * kG);

  // Do all heads carry the frequencies of head 0 (the layout make_rope_frequencies produces)?  Checked once per
  // block; if so the sines and cosines of a row are computed once per work item instead of once per head.
  int same_here = 1;
  for (int i = threadIdx.x; i < heads * kHD; i += blockDim.x) same_here &= (freq[i] == freq[i % kHD]) ? 1 : 0;
  const bool periodic = __syncthreads_and(same_here) != 0;

  // gamma as fp32 in shared memory, read once per work item (its 8-float pieces sit 32 bytes apart from lane to lane,
  // a bank conflict that would hurt inside the head loop but not once per item); the per-lane dgamma sums of the
  // block accumulate in `red`, one row per (warp, row slot), touched once per work item as well.  Keeping both out
  // of registers is what lets three blocks share an SM.
  float* gam_s = reinterpret_cast<float*>(qk_smem + kQkRingBytes + kQkWarps * kRPW * 2 * kHD * 4);  // [2 * kHD]
  for (int c = threadIdx.x; c < 2 * kHD; c += blockDim.x) gam_s[c] = __bfloat162float(gamma[c]);
  float* my_red = &red[warp * kRPW + grp][e0];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    my_red[j] = 0.f;
    my_red[kHD + j] = 0.f;
  }
  __syncthreads();

  // Work items: (row group, run of up to kQkHeadsPerItem heads); a run never mixes q and k heads, so the gamma vector
  // and the accumulator it feeds are chosen once per item.
  const int runs_q = (hq + kQkHeadsPerItem - 1) / kQkHeadsPerItem;
  const int runs = runs_q + (hk + kQkHeadsPerItem - 1) / kQkHeadsPerItem;
  // (row group, run) pairs are walked without divisions: a warp's next item lies warps_total items ahead
  const int row_groups = (M + kRPW - 1) / kRPW;
  const int warps_total = static_cast<int>(gridDim.x) * kQkWarps;
  const int step_rg = warps_total / runs, step_run = warps_total % runs;

  // Cursor over this warp's stream of (item, head); identical in all lanes except for the row.
  struct Cursor {
    int rg, run;  // row group and run of the current item (rg >= row_groups: past the end)
    int head, h_end, row;
  };
  auto open_item = [&](Cursor& c) {
    c.row = c.rg * kRPW + grp;
    if (c.run < runs_q) {
      c.head = c.run * kQkHeadsPerItem;
      c.h_end = min(hq, c.head + kQkHeadsPerItem);
    } else {
      c.head = hq + (c.run - runs_q) * kQkHeadsPerItem;
      c.h_end = min(heads, c.head + kQkHeadsPerItem);
    }
  };
  // Source addresses of the prefetch cursor, advanced by one head per stream position (a run never leaves q or k).
  const __nv_bfloat16 *src_dy = nullptr, *src_pre = nullptr;
  const float* src_ms = nullptr;
  auto open_sources = [&](const Cursor& c) {
    if (c.rg < row_groups && c.row < M) {
      src_dy = c.head < hq ? dq + c.row * ld_dq + c.head * kHD + e0 : dk + c.row * ld_dk + (c.head - hq) * kHD + e0;
      src_pre = preact + c.row * ld_pre + c.head * kHD + e0;
      src_ms = mean_sq + static_cast<long long>(c.row) * heads + c.head;
    }
  };
  auto next_item = [&](Cursor& c) {
    c.rg += step_rg;
    c.run += step_run;
    if (c.run >= runs) {
      c.run -= runs;
      ++c.rg;
    }
    open_item(c);
  };
  // issue the loads of the prefetch cursor's position into `slot` and step the cursor
  auto issue_and_step = [&](Cursor& c, int slot) {
    const bool live = c.rg < row_groups;
    if (live && c.row < M) {
      cp_async16(ring_a + slot * (kQkThreads * 16), src_dy);
      cp_async16(ring_b + slot * (kQkThreads * 16), src_pre);
      cp_async4(ring_m + slot * (kQkThreads * 4), src_ms);
      src_dy += kHD;
      src_pre += kHD;
      src_ms += 1;
    }
    cp_async_commit();  // one group per stream position, empty or not, so that the group count stays uniform
    if (live && ++c.head >= c.h_end) {
      next_item(c);
      open_sources(c);
    }
  };
  auto sincos4 = [&](const float* f, float pos, float* sn, float* cs) {
#pragma unroll
    for (int p2 = 0; p2 < 4; ++p2) {
      const float hi = f[2 * p2], lo = f[2 * p2 + 1];
      const float t = pos * hi;
      const float terr = fmaf(pos, hi, -t);
      const float l = fmaf(pos, lo, terr);
      const float frac = (t - rintf(t)) + l;
      __sincosf(kTwoPi * frac, &sn[p2], &cs[p2]);
    }
  };

  Cursor use, pre;
  {
    const int first = static_cast<int>(blockIdx.x) * kQkWarps + warp;
    use.rg = first / runs;
    use.run = first % runs;
  }
  open_item(use);
  pre = use;
  open_sources(pre);
#pragma unroll 1
  for (int i = 0; i < kQkDepth; ++i) issue_and_step(pre, i);

  int slot = 0;
#pragma unroll 1
  while (use.rg < row_groups) {
    // ---- one work item: heads [use.head, use.h_end) of row use.row
    const int row = use.row, h_begin = use.head, h_end = use.h_end;
    const bool row_ok = row < M;
    const bool is_q = h_begin < hq;
    float gam[8], g[8], sn[4], cs[4];
    {
      const float4 g0 = *reinterpret_cast<const float4*>(gam_s + (is_q ? 0 : kHD) + e0);
      const float4 g1 = *reinterpret_cast<const float4*>(gam_s + (is_q ? 0 : kHD) + e0 + 4);
      gam[0] = g0.x; gam[1] = g0.y; gam[2] = g0.z; gam[3] = g0.w;
      gam[4] = g1.x; gam[5] = g1.y; gam[6] = g1.z; gam[7] = g1.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] = 0.f;
    float pos = 0.f;
    if (row_ok) {
      pos = pos_is_float ? reinterpret_cast<const float*>(positions)[row] : static_cast<float>(reinterpret_cast<const int*>(positions)[row]);
      if (periodic) {
        const float4 f0 = __ldg(reinterpret_cast<const float4*>(freq + e0));
        const float4 f1 = __ldg(reinterpret_cast<const float4*>(freq + e0 + 4));
        const float fn[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
        sincos4(fn, pos, sn, cs);
      }
    }
    __nv_bfloat16* out_p = grad + (row_ok ? row : 0) * ld_grad + h_begin * kHD + e0;
    const float* freq_p = freq + h_begin * kHD + e0;
#pragma unroll 1
    for (int head = h_begin; head < h_end; ++head, out_p += kHD, freq_p += kHD) {
      cp_async_wait<kQkDepth - 1>();  // the group of this stream position has landed
      if (row_ok) {
        const uint4 a = ld_shared_v4(ring_a + slot * (kQkThreads * 16));
        const uint4 b = ld_shared_v4(ring_b + slot * (kQkThreads * 16));
        float msv;
        asm volatile("ld.shared.f32 %0, [%1];" : "=f"(msv) : "r"(ring_m + slot * (kQkThreads * 4)) : "memory");
        const float r = rsqrtf(msv + eps);
        if (!periodic) {
          const float4 f0 = __ldg(reinterpret_cast<const float4*>(freq_p));
          const float4 f1 = __ldg(reinterpret_cast<const float4*>(freq_p + 4));
          const float fn[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
          sincos4(fn, pos, sn, cs);
        }
        float dy[8], xh[8];
        {
          // bf16 -> fp32 is a 16-bit shift: one shift and one mask per packed pair
          const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            dy[2 * j] = __uint_as_float(aw[j] << 16);
            dy[2 * j + 1] = __uint_as_float(aw[j] & 0xffff0000u);
            xh[2 * j] = __uint_as_float(bw[j] << 16);
            xh[2 * j + 1] = __uint_as_float(bw[j] & 0xffff0000u);
          }
        }
        float dz[8], tz[8];
#pragma unroll
        for (int p2 = 0; p2 < 4; ++p2) {
          const float u = dy[2 * p2], w = dy[2 * p2 + 1];
          dz[2 * p2] = fmaf(u, cs[p2], w * sn[p2]);
          dz[2 * p2 + 1] = fmaf(w, cs[p2], -(u * sn[p2]));
        }
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          tz[j] = dz[j] * gam[j];
          dot = fmaf(tz[j], xh[j], dot);
        }
#pragma unroll
        for (int o = kG / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(group_mask, dot, o);
        const float ncoef = -(dot * r * r * r * (1.0f / kHD));
        uint32_t ow[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          ow[j] = pack_bf16x2(fmaf(r, tz[2 * j], xh[2 * j] * ncoef), fmaf(r, tz[2 * j + 1], xh[2 * j + 1] * ncoef));
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] = fmaf(dz[j] * xh[j], r, g[j]);
        *reinterpret_cast<uint4*>(out_p) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      }
      // refill the slot just consumed with the stream position kQkDepth ahead
      issue_and_step(pre, slot);
      slot = (slot + 1 == kQkDepth) ? 0 : slot + 1;
    }
    {
      // this lane is the only writer of its 16 slots of `red`
      float* acc = my_red + (is_q ? 0 : kHD);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += g[j];
    }
    next_item(use);
  }
  cp_async_wait<0>();

  // copy dv next to grad_pre so that one GEMM consumes [grad_pre | dv]
  if (dv != nullptr) {
    const long long col_off = static_cast<long long>(heads) * kHD;
    for (int rr = blockIdx.x; rr < M; rr += gridDim.x)
      for (int c8 = threadIdx.x; c8 < nv8; c8 += blockDim.x)
        *reinterpret_cast<uint4*>(grad + rr * ld_grad + col_off + c8 * 8) = *reinterpret_cast<const uint4*>(dv + rr * ld_dv + c8 * 8);
  }

  __syncthreads();
  for (int c = threadIdx.x; c < 2 * kHD; c += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kQkWarps * kRPW; ++w) s += red[w][c];
    partials[static_cast<long long>(blockIdx.x) * (2 * kHD) + c] = s;
  }
}

template <int kHD>
constexpr int qk_bwd_smem_bytes() {
  return kQkRingBytes + kQkWarps * (32 / (kHD / 8)) * 2 * kHD * 4 + 2 * kHD * 4;
}

// Column sums of the [nblocks, width] partials: 32 columns x 32 row-lanes per block, rows strided over the lanes, so that
// the few hundred partial rows are a dozen independent loads per thread rather than a long serial chain.
constexpr int kFoldRowLanes = 32;
__global__ void __launch_bounds__(32 * kFoldRowLanes) fold_partials_kernel(const float* __restrict__ partials, int nblocks, int width,
                                                                          float* __restrict__ out) {
  __shared__ float red[kFoldRowLanes][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (c < width) {
#pragma unroll 4
    for (int b = ry; b < nblocks; b += kFoldRowLanes) s += partials[static_cast<long long>(b) * width + c];
  }
  red[ry][cx] = s;
  __syncthreads();
  if (ry == 0 && c < width) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < kFoldRowLanes; ++j) t += red[j][cx];
    out[c] = t;
  }
}

inline int grid_for(long long total, int block) {
  long long g = (total + block - 1) / block;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace

namespace {
template <bool kSigmoidGate>
int run_dgated(const void* preact, int64_t ld_pre, const void* dout, int64_t ld_dout, void* grad_pre, int64_t ld_grad, int M, int F,
               void* stream) {
  if (!preact || !dout || !grad_pre) return fail(kBadArgument, "NULL pointer");
  if (M <= 0 || F <= 0 || F % 8 != 0) return fail(kBadArgument, "F must be a positive multiple of 8");
  if (ld_pre % 8 || ld_dout % 8 || ld_grad % 8 || ld_pre < 2 * F || ld_grad < 2 * F || ld_dout < F)
    return fail(kBadArgument, "leading dimensions must be multiples of 8 and cover the row");
  if (!aligned16(preact) || !aligned16(dout) || !aligned16(grad_pre)) return fail(kBadArgument, "pointers must be 16-byte aligned");
  const int F8 = F / 8;
  dswiglu_kernel<kSigmoidGate><<<grid_for(static_cast<long long>(M) * F8, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(preact), ld_pre, static_cast<const __nv_bfloat16*>(dout), ld_dout,
      static_cast<__nv_bfloat16*>(grad_pre), ld_grad, M, F8);
  return launch_check("gated-activation backward launch");
}
}  // namespace

extern "C" int coda_b200_dswiglu(const void* preact, int64_t ld_pre, const void* dout, int64_t ld_dout, void* grad_pre,
                                 int64_t ld_grad, int M, int F, void* stream) {
  return run_dgated<false>(preact, ld_pre, dout, ld_dout, grad_pre, ld_grad, M, F, stream);
}

extern "C" int coda_b200_dsigmoid_glu(const void* preact, int64_t ld_pre, const void* dout, int64_t ld_dout, void* grad_pre,
                                      int64_t ld_grad, int M, int F, void* stream) {
  return run_dgated<true>(preact, ld_pre, dout, ld_dout, grad_pre, ld_grad, M, F, stream);
}

extern "C" int coda_b200_dsigmoid(const void* out, int64_t ld_out, int out_is_fp32, const void* dout, int64_t ld_dout,
                                  void* grad_pre, int64_t ld_grad, int M, int N, void* stream) {
  if (!out || !dout || !grad_pre) return fail(kBadArgument, "NULL pointer");
  if (M <= 0 || N <= 0 || N % 8 != 0) return fail(kBadArgument, "N must be a positive multiple of 8");
  if (ld_out % 8 || ld_dout % 8 || ld_grad % 8 || ld_out < N || ld_dout < N || ld_grad < N)
    return fail(kBadArgument, "leading dimensions must be multiples of 8 and cover the row");
  if (!aligned16(out) || !aligned16(dout) || !aligned16(grad_pre)) return fail(kBadArgument, "pointers must be 16-byte aligned");
  const int N8 = N / 8;
  const int grid = grid_for(static_cast<long long>(M) * N8, 256);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_is_fp32)
    dsigmoid_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(out), ld_out, static_cast<const __nv_bfloat16*>(dout),
                                                 ld_dout, static_cast<__nv_bfloat16*>(grad_pre), ld_grad, M, N8);
  else
    dsigmoid_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(out), ld_out,
                                                         static_cast<const __nv_bfloat16*>(dout), ld_dout,
                                                         static_cast<__nv_bfloat16*>(grad_pre), ld_grad, M, N8);
  return launch_check("dsigmoid launch");
}

extern "C" int coda_b200_lse_finalize(const float* part_max, const float* part_sum, int tiles_n, const int32_t* target,
                                      const float* target_logit, int ignore_index, float* lse, float* losses, int M,
                                      void* stream) {
  if (!part_max || !part_sum || !target || !target_logit || !lse || !losses) return fail(kBadArgument, "NULL pointer");
  if (M <= 0 || tiles_n <= 0) return fail(kBadArgument, "M and tiles_n must be positive");
  const int rows_per_block = 8;
  lse_finalize_kernel<<<(M + rows_per_block - 1) / rows_per_block, rows_per_block * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      part_max, part_sum, tiles_n, target, target_logit, ignore_index, lse, losses, M);
  return launch_check("lse_finalize launch");
}

extern "C" int coda_b200_lse_finalize_zdz(const float* part_max, const float* part_sum, const float* part_sz, int tiles_n,
                                          const int32_t* target, const float* target_logit, int ignore_index, float* lse,
                                          float* losses, float* zdz, int M, void* stream) {
  if (!part_max || !part_sum || !part_sz || !target || !target_logit || !lse || !losses || !zdz) return fail(kBadArgument, "NULL pointer");
  if (M <= 0 || tiles_n <= 0) return fail(kBadArgument, "M and tiles_n must be positive");
  const int rows_per_block = 8;
  lse_finalize_kernel<<<(M + rows_per_block - 1) / rows_per_block, rows_per_block * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      part_max, part_sum, tiles_n, target, target_logit, ignore_index, lse, losses, M, part_sz, zdz);
  return launch_check("lse_finalize_zdz launch");
}

extern "C" int coda_b200_partial_rmsnorm(const void* x, int64_t ldx, const void* weight, float eps, void* residual, int64_t ld_res,
                                         void* h, int64_t ld_h, float* rstd, int M, int N, void* stream) {
  if (!x || !weight || !h || !rstd) return fail(kBadArgument, "NULL pointer");
  if (M <= 0 || N <= 0 || N % 8 || ldx % 8 || ld_h % 8 || ldx < N || ld_h < N) return fail(kBadArgument, "N and leading dimensions must be multiples of 8");
  if (!aligned16(x) || !aligned16(weight) || !aligned16(h)) return fail(kBadArgument, "pointers must be 16-byte aligned");
  if (residual != nullptr && (!aligned16(residual) || ld_res % 8 || ld_res < N)) return fail(kBadArgument, "bad residual buffer");
  partial_rmsnorm_kernel<<<(M + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), ldx, static_cast<const __nv_bfloat16*>(weight), eps, static_cast<__nv_bfloat16*>(residual),
      ld_res, static_cast<__nv_bfloat16*>(h), ld_h, rstd, M, N / 8);
  return launch_check("partial_rmsnorm launch");
}

extern "C" int coda_b200_rope_bwd_zdz(const void* y, int64_t ldy, const void* dy, int64_t ld_dy, const void* positions,
                                      int pos_is_float, const float* frequencies, float scale, void* dz, int64_t ld_dz, float* zdz,
                                      int M, int N, void* stream) {
  if (!y || !dy || !positions || !frequencies || !dz || !zdz) return fail(kBadArgument, "NULL pointer");
  if (M <= 0 || N <= 0 || N % 8 || ldy % 8 || ld_dy % 8 || ld_dz % 8 || ldy < N || ld_dy < N || ld_dz < N)
    return fail(kBadArgument, "N and leading dimensions must be multiples of 8");
  if (!aligned16(y) || !aligned16(dy) || !aligned16(dz) || !aligned16(frequencies)) return fail(kBadArgument, "pointers must be 16-byte aligned");
  rope_bwd_zdz_kernel<<<(M + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), ldy, static_cast<const __nv_bfloat16*>(dy), ld_dy, positions, pos_is_float, frequencies,
      scale, static_cast<__nv_bfloat16*>(dz), ld_dz, zdz, M, N / 8);
  return launch_check("rope_bwd_zdz launch");
}

extern "C" int coda_b200_lse_reduce(const float* part_max, const float* part_sum, int tiles_n, float* lse, int M, void* stream) {
  if (!part_max || !part_sum || !lse) return fail(kBadArgument, "NULL pointer");
  if (M <= 0 || tiles_n <= 0) return fail(kBadArgument, "M and tiles_n must be positive");
  const int rows_per_block = 8;
  lse_finalize_kernel<<<(M + rows_per_block - 1) / rows_per_block, rows_per_block * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      part_max, part_sum, tiles_n, nullptr, nullptr, 0, lse, nullptr, M);
  return launch_check("lse_reduce launch");
}

extern "C" int coda_b200_cross_entropy_fwd_bwd(void* logits, int64_t ld, const float* lse, const int32_t* target,
                                               int ignore_index, float* losses, int M, int N, void* stream) {
  if (!logits || !lse || !target || !losses) return fail(kBadArgument, "NULL pointer");
  if (M <= 0 || N <= 0 || N % 8 != 0 || ld % 8 != 0 || ld < N || !aligned16(logits))
    return fail(kBadArgument, "logits must be 16-byte aligned, N and ld multiples of 8");
  const int N8 = N / 8;
  if ((N8 + 255) / 256 > 65535) return fail(kBadArgument, "N too large for this grid");
  dim3 grid(M, (N8 + 255) / 256, 1);
  ce_fwd_bwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<__nv_bfloat16*>(logits), ld, lse, target,
                                                                        ignore_index, losses, N8);
  return launch_check("cross_entropy_fwd_bwd launch");
}

extern "C" int coda_b200_ce_grad_fixup(void* P, int64_t ldp, const float* part_max, int tiles_n, const float* lse,
                                       const int32_t* target, int ignore_index, int M, int N, void* stream) {
  if (!P || !part_max || !lse || !target) return fail(kBadArgument, "NULL pointer");
  if (M <= 0 || N <= 0 || N % 8 != 0 || ldp % 8 != 0 || ldp < N || !aligned16(P))
    return fail(kBadArgument, "P must be 16-byte aligned, N and ldp multiples of 8");
  if (tiles_n != coda_b200_lse_tiles(N)) return fail(kBadArgument, "tiles_n does not match coda_b200_lse_tiles(N)");
  const int N8 = N / 8;
  const int per_block = 256 * kFixPieces;
  if ((N8 + per_block - 1) / per_block > 65535) return fail(kBadArgument, "N too large for the fix-up grid");
  dim3 grid(M, (N8 + per_block - 1) / per_block, 1);
  ce_grad_fixup_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<__nv_bfloat16*>(P), ldp, part_max,
                                                                           tiles_n, 256, lse, target, ignore_index, N8);
  return launch_check("ce_grad_fixup launch");
}

extern "C" int64_t coda_b200_qknorm_rope_bwd_scratch_bytes(int M, int head_dim) {
  const long long blocks = (static_cast<long long>(M) + kQkRowsPerBlock - 1) / kQkRowsPerBlock;
  return blocks * 2 * head_dim * static_cast<long long>(sizeof(float));
}

extern "C" int coda_b200_qknorm_rope_bwd(const void* dq, int64_t ld_dq, const void* dk, int64_t ld_dk, const void* dv,
                                         int64_t ld_dv, int nv, const void* preact, int64_t ld_pre, const float* mean_sq,
                                         const void* gamma, const void* positions, int pos_is_float, const float* frequencies,
                                         int head_dim, int hq, int hk, float eps, void* grad, int64_t ld_grad, float* dgamma,
                                         void* scratch, int64_t scratch_bytes, int M, void* stream) {
  if (!preact || !mean_sq || !gamma || !positions || !frequencies || !grad || !dgamma || !scratch)
    return fail(kBadArgument, "NULL pointer");
  if (head_dim != 64 && head_dim != 128) return fail(kBadArgument, "head_dim must be 64 or 128");
  if (M <= 0 || hq < 0 || hk < 0 || hq + hk <= 0) return fail(kBadArgument, "bad extents");
  if ((hq > 0 && !dq) || (hk > 0 && !dk)) return fail(kBadArgument, "dq / dk required");
  if (scratch_bytes < coda_b200_qknorm_rope_bwd_scratch_bytes(M, head_dim)) return fail(kBadArgument, "scratch buffer too small");
  // 16-byte vector accesses on every row
  if (ld_dq % 8 || ld_dk % 8 || ld_pre % 8 || ld_grad % 8) return fail(kBadArgument, "row strides must be multiples of 8 elements");
  if ((hq > 0 && !aligned16(dq)) || (hk > 0 && !aligned16(dk)) || !aligned16(preact) || !aligned16(grad) || !aligned16(frequencies))
    return fail(kBadArgument, "misaligned pointer");
  if (dv != nullptr && (nv <= 0 || nv % 8 || ld_dv % 8 || !aligned16(dv))) return fail(kBadArgument, "bad dv extent / alignment");
  if (dv == nullptr && nv > 0) return fail(kBadArgument, "dv is required when nv > 0");
  // every row must fit inside its leading dimension: the kernel writes and reads rows with 16-byte accesses
  const long long size_q = static_cast<long long>(hq) * head_dim, size_k = static_cast<long long>(hk) * head_dim;
  const long long nv_cols = dv ? nv : 0;
  if (ld_pre < size_q + size_k) return fail(kBadArgument, "ld_pre is smaller than (hq + hk) * head_dim");
  if (ld_grad < size_q + size_k + nv_cols) return fail(kBadArgument, "ld_grad is smaller than (hq + hk) * head_dim + nv");
  if (hq > 0 && ld_dq < size_q) return fail(kBadArgument, "ld_dq is smaller than hq * head_dim");
  if (hk > 0 && ld_dk < size_k) return fail(kBadArgument, "ld_dk is smaller than hk * head_dim");
  if (dv != nullptr && ld_dv < nv) return fail(kBadArgument, "ld_dv is smaller than nv");
  // persistent grid: as many blocks as are resident at once, never more than the workspace has partial rows for
  // (one per kQkRowsPerBlock input rows) nor than there are work items for
  const int rows_per_warp = 32 / (head_dim / 8);
  const long long items = ((static_cast<long long>(M) + rows_per_warp - 1) / rows_per_warp) *
                          ((hq + kQkHeadsPerItem - 1) / kQkHeadsPerItem + (hk + kQkHeadsPerItem - 1) / kQkHeadsPerItem);
  if (items > 0x7fffffffLL) return fail(kBadArgument, "too many (row, head) items for one launch");
  long long blocks_ll = (items + kQkWarps - 1) / kQkWarps;
  const long long cap = static_cast<long long>(sm_count()) * kQkBlocksPerSm;
  const long long ws_rows = (static_cast<long long>(M) + kQkRowsPerBlock - 1) / kQkRowsPerBlock;
  if (blocks_ll > cap) blocks_ll = cap;
  if (blocks_ll > ws_rows) blocks_ll = ws_rows;
  const int blocks = static_cast<int>(blocks_ll);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* partials = static_cast<float*>(scratch);
  const int nv8 = dv ? nv / 8 : 0;
  {
    // the ring needs more than the default 48 KB of dynamic shared memory: opt in once per device
    static std::atomic<unsigned long long> attr_set{0ull};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || ((attr_set.load(std::memory_order_acquire) >> dev) & 1ull) == 0ull) {
      cudaError_t e = cudaFuncSetAttribute(qknorm_rope_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, qk_bwd_smem_bytes<128>());
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(qknorm_rope_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, qk_bwd_smem_bytes<64>());
      if (e != cudaSuccess) return fail(kCudaError, std::string("cudaFuncSetAttribute(qknorm_rope_bwd smem): ") + cudaGetErrorString(e));
      if (dev >= 0 && dev < 64) attr_set.fetch_or(1ull << dev, std::memory_order_release);
    }
  }
  if (head_dim == 128)
    qknorm_rope_bwd_kernel<128><<<blocks, kQkThreads, qk_bwd_smem_bytes<128>(), st>>>(
        static_cast<const __nv_bfloat16*>(dq), ld_dq, static_cast<const __nv_bfloat16*>(dk), ld_dk,
        static_cast<const __nv_bfloat16*>(dv), ld_dv, nv8, static_cast<const __nv_bfloat16*>(preact), ld_pre, mean_sq,
        static_cast<const __nv_bfloat16*>(gamma), positions, pos_is_float, frequencies, hq, hk, eps,
        static_cast<__nv_bfloat16*>(grad), ld_grad, partials, M);
  else
    qknorm_rope_bwd_kernel<64><<<blocks, kQkThreads, qk_bwd_smem_bytes<64>(), st>>>(
        static_cast<const __nv_bfloat16*>(dq), ld_dq, static_cast<const __nv_bfloat16*>(dk), ld_dk,
        static_cast<const __nv_bfloat16*>(dv), ld_dv, nv8, static_cast<const __nv_bfloat16*>(preact), ld_pre, mean_sq,
        static_cast<const __nv_bfloat16*>(gamma), positions, pos_is_float, frequencies, hq, hk, eps,
        static_cast<__nv_bfloat16*>(grad), ld_grad, partials, M);
  int rc = launch_check("qknorm_rope_bwd launch");
  if (rc != kOk) return rc;
  fold_partials_kernel<<<(2 * head_dim + 31) / 32, 32 * kFoldRowLanes, 0, st>>>(partials, blocks, 2 * head_dim, dgamma);
  return launch_check("fold_partials launch");
}

// ------------------------------------------------------------------ QK-norm + RoPE backward without a caller-provided workspace
// Some hosts cannot give this library a scratch buffer: a plain C or ctypes
// caller that owns nothing but its input and output arrays, or a process that
// reserved all device memory at start-up and forbids cudaMalloc afterwards
// (cudaMalloc synchronises the device and may fail late under memory pressure).
// For them the per-block partial sums of dgamma live in this fixed array, which
// every GPU that loads the library keeps resident until the process exits.
constexpr int kNoAllocMaxRows = 16384;                                                // largest M accepted
constexpr int kNoAllocMaxBlocks = (kNoAllocMaxRows + kQkRowsPerBlock - 1) / kQkRowsPerBlock;  // 1024 partial rows
constexpr int kNoAllocScratchFloats = kNoAllocMaxBlocks * 2 * 128;                    // 1 MiB of fp32
static __device__ __align__(256) float g_qk_bwd_scratch[kNoAllocScratchFloats];

namespace {
// Device address of g_qk_bwd_scratch on the current device.  In host code the
// array's name is only a handle for the runtime, never a pointer a kernel may
// dereference, so the address is looked up once per device and cached.
int noalloc_scratch_ptr(float** out, const void* caller_buffer) {
  static std::atomic<float*> cached[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(kCudaError, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(kBadArgument, "device ordinal out of range for the built-in scratch table");
  // The array used is the current device's copy: refuse a call whose buffers live on another GPU rather than run the
  // kernel against the wrong device's scratch.
  cudaPointerAttributes attr;
  const cudaError_t pe = cudaPointerGetAttributes(&attr, caller_buffer);
  if (pe != cudaSuccess) (void)cudaGetLastError();  // an address the runtime does not know: nothing to compare, clear the error
  if (pe == cudaSuccess && attr.type == cudaMemoryTypeDevice && attr.device != dev)
    return fail(kBadArgument, "the buffers of this call live on device " + std::to_string(attr.device) + " but device " +
                                  std::to_string(dev) + " is current: make the owning device current first");
  float* ptr = cached[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_qk_bwd_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(kCudaError, std::string("cudaGetSymbolAddress(g_qk_bwd_scratch): ") + cudaGetErrorString(e));
    ptr = static_cast<float*>(p);
    cached[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return kOk;
}
}  // namespace

extern "C" int coda_b200_qknorm_rope_bwd_noalloc(const void* dq, int64_t ld_dq, const void* dk, int64_t ld_dk, const void* dv,
                                                 int64_t ld_dv, int nv, const void* preact, int64_t ld_pre,
                                                 const float* mean_sq, const void* gamma, const void* positions,
                                                 int pos_is_float, const float* frequencies, int head_dim, int hq, int hk,
                                                 float eps, void* grad, int64_t ld_grad, float* dgamma, int M, void* stream) {
  if (M > kNoAllocMaxRows)
    return fail(kBadArgument, "coda_b200_qknorm_rope_bwd_noalloc handles at most " + std::to_string(kNoAllocMaxRows) +
                                  " rows per call (got " + std::to_string(M) + "); split the batch or use coda_b200_qknorm_rope_bwd");
  if (head_dim != 64 && head_dim != 128) return fail(kBadArgument, "head_dim must be 64 or 128");
  if (grad == nullptr) return fail(kBadArgument, "NULL pointer");
  float* scratch = nullptr;
  const int rc = noalloc_scratch_ptr(&scratch, grad);
  if (rc != kOk) return rc;
  return coda_b200_qknorm_rope_bwd(dq, ld_dq, dk, ld_dk, dv, ld_dv, nv, preact, ld_pre, mean_sq, gamma, positions, pos_is_float,
                                   frequencies, head_dim, hq, hk, eps, grad, ld_grad, dgamma, scratch,
                                   static_cast<int64_t>(sizeof(float)) * kNoAllocScratchFloats, M, stream);
}
