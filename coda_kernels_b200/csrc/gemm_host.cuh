// Host-side launch glue for the tcgen05 GEMM core: operand description, TMA
// tensor-map encoding, grid sizing and the (cluster) launch itself.  Nothing in
// here allocates device memory or synchronises the device.
#pragma once

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <type_traits>

#include "epilogues.cuh"

namespace cb {

// C-ABI return codes.
enum : int {
  kOk = 0,
  kBadArgument = -1,    // shape / alignment / stride the kernels cannot take
  kBadLayout = -2,      // operand is neither row- nor column-contiguous
  kCudaError = -3,      // a CUDA runtime call failed
  kNoDriverEntry = -4,  // cuTensorMapEncodeTiled could not be resolved
};

inline thread_local std::string g_last_error;
inline int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

// Process-wide tuning options (set through coda_b200_set_option).  Each field is an atomic, so that a host thread
// that changes one while another launches never tears a value; a launch reads every option once, at its start.
struct Options {
  std::atomic<int> cta_group{2};  // 1 = one CTA per tile (128 rows), 2 = CTA pair per tile (256 rows)
  std::atomic<int> group_m{0};    // raster group in tiles; 0 = default
  std::atomic<int> max_ctas{0};   // cap on the persistent grid; 0 = all SMs
  std::atomic<int> tile_n{0};     // 0 = choose per problem; 64, 128 or 256 forces the column-tile width where it is built
  std::atomic<int> epi_tma{1};    // 1 = epilogues stage their output in shared memory and store it with TMA; 0 = per-thread stores
  std::atomic<int> split_tail{1};  // 1 = a plain GEMM given a workspace may cut the tiles of its last round along K
  // Measurement aid: KB of extra global loads / shared stores per k-block and CTA issued by the epilogue warps while the
  // mainloop runs (the traffic an operand-transforming prologue would add); results are unaffected.  0 = off.
  std::atomic<int> probe_ld_kb{0};
  std::atomic<int> probe_st_kb{0};
};
inline Options& options() {
  static Options o;
  return o;
}

// A 2-D bf16 operand given by its two element strides; exactly one must be 1.
// `rows` indexes the M (for A) or N (for B) dimension, `depth` the contraction.
struct Operand {
  const void* ptr;
  long long stride_row;    // elements between consecutive rows
  long long stride_depth;  // elements between consecutive contraction indices
};

inline bool classify(const Operand& o, long long rows, long long depth, bool* mn_major, long long* ld) {
  if (o.stride_depth == 1 && (o.stride_row >= depth || rows == 1)) {
    *mn_major = false;
    *ld = o.stride_row;
    return true;
  }
  if (o.stride_row == 1 && (o.stride_depth >= rows || depth == 1)) {
    *mn_major = true;
    *ld = o.stride_depth;
    return true;
  }
  return false;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      f = nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(f);
  }();
  return fn;
}

// bf16 matrix with `inner` contiguous elements per line and `outer` lines
// `ld` elements apart; box = 64 x box_outer, 128-byte swizzle, zero fill.
inline int make_tmap_bf16(CUtensorMap* m, const void* ptr, long long inner, long long outer, long long ld, int box_outer) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(kNoDriverEntry, "cuTensorMapEncodeTiled not available from the CUDA driver");
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) return fail(kBadArgument, "operand base address must be 16-byte aligned");
  if (outer > 1 && (ld * 2) % 16 != 0) return fail(kBadArgument, "operand leading dimension must be a multiple of 8 elements");
  if (inner % 8 != 0) return fail(kBadArgument, "operand contiguous extent must be a multiple of 8 elements");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>((outer > 1 ? ld : inner) * 2)};
  cuuint32_t box[2] = {64u, static_cast<cuuint32_t>(box_outer)};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kCudaError, "cuTensorMapEncodeTiled failed with code " + std::to_string(static_cast<int>(r)));
  return kOk;
}

// Tensor map of a row-major [rows, cols] output (bf16: elem_bytes 2, fp32: 4) for the staged epilogue stores:
// box = box_cols columns x 32 rows, swizzled by the box's row width (32, 64 or 128 bytes).
inline int make_tmap_out(CUtensorMap* m, const void* ptr, int elem_bytes, long long cols, long long rows, long long ld, int box_cols) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return fail(kNoDriverEntry, "cuTensorMapEncodeTiled not available from the CUDA driver");
  if ((reinterpret_cast<uintptr_t>(ptr) & 15u) != 0) return fail(kBadArgument, "output base address must be 16-byte aligned");
  if ((ld * elem_bytes) % 16 != 0 || ld < cols) return fail(kBadArgument, "output leading dimension must cover the row and be a multiple of 16 bytes");
  const int row_bytes = box_cols * elem_bytes;
  CUtensorMapSwizzle sw = row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
  if (row_bytes != 128 && row_bytes != 64 && row_bytes != 32) return fail(kBadArgument, "staged sub-tile rows must be 32, 64 or 128 bytes");
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld * elem_bytes)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), 32u};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(m, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kCudaError, "cuTensorMapEncodeTiled (output) failed with code " + std::to_string(static_cast<int>(r)));
  return kOk;
}
// (The same geometry serves the epilogues' second-operand loads: a 32 x 32 box that lands swizzled in a load slot,
// rows and columns outside the matrix reading as zero.)
template <typename T>
inline int make_tmap_out(CUtensorMap* m, T* ptr, long long cols, long long rows, long long ld, int box_cols = 32) {
  return make_tmap_out(m, static_cast<const void*>(ptr), static_cast<int>(sizeof(T)), cols, rows, ld, box_cols);
}

inline int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

// The options one launch works with, read once.
struct LaunchOptions {
  int cta_group, group_m, max_ctas, tile_n, epi_tma, probe_ld_kb, probe_st_kb, split_tail;
};
inline LaunchOptions launch_options() {
  const Options& o = options();
  return LaunchOptions{o.cta_group.load(), o.group_m.load(), o.max_ctas.load(), o.tile_n.load(),
                       o.epi_tma.load(),   o.probe_ld_kb.load(), o.probe_st_kb.load(), o.split_tail.load()};
}

// ------------------------------------------------------------------ tail split
// Does the epilogue type know how to park a partial accumulator in the workspace?
template <class E, class = void>
struct has_split_tail : std::false_type {};
template <class E>
struct has_split_tail<E, std::enable_if_t<E::kSplitTail>> : std::true_type {};

// Tiles are dealt to the CTA pairs round-robin; the `tail = num_tiles mod clusters` tiles of the last round keep only
// `tail` clusters busy for a whole contraction.  Cutting each tail tile into `split` ranges of k-blocks shortens that
// round to ceil(tail * split / clusters) * num_kb / split k-blocks, at the price of one fp32 round trip of every tail
// tile through the workspace and a follow-up kernel.  Returns the split (1 = leave the schedule alone): the one that
// minimises the tail's length in k-blocks, if it saves at least 15 % of it.  The workspace holds at most
// 2 * clusters partial tiles.
constexpr int kSplitOverheadKb = 12;  // partial epilogue + the follow-up pass, in k-block times
inline int plan_tail_split(long long num_tiles, int num_kb, int clusters, int* tail_out) {
  const int tail = static_cast<int>(num_tiles % clusters);
  *tail_out = tail;
  if (tail == 0 || clusters < 2 || num_kb < 16) return 1;
  const int max_split = std::min(std::min(2 * clusters / tail, num_kb / 8), 64);
  int best = 1;
  long long best_cost = num_kb;
  for (int s = 2; s <= max_split; ++s) {
    const long long rounds = (static_cast<long long>(tail) * s + clusters - 1) / clusters;
    const long long cost = rounds * ((num_kb + s - 1) / s) + kSplitOverheadKb;
    if (cost < best_cost) {
      best_cost = cost;
      best = s;
    }
  }
  return (best > 1 && best_cost * 100 <= static_cast<long long>(num_kb) * 85) ? best : 1;
}
inline long long split_workspace_bytes(int clusters, int tile_m, int bn) {
  return 2LL * clusters * tile_m * bn * static_cast<long long>(sizeof(float));
}
inline int full_clusters(const LaunchOptions& opt, int cta_group) {
  int sms = sm_count();
  if (opt.max_ctas > 0 && opt.max_ctas < sms) sms = opt.max_ctas;
  const int clusters = sms / cta_group;
  return clusters < 1 ? 1 : clusters;
}

// Adds the parts of every tail tile (in part order: the result does not depend on timing), applies alpha, converts
// and writes the tile to D.  Block (t, b) handles rows 4 b .. 4 b + 3 of tail tile t, one 16-byte group of four columns per
// thread (a 256-column tile): small blocks, because a launch has only a handful of tail tiles and each output needs
// `sk_split` loads from slabs that are far apart.
constexpr int kFinalizeRows = 4;
template <typename OutT>
__global__ void __launch_bounds__(256) split_finalize_kernel(const float* __restrict__ ws, OutT* __restrict__ D, long long ldd,
                                                             GemmShape shape, int first_tail_tile, int tile_m, int bn,
                                                             const float* __restrict__ alpha) {
  int tm, tn;
  tile_coords(shape, first_tail_tile + static_cast<int>(blockIdx.x), tm, tn);
  const float a = alpha != nullptr ? __ldg(alpha) : 1.0f;
  const int groups = bn / 4;
  const long long slab_stride = static_cast<long long>(tile_m) * bn;  // floats per slab
  for (int idx = threadIdx.x; idx < kFinalizeRows * groups; idx += 256) {
    const int r = blockIdx.y * kFinalizeRows + idx / groups, g = idx % groups;
    const int row = tm * tile_m + r, col = tn * bn + g * 4;
    if (row >= shape.M || col >= shape.N) continue;  // N is a multiple of 8: a group of 4 is all in or all out
    // part p of tail tile t sits in slab p * sk_tail + t
    const float* src = ws + blockIdx.x * slab_stride + static_cast<long long>(r) * bn + g * 4;
    float4 acc = __ldcs(reinterpret_cast<const float4*>(src));
#pragma unroll 4
    for (int part = 1; part < shape.sk_split; ++part) {
      const float4 v = __ldcs(reinterpret_cast<const float4*>(src + static_cast<long long>(part) * shape.sk_tail * slab_stride));
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    OutT* dst = D + static_cast<long long>(row) * ldd + col;
    if constexpr (sizeof(OutT) == 4) {
      *reinterpret_cast<float4*>(dst) = make_float4(acc.x * a, acc.y * a, acc.z * a, acc.w * a);
    } else {
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16x2(acc.x * a, acc.y * a), pack_bf16x2(acc.z * a, acc.w * a));
    }
  }
}

// With a prologue policy (`Pro`, see gemm_core.cuh) `a_ptr` is the raw matrix that TMA loads into the A slot and the
// transform warps rewrite in place; `pp` carries what else they need.
template <int kCtaGroup, int kBN, bool kAMn, bool kBMn, class Epi, class Pro = ProNone>
int launch_gemm_cfg(const void* a_ptr, long long lda, const void* b_ptr, long long ldb, int M, int N, int K,
                    const typename Epi::Params& ep, int* status, cudaStream_t stream, const LaunchOptions& opt,
                    const typename Pro::Params& pp = {}) {
  using Cfg = GemmCfg<kCtaGroup, kBN, Epi::kLoadRingBytes, Pro::kStageExtraBytes>;
  CUtensorMap ta, tb;
  int rc;
  // K-major: lines run along K; box = 64 k x (rows of the tile).  MN-major: lines run along M/N; box = 64 x 64 k.
  if (!kBMn) rc = make_tmap_bf16(&tb, b_ptr, K, N, ldb, Cfg::kBNcta);
  else rc = make_tmap_bf16(&tb, b_ptr, N, K, ldb, kBlockK);
  if (rc != kOk) return rc;
  if (!kAMn) rc = make_tmap_bf16(&ta, a_ptr, K, M, lda, kBlockM);
  else rc = make_tmap_bf16(&ta, a_ptr, M, K, lda, kBlockK);
  if (rc != kOk) return rc;

  GemmShape shape;
  shape.M = M;
  shape.N = N;
  shape.K = K;
  const int tile_m = kBlockM * kCtaGroup;
  shape.tiles_m = (M + tile_m - 1) / tile_m;
  shape.tiles_n = (N + kBN - 1) / kBN;
  shape.group_m = opt.group_m > 0 ? opt.group_m : (kCtaGroup == 2 ? 8 : 16);
  // per epilogue warp (four per CTA) and k-block, in bytes, rounded down to whole 512-byte warp accesses
  shape.probe_ld_bytes = opt.probe_ld_kb * 1024 / kNumEpiWarps / 512 * 512;
  shape.probe_st_bytes = opt.probe_st_kb * 1024 / kNumEpiWarps / 512 * 512;
  shape.probe_src = a_ptr;
  shape.probe_span = static_cast<long long>(M) * K * 2;  // the A operand's own bytes (valid for either major when densely packed)
  if ((kAMn ? lda != M : lda != K)) shape.probe_ld_bytes = 0;  // strided operand: no dense span to read from
  const long long num_tiles = static_cast<long long>(shape.tiles_m) * shape.tiles_n;
  if (num_tiles <= 0 || num_tiles > 0x7fffffffLL) return fail(kBadArgument, "tile count out of range");
  const int num_kb = (K + kBlockK - 1) / kBlockK;
  shape.sk_tail = 0;
  shape.sk_split = 1;
  typename Epi::Params ep_sk = ep;  // what the kernel receives (gains the workspace map if the tail is split)
  if constexpr (has_split_tail<Epi>::value && std::is_same<Pro, ProNone>::value) {
    const int all = full_clusters(opt, kCtaGroup);
    if (opt.split_tail != 0 && ep.ws != nullptr && ep.ws_bytes >= split_workspace_bytes(all, tile_m, kBN)) {
      shape.sk_split = plan_tail_split(num_tiles, num_kb, all, &shape.sk_tail);
      if (shape.sk_split > 1) {
        rc = make_tmap_out(&ep_sk.tm_ws, ep.ws, kBN, 2LL * all * tile_m, kBN);
        if (rc != kOk) return rc;
      }
    }
  }

  auto kern = gemm_kernel<kCtaGroup, kBN, kAMn, kBMn, Epi, Pro>;
  // One bit per device: setting the attribute twice is harmless, so two threads racing here only repeat the call.
  static std::atomic<unsigned long long> attr_set{0ull};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || ((attr_set.load(std::memory_order_acquire) >> dev) & 1ull) == 0ull) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg::kSmemBytes));
    if (e != cudaSuccess) return fail(kCudaError, std::string("cudaFuncSetAttribute(smem): ") + cudaGetErrorString(e));
    if (kCtaGroup == 2) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 0);
      (void)e;
    }
    if (dev >= 0 && dev < 64) attr_set.fetch_or(1ull << dev, std::memory_order_release);
  }
  int sms = sm_count();
  if (opt.max_ctas > 0 && opt.max_ctas < sms) sms = opt.max_ctas;
  int clusters = sms / kCtaGroup;
  if (clusters < 1) clusters = 1;
  if (clusters > num_tiles && shape.sk_split <= 1) clusters = static_cast<int>(num_tiles);

  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(clusters * kCtaGroup), 1, 1);
  cfg.blockDim = dim3(kNumThreads + Pro::kWarps * 32, 1, 1);
  cfg.dynamicSmemBytes = Cfg::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (kCtaGroup == 2) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, ta, tb, shape, ep_sk, status, pp);
  if (e != cudaSuccess) return fail(kCudaError, std::string("GEMM launch failed: ") + cudaGetErrorString(e));
  if constexpr (has_split_tail<Epi>::value && std::is_same<Pro, ProNone>::value) {
    if (shape.sk_split > 1) {
      const dim3 grid(static_cast<unsigned>(shape.sk_tail), static_cast<unsigned>(tile_m / kFinalizeRows), 1);
      split_finalize_kernel<<<grid, 256, 0, stream>>>(ep.ws, ep.D, ep.ldd, shape, static_cast<int>(num_tiles) - shape.sk_tail, tile_m, kBN,
                                                       ep.alpha);
      e = cudaGetLastError();
      if (e != cudaSuccess) return fail(kCudaError, std::string("tail-split follow-up launch failed: ") + cudaGetErrorString(e));
    }
  }
  return kOk;
}

// Column-tile width for epilogues that are built for several widths.  A narrower tile wins when the wide one would
// leave the last wave of the persistent grid mostly empty (few output tiles) or when N itself is narrow; otherwise
// the wide tile is kept, since it reads A once per 256 instead of once per 128 output columns.
inline int choose_tile_n(int M, int N, const LaunchOptions& opt, bool has64) {
  const int forced = opt.tile_n;
  if (forced == 128 || forced == 256 || (forced == 64 && has64)) return forced;
  if (N <= 64 && has64) return 64;  // e.g. one gate per attention head: a streaming kernel, bound by reading A
  if (N <= 128) return 128;
  int sms = sm_count();
  if (opt.max_ctas > 0 && opt.max_ctas < sms) sms = opt.max_ctas;
  const int cta_group = opt.cta_group == 2 ? 2 : 1;
  const long long clusters = sms / cta_group > 0 ? sms / cta_group : 1;
  const long long tiles_m = (M + kBlockM * cta_group - 1) / (kBlockM * cta_group);
  const long long w256 = (tiles_m * ((N + 255) / 256) + clusters - 1) / clusters;
  const long long w128 = (tiles_m * ((N + 127) / 128) + clusters - 1) / clusters;
  // Cost in units of one 256-wide wave.  A 128-wide wave costs about 0.75 of it, not 0.5: with N = 128 each MMA
  // reads as many operand bytes from shared memory per cycle as the SM can deliver (measured: forcing the narrow
  // tile on 6144- and 5120-wide outputs lost 10-15 % of a step), so it only pays for narrow or single-wave outputs.
  return (w128 * 0.75 < w256 * 0.97) ? 128 : 256;
}

// Dispatch on CTA grouping, operand majors and (if kNarrow) column-tile width.
// kAllowMajors: bit0 = allow A MN-major, bit1 = allow B MN-major.  kNarrow: 0 = 256-column tiles only, 1 = also
// 128, 2 = also 128 and (for K-major x K-major operands) 64.
// The caller has encoded the output tensor maps of `ep`; `ep.use_tma` is filled in here from the options.
template <class Epi, int kAllowMajors, int kNarrow = 0>
int launch_gemm(const Operand& A, const Operand& B, int M, int N, int K, typename Epi::Params& ep, int* status,
                cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return fail(kBadArgument, "GEMM extents must be positive");
  if (status == nullptr) return fail(kBadArgument, "device status word is required");
  bool a_mn, b_mn;
  long long lda, ldb;
  if (!classify(A, M, K, &a_mn, &lda)) return fail(kBadLayout, "A must be contiguous along one of its two dimensions");
  if (!classify(B, N, K, &b_mn, &ldb)) return fail(kBadLayout, "B must be contiguous along one of its two dimensions");
  const LaunchOptions opt = launch_options();
  ep.use_tma = opt.epi_tma;
  const bool two = opt.cta_group == 2;
  int tile_n = 256;
  if constexpr (kNarrow > 0) tile_n = choose_tile_n(M, N, opt, kNarrow == 2 && !a_mn && !b_mn);
  if constexpr (has_split_tail<Epi>::value) {
    // with a workspace, a wide output whose tiles do not fill the last round is balanced by splitting that round's
    // tiles instead of by narrower tiles
    const int group = two ? 2 : 1;
    const long long tiles256 = static_cast<long long>((M + kBlockM * group - 1) / (kBlockM * group)) * ((N + 255) / 256);
    int tail = 0;
    if (opt.split_tail != 0 && ep.ws != nullptr && N > 128 &&
        plan_tail_split(tiles256, (K + kBlockK - 1) / kBlockK, full_clusters(opt, group), &tail) > 1)
      tile_n = 256;
  }
#define CB_LAUNCH_BN(BN, AM, BM)                                                                                   \
  (two ? launch_gemm_cfg<2, BN, AM, BM, Epi>(A.ptr, lda, B.ptr, ldb, M, N, K, ep, status, stream, opt)               \
       : launch_gemm_cfg<1, BN, AM, BM, Epi>(A.ptr, lda, B.ptr, ldb, M, N, K, ep, status, stream, opt))
#define CB_LAUNCH(AM, BM)                                                \
  do {                                                                   \
    if constexpr (kNarrow > 0) {                                         \
      if (tile_n == 128) return CB_LAUNCH_BN(128, AM, BM);               \
    }                                                                    \
    return CB_LAUNCH_BN(256, AM, BM);                                    \
  } while (0)
  if (!a_mn && !b_mn) {
    if constexpr (kNarrow == 2) {
      if (tile_n == 64) return CB_LAUNCH_BN(64, false, false);
    }
    CB_LAUNCH(false, false);
  }
  if constexpr ((kAllowMajors & 2) != 0) {
    if (!a_mn && b_mn) CB_LAUNCH(false, true);
  }
  if constexpr ((kAllowMajors & 1) != 0) {
    if (a_mn && !b_mn) CB_LAUNCH(true, false);
  }
  if constexpr (kAllowMajors == 3) {
    if (a_mn && b_mn) CB_LAUNCH(true, true);
  }
#undef CB_LAUNCH
#undef CB_LAUNCH_BN
  return fail(kBadLayout, "this fused GEMM needs both operands contiguous along the contraction dimension");
}

}  // namespace cb
