// Fused epilogues for the tcgen05 GEMM core.  With the 32x32b TMEM load shape
// every epilogue thread owns one accumulator row and reads runs of 32
// consecutive fp32 columns, so gate/up pairs, whole attention heads and the
// row-wise max / sum-exp of a tile are all thread-local: no shuffles needed.
//
// Output path: TMEM -> registers -> fused math -> the warp's staging ring in
// shared memory (swizzled so that the 16-byte pieces of 8 neighbouring rows
// fall into different banks) -> one TMA store per 32-row x 32-column sub-tile,
// clipped by the hardware at the matrix edges.  The TMEM load of chunk i+1 is
// issued before the math of chunk i.  Each Params carries `use_tma`; with 0 the
// epilogue writes with per-thread 16-byte global stores instead (kept as the
// comparison path and for callers whose output cannot be described by a
// tensor map).
//
// Each epilogue provides
//   struct Params                          plain-old-data kernel argument (holds the output tensor maps)
//   template <int kBN> static void run(p, ctx)   once per tile per epilogue thread
#pragma once

#include "gemm_core.cuh"

namespace cb {

// Store 32 consecutive values of one row, 16 bytes at a time, predicated on the
// column tail.  `ncols` = number of valid columns starting at v[0] (a multiple of 8).
__device__ __forceinline__ void store_row32(__nv_bfloat16* dst, const float* v, int ncols) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (j * 8 < ncols) {
      uint4 u;
      u.x = pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]);
      u.y = pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]);
      u.z = pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]);
      u.w = pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]);
      *reinterpret_cast<uint4*>(dst + j * 8) = u;
    }
  }
}
__device__ __forceinline__ void store_row32(float* dst, const float* v, int ncols) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (j * 4 < ncols) {
      *reinterpret_cast<float4*>(dst + j * 4) = make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
    }
  }
}

// ------------------------------------------------------------------ staging ring + TMA store
// Address of 16-byte piece `piece` of row `row` inside a staged sub-tile whose rows are kRowBytes long, in the
// swizzle mode a tensor map with that inner box width uses (32-, 64- or 128-byte swizzle: the piece index is XORed
// with the address bits three positions above it).  `tile` must be aligned to 8 rows (256 / 512 / 1024 bytes).
template <int kRowBytes>
__device__ __forceinline__ uint32_t stage_addr(uint32_t tile, int row, int piece) {
  static_assert(kRowBytes == 32 || kRowBytes == 64 || kRowBytes == 128, "row width of a staged sub-tile");
  if constexpr (kRowBytes == 128) return tile + row * 128 + ((piece ^ (row & 7)) << 4);
  else if constexpr (kRowBytes == 64) return tile + row * 64 + ((piece ^ ((row >> 1) & 3)) << 4);
  else return tile + row * 32 + ((piece ^ ((row >> 2) & 1)) << 4);
}

// kCount consecutive values of this lane's row as bf16 (kCount = 32: 64-byte rows, 16: 32-byte rows).
template <int kCount>
__device__ __forceinline__ void stage_row_bf16(uint32_t tile, int lane, const float* v) {
#pragma unroll
  for (int j = 0; j < kCount / 8; ++j)
    st_shared_v4(stage_addr<kCount * 2>(tile, lane, j), pack_bf16x2(v[j * 8 + 0], v[j * 8 + 1]), pack_bf16x2(v[j * 8 + 2], v[j * 8 + 3]),
                 pack_bf16x2(v[j * 8 + 4], v[j * 8 + 5]), pack_bf16x2(v[j * 8 + 6], v[j * 8 + 7]));
}
// 32 consecutive fp32 values of this lane's row (128-byte rows).
__device__ __forceinline__ void stage_row_f32(uint32_t tile, int lane, const float* v) {
#pragma unroll
  for (int j = 0; j < 8; ++j)
    st_shared_v4(stage_addr<128>(tile, lane, j), __float_as_uint(v[j * 4]), __float_as_uint(v[j * 4 + 1]),
                 __float_as_uint(v[j * 4 + 2]), __float_as_uint(v[j * 4 + 3]));
}
__device__ __forceinline__ void stage_row(uint32_t tile, int lane, const float* v, __nv_bfloat16*) { stage_row_bf16<32>(tile, lane, v); }
__device__ __forceinline__ void stage_row(uint32_t tile, int lane, const float* v, float*) { stage_row_f32(tile, lane, v); }

// Claim the next slot of the warp's ring: the TMA store that last read it (two groups ago) must have finished reading.
__device__ __forceinline__ uint32_t ring_acquire(const EpiCtx& c) {
  if (c.lane == 0) tma_store_wait_read<kRingSlots - 1>();
  __syncwarp();
  return c.ring + c.slot * kRingSlotBytes;
}
// Every lane has written its row: make the writes visible to the TMA engine.  Lane 0 then issues the stores.
__device__ __forceinline__ void ring_publish() {
  fence_proxy_async_smem();
  __syncwarp();
}
// One TMA store of a staged sub-tile to rows row0 .. row0+31, columns from x (issued by lane 0).  A warp whose rows all
// lie below the matrix issues nothing.
__device__ __forceinline__ void store_tile(const EpiCtx& c, const CUtensorMap* m, uint32_t tile, int x) {
  if (c.row0 < c.M) tma_store_2d(m, tile, x, c.row0);
}
// Close the bulk group of this slot (lane 0) and move on.
__device__ __forceinline__ void ring_commit(EpiCtx& c) {
  if (c.lane == 0) tma_store_commit();
  c.slot = (c.slot + 1 == kRingSlots) ? 0u : c.slot + 1;
}

// ------------------------------------------------------------------ second-operand tiles by TMA
// Lane 0 arms the slot's mbarrier and issues `nboxes` (1 or 2) loads of 32-row x 32-column bf16 boxes at columns
// x, x + 32 of rows row0 .. row0 + 31 into load slot `s`; they land in the 64-byte swizzle, 2 KB per box, with rows and
// columns outside the matrix zero-filled.  Every lane of the warp must have finished reading the slot's previous
// contents (the caller places a __syncwarp between the last read and this call).
__device__ __forceinline__ void operand_issue(const EpiCtx& c, int s, const CUtensorMap* m0, int x0, const CUtensorMap* m1, int x1) {
  if (c.lane == 0) {
    const uint32_t bar = c.ld_bar + 8 * s;
    const uint32_t dst = c.ld_ring + s * kLoadSlotBytes;
    mbar_arrive_expect_tx(bar, m1 != nullptr ? 4096u : 2048u);
    tma_load_2d(dst, m0, bar, x0, c.row0);
    if (m1 != nullptr) tma_load_2d(dst + 2048, m1, bar, x1, c.row0);
  }
}
// All lanes: wait (bounded) until the loads of slot `s` have landed; flips the slot's parity.  Returns false if the
// wait expired (the code is in the abort word; the caller carries on with whatever the slot holds).
__device__ __forceinline__ bool operand_wait(EpiCtx& c, int s) {
  const uint32_t parity = (c.ld_phase >> s) & 1u;
  c.ld_phase ^= (1u << s);
  return mbar_wait(c.ld_bar + 8 * s, parity, c.abort_word, kErrTimeoutEpiLoad);
}
// This lane's row of box `box` (0 or 1) of slot `s`: 32 bf16 -> fp32.
__device__ __forceinline__ void operand_row32(const EpiCtx& c, int s, int box, float* v) {
  const uint32_t tile = c.ld_ring + s * kLoadSlotBytes + box * 2048;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint4 u = ld_shared_v4(stage_addr<64>(tile, c.lane, j));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      v[j * 8 + 2 * k] = __uint_as_float(w[k] << 16);
      v[j * 8 + 2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
    }
  }
}

// Calls f(ch, v) for ch = 0 .. n-1 with v = accumulator columns [32 ch, 32 ch + 32) of this thread's row.  Two
// register buffers: the TMEM load of chunk ch+1 is in flight while f works on chunk ch.  `n` is warp-uniform.
template <class F>
__device__ __forceinline__ void for_chunks(uint32_t taddr, int n, F&& f) {
  if (n <= 0) return;
  float va[32], vb[32];
  tmem_ld32(taddr, va);
#pragma unroll 1
  for (int ch = 0; ch < n; ch += 2) {
    tmem_ld_wait();
    if (ch + 1 < n) tmem_ld32(taddr + (ch + 1) * 32, vb);
    f(ch, va);
    if (ch + 1 < n) {
      tmem_ld_wait();
      if (ch + 2 < n) tmem_ld32(taddr + (ch + 2) * 32, va);
      f(ch + 1, vb);
    }
  }
}

// Number of 32-column chunks of a kBN-wide tile starting at column n0 that hold at least one valid column.
template <int kBN>
__device__ __forceinline__ int valid_chunks(int n0, int N) {
  const int left = N - n0;
  return left >= kBN ? kBN / 32 : (left + 31) / 32;
}

// 32 consecutive elements of a second [M, N] operand row (bf16 or fp32) as fp32; pieces beyond `ncols` read as zero.
__device__ __forceinline__ void load_row32_any(const void* base, int is_fp32, long long elem_off, float* v, int ncols, bool row_ok) {
  if (is_fp32) {
    const float* src = static_cast<const float*>(base) + elem_off;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row_ok && j * 4 < ncols) f = *reinterpret_cast<const float4*>(src + j * 4);
      v[j * 4] = f.x; v[j * 4 + 1] = f.y; v[j * 4 + 2] = f.z; v[j * 4 + 3] = f.w;
    }
  } else {
    const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(base) + elem_off;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 u = make_uint4(0u, 0u, 0u, 0u);
      if (row_ok && j * 8 < ncols) u = *reinterpret_cast<const uint4*>(src + j * 8);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = unpack_bf16x2(w[k]);
        v[j * 8 + 2 * k] = f.x;
        v[j * 8 + 2 * k + 1] = f.y;
      }
    }
  }
}

// ------------------------------------------------------------------ plain / sigmoid
// D = act(alpha * acc + C).  Replaces the reference's `_gemm`, the `C=` form of `gemm` (quack_gemm_add),
// `_gemm_scalar_scale_epi` and `_gemm_sigmoid_epi` (coda/core/gemm/functional.py:35-69, 94-113, 199-217).
enum class Act { kNone, kSigmoid };

template <typename OutT, Act kAct>
struct EpiStore {
  static constexpr uint32_t kLoadRingBytes = 0;
  static constexpr bool kSplitTail = true;  // can park a partial accumulator in the tail-split workspace
  struct Params {
    alignas(64) CUtensorMap tm_d;   // D as [M, N], box 32 x 32
    alignas(64) CUtensorMap tm_ws;  // tail-split workspace as [slabs * tile rows, kBN] fp32, box 32 x 32 (unused otherwise)
    OutT* D;
    long long ldd;
    const float* alpha;  // device scalar or nullptr (= 1)
    const void* C;       // [M, N] addend (bf16 or fp32) or nullptr; may alias D
    long long ldc;
    int c_is_fp32;
    int use_tma;
    float* ws = nullptr;     // host side: tail-split workspace offered by the caller (nullptr: whole tiles only)
    long long ws_bytes = 0;
  };

  template <int kBN>
  __device__ static void run(const Params& p, EpiCtx& c) {
    if (c.part_row0 >= 0) {
      // One part of a tail tile: the raw fp32 accumulator goes to its workspace slab (always through the staging
      // ring and TMA stores; the slab is a whole tile, so nothing is clipped).  alpha, the conversion and the store
      // to D happen when the parts are added.
      for_chunks(c.taddr, kBN / 32, [&](int ch, float* v) {
        const uint32_t tile = ring_acquire(c);
        stage_row_f32(tile, c.lane, v);
        ring_publish();
        if (c.lane == 0) tma_store_2d(&p.tm_ws, tile, ch * 32, c.part_row0);
        ring_commit(c);
      });
      return;
    }
    const float alpha = p.alpha ? __ldg(p.alpha) : 1.0f;
    const bool row_ok = c.row < c.M;
    OutT* drow = p.D + static_cast<long long>(c.row) * p.ldd + c.n0;
    for_chunks(c.taddr, valid_chunks<kBN>(c.n0, c.N), [&](int ch, float* v) {
      const int col = c.n0 + ch * 32;
      if (p.C != nullptr) {
        float t[32];
        load_row32_any(p.C, p.c_is_fp32, static_cast<long long>(c.row) * p.ldc + col, t, c.N - col, row_ok);
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = fmaf(v[j], alpha, t[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= alpha;
      }
      if constexpr (kAct == Act::kSigmoid) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = fast_sigmoid(v[j]);
      }
      if (p.use_tma) {
        const uint32_t tile = ring_acquire(c);
        stage_row(tile, c.lane, v, static_cast<OutT*>(nullptr));
        ring_publish();
        if (c.lane == 0) store_tile(c, &p.tm_d, tile, col);
        ring_commit(c);
      } else if (row_ok) {
        store_row32(drow + ch * 32, v, c.N - col);
      }
    });
  }
};

// ------------------------------------------------------------------ SwiGLU
// preact[:, c] = bf16(acc[:, c]); postact[:, j] = bf16(silu(acc[:, 2j]) * acc[:, 2j+1]),
// both from the unrounded accumulator.  Replaces `_gemm_swiglu_epi`
// (coda/core/gemm/functional.py:237-258, epilogue coda/core/gemm/epilogues.py:44-47).
// kSigmoidGate selects the gate: silu(gate) * up (SwiGLU, the reference op) or sigmoid(gate) * up (a plain sigmoid
// gate on a value projection: the "gated projection" reading of the sigmoid benchmark configuration, an extension
// with no counterpart in the reference).
template <bool kSigmoidGate>
struct EpiGated {
  static constexpr uint32_t kLoadRingBytes = 0;
  struct Params {
    alignas(64) CUtensorMap tm_pre;   // preact as [M, N], box 32 x 32
    alignas(64) CUtensorMap tm_post;  // postact as [M, N/2], box 16 x 32
    __nv_bfloat16* preact;  // [M, N]
    long long ld_pre;
    __nv_bfloat16* postact;  // [M, N/2]
    long long ld_post;
    const float* row_scale;  // [M] fp32 or nullptr: acc is multiplied by row_scale[row] first (deferred RMSNorm)
    int use_tma;
  };

  template <int kBN>
  __device__ static void run(const Params& p, EpiCtx& c) {
    const bool row_ok = c.row < c.M;
    const float rs = (p.row_scale != nullptr && row_ok) ? __ldg(p.row_scale + c.row) : 1.0f;
    __nv_bfloat16* pre = p.preact + static_cast<long long>(c.row) * p.ld_pre + c.n0;
    __nv_bfloat16* post = p.postact + static_cast<long long>(c.row) * p.ld_post + c.n0 / 2;
    for_chunks(c.taddr, valid_chunks<kBN>(c.n0, c.N), [&](int ch, float* v) {
      const int col = c.n0 + ch * 32;
      float o[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float g = v[2 * j] * rs, u = v[2 * j + 1] * rs;
        v[2 * j] = g;
        v[2 * j + 1] = u;
        o[j] = kSigmoidGate ? fast_sigmoid(g) * u : g * fast_sigmoid(g) * u;
      }
      if (p.use_tma) {
        const uint32_t tile = ring_acquire(c);  // [preact 32 x 64 B | postact 32 x 32 B]
        stage_row_bf16<32>(tile, c.lane, v);
        stage_row_bf16<16>(tile + 2048, c.lane, o);
        ring_publish();
        if (c.lane == 0) {
          store_tile(c, &p.tm_pre, tile, col);
          store_tile(c, &p.tm_post, tile + 2048, col / 2);
        }
        ring_commit(c);
      } else if (row_ok) {
        const int ncols = c.N - col;
        store_row32(pre + ch * 32, v, ncols);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          if (j * 16 < ncols) {  // N is a multiple of 16 for this op, so half-chunks are all-or-nothing
            uint4 u4;
            u4.x = pack_bf16x2(o[j * 8 + 0], o[j * 8 + 1]);
            u4.y = pack_bf16x2(o[j * 8 + 2], o[j * 8 + 3]);
            u4.z = pack_bf16x2(o[j * 8 + 4], o[j * 8 + 5]);
            u4.w = pack_bf16x2(o[j * 8 + 6], o[j * 8 + 7]);
            *reinterpret_cast<uint4*>(post + ch * 16 + j * 8) = u4;
          }
        }
      }
    });
  }
};

using EpiSwiGLU = EpiGated<false>;
using EpiSigmoidGLU = EpiGated<true>;

// ------------------------------------------------------------------ log-sum-exp partials (+ optional probability store)
// Per (row, column-tile): m = max_j acc, s = sum_j exp(acc - m).  The tile that
// contains the row's target column also records that logit (fp32, unrounded).
// kStore selects what else is written: kLseStoreNone nothing; kLseStoreProbs the
// tile's unnormalised probabilities exp(acc - m) in bf16, so that the backward
// never needs the logits (a later in-place pass rescales them by exp(m - lse)
// and subtracts the one-hot); kLseStoreLogits the bf16 logits themselves, the
// reference's own dataflow.  Replaces `_gemm_lse_epi` / `_lse_select_logits_epi`
// (coda/core/gemm/functional.py:342-368, 453-493).
constexpr int kLseStoreNone = 0, kLseStoreProbs = 1, kLseStoreLogits = 2;

template <int kStore>
struct EpiLse {
  static constexpr uint32_t kLoadRingBytes = 0;
  struct Params {
    alignas(64) CUtensorMap tm_p;  // P as [M, N], box 32 x 32 (unused for kLseStoreNone)
    __nv_bfloat16* P;  // [M, N] or nullptr
    long long ldp;
    float* part_max;  // [M, tiles_n]
    float* part_sum;  // [M, tiles_n]
    int tiles_n;
    const int* target;    // [M] or nullptr (no target pick)
    float* target_logit;  // [M]; written only by the tile holding the target column
    const float* row_scale;  // [M] fp32 or nullptr: logits = acc * row_scale[row] (deferred RMSNorm)
    float* part_sz;          // [M, tiles_n] or nullptr: sum_j exp(z_j - m) * z_j, for sum_j z_j * dlogit_j
    int use_tma;
  };

  template <int kBN>
  __device__ static void run(const Params& p, EpiCtx& c) {
    const bool row_ok = c.row < c.M;
    const int nvalid = min(kBN, c.N - c.n0);  // valid columns in this tile (>= 1)
    const int nch = (nvalid + 31) / 32;
    constexpr float kLog2e = 1.4426950408889634f;
    const float rs = (p.row_scale != nullptr && row_ok) ? __ldg(p.row_scale + c.row) : 1.0f;
    // pass 1: row maximum over the tile (of the raw accumulator; the row scale is positive)
    float mx = -INFINITY;
    for_chunks(c.taddr, nch, [&](int ch, float* v) {
      const int lim = nvalid - ch * 32;
      if (lim >= 32) {
#pragma unroll
        for (int j = 0; j < 32; ++j) mx = fmaxf(mx, v[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j < lim) mx = fmaxf(mx, v[j]);
      }
    });
    mx *= rs;
    // pass 2: exponentials, their sum, target logit, optional store
    const int tgt = (row_ok && p.target != nullptr) ? __ldg(p.target + c.row) : -1;
    const int tcol = tgt - c.n0;  // target column relative to this tile
    float sum = 0.f, tlogit = 0.f, sz = 0.f;
    const bool want_sz = p.part_sz != nullptr;
    __nv_bfloat16* prow = (kStore != kLseStoreNone) ? p.P + static_cast<long long>(c.row) * p.ldp + c.n0 : nullptr;
    const float mxs = mx * kLog2e;
    const float rsl = rs * kLog2e;
    for_chunks(c.taddr, nch, [&](int ch, float* v) {
      const int lim = nvalid - ch * 32;
      const int trel = tcol - ch * 32;
      if (trel >= 0 && trel < 32) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (j == trel) tlogit = v[j] * rs;
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float e = (j < lim) ? fast_exp2(fmaf(v[j], rsl, -mxs)) : 0.f;
        sum += e;
        if (want_sz) sz = fmaf(e, v[j] * rs, sz);
        v[j] = (kStore == kLseStoreLogits) ? v[j] * rs : e;
      }
      if constexpr (kStore != kLseStoreNone) {
        if (p.use_tma) {
          const uint32_t tile = ring_acquire(c);
          stage_row_bf16<32>(tile, c.lane, v);
          ring_publish();
          if (c.lane == 0) store_tile(c, &p.tm_p, tile, c.n0 + ch * 32);
          ring_commit(c);
        } else if (row_ok) {
          store_row32(prow + ch * 32, v, lim);
        }
      }
    });
    if (row_ok) {
      p.part_max[static_cast<long long>(c.row) * p.tiles_n + c.tn] = mx;
      p.part_sum[static_cast<long long>(c.row) * p.tiles_n + c.tn] = sum;
      if (want_sz) p.part_sz[static_cast<long long>(c.row) * p.tiles_n + c.tn] = sz;
      if (tcol >= 0 && tcol < nvalid) p.target_logit[c.row] = tlogit;
    }
  }
};

// ------------------------------------------------------------------ per-head RMSNorm + RoPE on q,k; plain store for v
// Columns are [q heads | k heads | v heads], each head kHD wide.  For q and k:
//   ms = mean(acc^2) over the head (fp32, unrounded acc), r = rsqrt(ms + eps)
//   y  = acc * gamma * r;  (y0, y1) at columns (2p, 2p+1) rotated by the angle
//   2*pi*frac(pos * (hi + lo)) with (hi, lo) = frequencies[2p], frequencies[2p+1]
//   evaluated with the two-term product so that large positions stay accurate.
// Outputs: rotated qk, bf16 preact, ms; v columns are stored unchanged.
// Replaces `_gemm_qknorm_rope_epi` + the separate v GEMM
// (coda/core/gemm/functional.py:1079-1152, coda/core/gemm/epilogues.py:232-259,
// angle scheme coda/core/ops/math_utils.py:181-195).
template <int kHD>
struct EpiQKNormRope {
  static constexpr uint32_t kLoadRingBytes = 0;
  struct Params {
    alignas(64) CUtensorMap tm_qk;   // qk as [M, size_qk], box 32 x 32
    alignas(64) CUtensorMap tm_pre;  // preact as [M, size_qk], box 32 x 32
    alignas(64) CUtensorMap tm_v;    // v as [M, size_v], box 32 x 32 (unused without v columns)
    __nv_bfloat16* qk;  // [M, size_qk]
    long long ld_qk;
    __nv_bfloat16* preact;  // [M, size_qk]
    long long ld_pre;
    __nv_bfloat16* v;  // [M, size_v] or nullptr when N == size_qk
    long long ld_v;
    float* mean_sq;              // [M, hq + hk]
    const __nv_bfloat16* gamma;  // [2 * kHD] = [gamma_q | gamma_k]
    const void* positions;       // [M] int32 or fp32
    int pos_is_float;
    const float* freq;  // [(hq + hk) * kHD] interleaved (hi, lo)
    int hq, hk;
    float eps;
    const float* row_scale;  // [M] fp32 or nullptr: q, k (statistic and output) and v use acc * row_scale[row]; preact keeps acc
    int use_tma;
  };

  template <int kBN>
  __device__ static void run(const Params& p, EpiCtx& c) {
    const bool row_ok = c.row < c.M;
    const int safe_row = row_ok ? c.row : 0;
    const float pos = p.pos_is_float ? __ldg(reinterpret_cast<const float*>(p.positions) + safe_row)
                                     : static_cast<float>(__ldg(reinterpret_cast<const int*>(p.positions) + safe_row));
    const int nheads_qk = p.hq + p.hk;
    constexpr float kTwoPi = 6.283185307179586f;
    constexpr int kChunks = kHD / 32;
    const float rs = (p.row_scale != nullptr && row_ok) ? __ldg(p.row_scale + c.row) : 1.0f;
#pragma unroll 1
    for (int h = 0; h < kBN / kHD; ++h) {
      const int col0 = c.n0 + h * kHD;
      if (col0 >= c.N) break;
      const int head = col0 / kHD;
      const uint32_t t0 = c.taddr + h * kHD;
      if (head >= nheads_qk) {
        // v head: plain bf16 store
        const int vcol0 = col0 - nheads_qk * kHD;
        __nv_bfloat16* vrow = p.v + static_cast<long long>(c.row) * p.ld_v + vcol0;
        for_chunks(t0, kChunks, [&](int ch, float* v) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= rs;
          if (p.use_tma) {
            const uint32_t tile = ring_acquire(c);
            stage_row_bf16<32>(tile, c.lane, v);
            ring_publish();
            if (c.lane == 0) store_tile(c, &p.tm_v, tile, vcol0 + ch * 32);
            ring_commit(c);
          } else if (row_ok) {
            store_row32(vrow + ch * 32, v, 32);
          }
        });
        continue;
      }
      // pass 1: mean square of the head
      float ss = 0.f;
      for_chunks(t0, kChunks, [&](int, float* v) {
#pragma unroll
        for (int j = 0; j < 32; ++j) ss = fmaf(v[j], v[j], ss);
      });
      const float ms = ss * (1.0f / kHD) * rs * rs;  // statistic of acc * row_scale
      const float r = rsqrtf(ms + p.eps) * rs;
      if (row_ok) p.mean_sq[static_cast<long long>(c.row) * nheads_qk + head] = ms;
      const __nv_bfloat16* gam = p.gamma + (head < p.hq ? 0 : kHD);
      __nv_bfloat16* prow = p.preact + static_cast<long long>(c.row) * p.ld_pre + col0;
      __nv_bfloat16* orow = p.qk + static_cast<long long>(c.row) * p.ld_qk + col0;
      // pass 2: normalise, rotate, store
      for_chunks(t0, kChunks, [&](int ch, float* v) {
        uint32_t tile = 0;
        if (p.use_tma) {
          tile = ring_acquire(c);  // [preact 32 x 64 B | rotated 32 x 64 B]
          stage_row_bf16<32>(tile, c.lane, v);
        } else if (row_ok) {
          store_row32(prow + ch * 32, v, 32);
        }
        // gamma and the (hi, lo) frequency pairs of these 32 columns: the same addresses in every lane, 16 bytes per load
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const int e8 = ch * 32 + q4 * 8;  // element index inside the head
          const uint4 g4 = __ldg(reinterpret_cast<const uint4*>(gam + e8));
          const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            const float4 f4 = __ldg(reinterpret_cast<const float4*>(p.freq + col0 + e8 + 4 * h2));
            const float fh[2] = {f4.x, f4.z}, fl[2] = {f4.y, f4.w};
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              const int j = q4 * 4 + h2 * 2 + k;
              const float2 g = unpack_bf16x2(gw[h2 * 2 + k]);
              const float y0 = v[2 * j] * g.x * r;
              const float y1 = v[2 * j + 1] * g.y * r;
              const float t = pos * fh[k];
              const float terr = fmaf(pos, fh[k], -t);
              const float l = fmaf(pos, fl[k], terr);
              const float frac = (t - rintf(t)) + l;
              float sn, cs;
              __sincosf(kTwoPi * frac, &sn, &cs);
              v[2 * j] = y0 * cs - y1 * sn;
              v[2 * j + 1] = y0 * sn + y1 * cs;
            }
          }
        }
        if (p.use_tma) {
          stage_row_bf16<32>(tile + 2048, c.lane, v);
          ring_publish();
          if (c.lane == 0) {
            store_tile(c, &p.tm_pre, tile, col0 + ch * 32);
            store_tile(c, &p.tm_qk, tile + 2048, col0 + ch * 32);
          }
          ring_commit(c);
        } else if (row_ok) {
          store_row32(orow + ch * 32, v, 32);
        }
      });
    }
  }
};

}  // namespace cb
