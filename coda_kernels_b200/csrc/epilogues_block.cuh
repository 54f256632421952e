// Epilogues of the GEMMs that sit between the fused-linear operators inside a transformer layer: the residual add
// with deferred RMSNorm, its backward, and the down-projection dgrad that runs the SwiGLU derivative in place of a
// separate element-wise pass.  Same conventions as epilogues.cuh: one accumulator row per epilogue thread.
#pragma once

#include "epilogues.cuh"

namespace cb {

// 32 consecutive bf16 of one row -> fp32, 16 bytes at a time; groups of 8 beyond `ncols` read as zero.
__device__ __forceinline__ void load_row32(const __nv_bfloat16* src, float* v, int ncols, bool row_ok) {
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

// Same address for every lane of the warp (a per-column vector): read through the read-only path.
__device__ __forceinline__ void load_colvec32(const __nv_bfloat16* src, float* v, int ncols) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 u = make_uint4(0u, 0u, 0u, 0u);
    if (j * 8 < ncols) u = __ldg(reinterpret_cast<const uint4*>(src + j * 8));
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = unpack_bf16x2(w[k]);
      v[j * 8 + 2 * k] = f.x;
      v[j * 8 + 2 * k + 1] = f.y;
    }
  }
}

// ------------------------------------------------------------------ RoPE on every column (v columns carry frequency 0)
// D = rotate(acc * row_scale[row]) with the angle of each adjacent column pair taken from `freq` (hi, lo turns) and
// the row's position.  Replaces `_gemm_rope_epi` / `_gemm_rmsnorm_rope_epi` (coda/core/gemm/functional.py:955-1062).
struct EpiRope {
  static constexpr uint32_t kLoadRingBytes = 0;
  struct Params {
    alignas(64) CUtensorMap tm_d;  // D as [M, N], box 32 x 32
    __nv_bfloat16* D;
    long long ldd;
    const float* row_scale;  // [M] or nullptr
    const void* positions;   // [M] int32 or fp32
    int pos_is_float;
    const float* freq;  // [N]
    int use_tma;
  };

  template <int kBN>
  __device__ static void run(const Params& p, EpiCtx& c) {
    constexpr float kTwoPi = 6.283185307179586f;
    const bool row_ok = c.row < c.M;
    const int safe_row = row_ok ? c.row : 0;
    const float rs = (p.row_scale != nullptr && row_ok) ? __ldg(p.row_scale + c.row) : 1.0f;
    const float pos = p.pos_is_float ? __ldg(reinterpret_cast<const float*>(p.positions) + safe_row)
                                     : static_cast<float>(__ldg(reinterpret_cast<const int*>(p.positions) + safe_row));
    for_chunks(c.taddr, valid_chunks<kBN>(c.n0, c.N), [&](int ch, float* v) {
      const int col = c.n0 + ch * 32;
      const int ncols = c.N - col;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float2 f = make_float2(0.f, 0.f);
        if (2 * j < ncols) f = __ldg(reinterpret_cast<const float2*>(p.freq + col + 2 * j));
        const float t = pos * f.x;
        const float terr = fmaf(pos, f.x, -t);
        const float l = fmaf(pos, f.y, terr);
        const float frac = (t - rintf(t)) + l;
        float sn, cs;
        __sincosf(kTwoPi * frac, &sn, &cs);
        const float a = v[2 * j] * rs, b = v[2 * j + 1] * rs;
        v[2 * j] = a * cs - b * sn;
        v[2 * j + 1] = a * sn + b * cs;
      }
      if (p.use_tma) {
        const uint32_t tile = ring_acquire(c);
        stage_row_bf16<32>(tile, c.lane, v);
        ring_publish();
        if (c.lane == 0) store_tile(c, &p.tm_d, tile, col);
        ring_commit(c);
      } else if (row_ok) {
        store_row32(p.D + static_cast<long long>(c.row) * p.ldd + col, v, ncols);
      }
    });
  }
};

// ------------------------------------------------------------------ residual add + partial RMSNorm
// pre = acc + C;  post = pre * weight[col];  per (row, column tile) sum of pre^2 (fp32, unrounded).  The row's
// rstd = rsqrt(sum / N + eps) is formed afterwards and applied by the GEMM that consumes `post`.  Replaces
// `_gemm_residual_partial_rmsnorm_epi` (coda/core/gemm/functional.py:573-613; epilogues.py:72-80).
struct EpiResidualNorm {
  static constexpr uint32_t kLoadRingBytes = kLoadRingBytesPerWarp;
  struct Params {
    alignas(64) CUtensorMap tm_pre;   // pre as [M, N], box 32 x 32
    alignas(64) CUtensorMap tm_post;  // post as [M, N], box 32 x 32
    alignas(64) CUtensorMap tm_c;     // C as [M, N], box 32 x 32 (load)
    const __nv_bfloat16* C;  // [M, N] residual (may alias pre or post)
    long long ldc;
    __nv_bfloat16* pre;  // [M, N]
    long long ld_pre;
    __nv_bfloat16* post;  // [M, N]
    long long ld_post;
    const __nv_bfloat16* weight;  // [N]
    float* part_sq;               // [M, tiles_n]
    int tiles_n;
    int use_tma;
  };

  template <int kBN>
  __device__ static void run(const Params& p, EpiCtx& c) {
    const bool row_ok = c.row < c.M;
    const long long r = c.row;
    float sq = 0.f;
    const int n = valid_chunks<kBN>(c.n0, c.N);
    if (p.use_tma) operand_issue(c, 0, &p.tm_c, c.n0, nullptr, 0);
    for_chunks(c.taddr, n, [&](int ch, float* v) {
      const int col = c.n0 + ch * 32;
      const int ncols = c.N - col;
      float t[32];
      if (p.use_tma) {
        __syncwarp();  // every lane is done with the slot the next load goes to
        if (ch + 1 < n) operand_issue(c, (ch + 1) & 1, &p.tm_c, col + 32, nullptr, 0);
        operand_wait(c, ch & 1);
        operand_row32(c, ch & 1, 0, t);
      } else {
        load_row32(p.C + r * p.ldc + col, t, ncols, row_ok);
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        v[j] += t[j];
        if (j < ncols) sq = fmaf(v[j], v[j], sq);
      }
      uint32_t tile = 0;
      if (p.use_tma) {
        tile = ring_acquire(c);  // [pre 32 x 64 B | post 32 x 64 B]
        stage_row_bf16<32>(tile, c.lane, v);
      } else if (row_ok) {
        store_row32(p.pre + r * p.ld_pre + col, v, ncols);
      }
      load_colvec32(p.weight + col, t, ncols);
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] *= t[j];
      if (p.use_tma) {
        stage_row_bf16<32>(tile + 2048, c.lane, v);
        ring_publish();
        if (c.lane == 0) {
          store_tile(c, &p.tm_pre, tile, col);
          store_tile(c, &p.tm_post, tile + 2048, col);
        }
        ring_commit(c);
      } else if (row_ok) {
        store_row32(p.post + r * p.ld_post + col, v, ncols);
      }
    });
    if (row_ok) p.part_sq[r * p.tiles_n + c.tn] = sq;
  }
};

// ------------------------------------------------------------------ down-projection dgrad through SwiGLU
// acc = d(postact) [M, F];  Z = stored preact [M, 2F] (gate, up interleaved).  Writes dZ = dswiglu(Z, acc) [M, 2F],
// postact = silu(gate) * up [M, F] (recomputed for the wgrad), and per (row, tile) sum of Z * dZ.  Replaces
// `_gemm_swiglu_bwd_zdz_epi(_scaled)` (coda/core/gemm/functional.py:827-910; epilogues.py:105-127).
struct EpiSwigluBwdZdz {
  static constexpr uint32_t kLoadRingBytes = kLoadRingBytesPerWarp;
  struct Params {
    alignas(64) CUtensorMap tm_dz;    // dZ as [M, 2N], box 32 x 32
    alignas(64) CUtensorMap tm_post;  // postact as [M, N], box 32 x 32
    alignas(64) CUtensorMap tm_z;     // Z as [M, 2N], box 32 x 32 (load)
    const __nv_bfloat16* Z;  // [M, 2N] (may alias dZ)
    long long ldz;
    __nv_bfloat16* dZ;  // [M, 2N]
    long long ld_dz;
    __nv_bfloat16* postact;  // [M, N]
    long long ld_post;
    float* part_zdz;  // [M, tiles_n]
    int tiles_n;
    int use_tma;
  };

  template <int kBN>
  __device__ static void run(const Params& p, EpiCtx& c) {
    const bool row_ok = c.row < c.M;
    const long long r = c.row;
    float zdz = 0.f;
    const int n = valid_chunks<kBN>(c.n0, c.N);
    if (p.use_tma) operand_issue(c, 0, &p.tm_z, 2 * c.n0, &p.tm_z, 2 * c.n0 + 32);
    for_chunks(c.taddr, n, [&](int ch, float* t) {
      const int col = c.n0 + ch * 32;  // column of acc / postact; Z and dZ columns are 2*col ..
      const int ncols = c.N - col;
      float za[32], zb[32];
      if (p.use_tma) {
        __syncwarp();  // every lane is done with the slot the next load goes to
        if (ch + 1 < n) operand_issue(c, (ch + 1) & 1, &p.tm_z, 2 * col + 64, &p.tm_z, 2 * col + 96);
        operand_wait(c, ch & 1);
        operand_row32(c, ch & 1, 0, za);
        operand_row32(c, ch & 1, 1, zb);
      } else {
        load_row32(p.Z + r * p.ldz + 2 * col, za, 2 * ncols, row_ok);
        load_row32(p.Z + r * p.ldz + 2 * col + 32, zb, 2 * ncols - 32, row_ok);
      }
      float out[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float x = (j < 16) ? za[2 * j] : zb[2 * (j - 16)];
        const float y = (j < 16) ? za[2 * j + 1] : zb[2 * (j - 16) + 1];
        const float s = fast_sigmoid(x);
        const float g = t[j];
        const float dx = g * y * (s + x * s * (1.0f - s));
        const float dy = g * x * s;
        out[j] = x * s * y;
        if (j < ncols) zdz = fmaf(dx, x, fmaf(dy, y, zdz));
        if (j < 16) {
          za[2 * j] = dx;
          za[2 * j + 1] = dy;
        } else {
          zb[2 * (j - 16)] = dx;
          zb[2 * (j - 16) + 1] = dy;
        }
      }
      if (p.use_tma) {
        uint32_t tile = ring_acquire(c);  // [dZ first 32 columns | dZ next 32 columns]
        stage_row_bf16<32>(tile, c.lane, za);
        stage_row_bf16<32>(tile + 2048, c.lane, zb);
        ring_publish();
        if (c.lane == 0) {
          store_tile(c, &p.tm_dz, tile, 2 * col);
          if (2 * ncols > 32) store_tile(c, &p.tm_dz, tile + 2048, 2 * col + 32);
        }
        ring_commit(c);
        tile = ring_acquire(c);
        stage_row_bf16<32>(tile, c.lane, out);
        ring_publish();
        if (c.lane == 0) store_tile(c, &p.tm_post, tile, col);
        ring_commit(c);
      } else if (row_ok) {
        store_row32(p.dZ + r * p.ld_dz + 2 * col, za, 2 * ncols);
        store_row32(p.dZ + r * p.ld_dz + 2 * col + 32, zb, 2 * ncols - 32);
        store_row32(p.postact + r * p.ld_post + col, out, ncols);
      }
    });
    if (row_ok) p.part_zdz[r * p.tiles_n + c.tn] = zdz;
  }
};

// ------------------------------------------------------------------ RMSNorm backward on a dgrad
// y = alpha * acc;  n = pre * rstd[row];  dX = (y * weight[col] - n * zdz[row]) * rstd[row] (+ dX if accumulating);
// normed = n * weight[col];  dweight[col] += sum over rows of y * n, delivered as one partial row per 32-row slab
// (each epilogue warp folds its 32 rows with a shuffle transpose-reduce).  Replaces
// `_gemm_residual_partial_rmsnorm_bwd_epi_{store,accum}` (coda/core/gemm/functional.py:655-764; epilogues.py:130-168).
struct EpiRmsnormBwd {
  static constexpr uint32_t kLoadRingBytes = kLoadRingBytesPerWarp;
  struct Params {
    alignas(64) CUtensorMap tm_dx;      // dX as [M, N], box 32 x 32 (store, and load when accumulating)
    alignas(64) CUtensorMap tm_normed;  // normed as [M, N], box 32 x 32
    alignas(64) CUtensorMap tm_pre;     // pre as [M, N], box 32 x 32 (load)
    const __nv_bfloat16* pre;  // [M, N]
    long long ld_pre;
    __nv_bfloat16* dX;  // [M, N]
    long long ld_dx;
    __nv_bfloat16* normed;  // [M, N] (may alias pre)
    long long ld_normed;
    const __nv_bfloat16* weight;  // [N]
    const float* rstd;            // [M]
    const float* zdz;             // [M]
    const float* alpha;           // device scalar or nullptr
    float* part_dw;               // [ceil(M / 32), N]
    int accumulate;
    int use_tma;
  };

  template <int kBN>
  __device__ static void run(const Params& p, EpiCtx& c) {
    const bool row_ok = c.row < c.M;
    const long long r = c.row;
    const float alpha = p.alpha ? __ldg(p.alpha) : 1.0f;
    const float rstd = row_ok ? __ldg(p.rstd + c.row) : 0.f;
    const float zdz = row_ok ? __ldg(p.zdz + c.row) : 0.f;
    const long long slab = c.row0 / 32;  // the warp's 32 rows start at a multiple of 32
    const int n = valid_chunks<kBN>(c.n0, c.N);
    const CUtensorMap* acc_map = p.accumulate ? &p.tm_dx : nullptr;
    if (p.use_tma) operand_issue(c, 0, &p.tm_pre, c.n0, acc_map, c.n0);
    for_chunks(c.taddr, n, [&](int ch, float* y) {
      const int col = c.n0 + ch * 32;
      const int ncols = c.N - col;
      float nn[32], w[32], d[32];
      if (p.use_tma) {
        __syncwarp();  // every lane is done with the slot the next load goes to
        if (ch + 1 < n) operand_issue(c, (ch + 1) & 1, &p.tm_pre, col + 32, acc_map, col + 32);
        operand_wait(c, ch & 1);
        operand_row32(c, ch & 1, 0, nn);
        if (p.accumulate) operand_row32(c, ch & 1, 1, d);
      } else {
        load_row32(p.pre + r * p.ld_pre + col, nn, ncols, row_ok);
        if (p.accumulate) load_row32(p.dX + r * p.ld_dx + col, d, ncols, row_ok);
      }
      load_colvec32(p.weight + col, w, ncols);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        y[j] *= alpha;
        nn[j] *= rstd;
        const float dx = (y[j] * w[j] - nn[j] * zdz) * rstd;
        d[j] = p.accumulate ? d[j] + dx : dx;
        w[j] *= nn[j];     // normed
        y[j] *= nn[j];     // this row's contribution to dweight (zero for rows >= M: acc and pre read as zero)
      }
      if (p.use_tma) {
        const uint32_t tile = ring_acquire(c);  // [dX 32 x 64 B | normed 32 x 64 B]
        stage_row_bf16<32>(tile, c.lane, d);
        stage_row_bf16<32>(tile + 2048, c.lane, w);
        ring_publish();
        if (c.lane == 0) {
          store_tile(c, &p.tm_dx, tile, col);
          store_tile(c, &p.tm_normed, tile + 2048, col);
        }
        ring_commit(c);
      } else if (row_ok) {
        store_row32(p.dX + r * p.ld_dx + col, d, ncols);
        store_row32(p.normed + r * p.ld_normed + col, w, ncols);
      }
      // transpose-reduce over the warp's 32 rows: afterwards lane l holds the sum of column col + l in y[0]
#pragma unroll
      for (int o = 16; o >= 1; o >>= 1) {
        const bool upper = (c.lane & o) != 0;
#pragma unroll
        for (int i = 0; i < o; ++i) {
          const float keep = upper ? y[i + o] : y[i];
          const float send = upper ? y[i] : y[i + o];
          y[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
      }
      if (slab * 32 < c.M && c.lane < ncols) p.part_dw[slab * c.N + col + c.lane] = y[0];
    });
  }
};

}  // namespace cb
