// Persistent, warp-specialised bf16 GEMM core for sm_100a.
//
//   D[M, N] = epilogue( A[M, K] * B[N, K]^T ),  fp32 accumulation in tensor memory.
//
// Roles inside one CTA of 192 threads:
//   warp 0      TMA producer   global -> 128-byte-swizzled shared-memory ring (one elected lane)
//   warp 1      MMA issuer     tcgen05.mma, accumulators in TMEM (one elected lane); owns TMEM alloc/dealloc
//   warps 2..5  epilogue       tcgen05.ld TMEM -> registers -> fused math -> global stores
//
// Two accumulator stages live in TMEM so the epilogue of tile i overlaps the
// mainloop of tile i+1.  With kCtaGroup == 2 two CTAs (a cluster of 2) share one
// 256 x kBN tile: each CTA loads its own 128 rows of A and its own half of B,
// the leader CTA issues tcgen05.mma.cta_group::2, and each CTA drains its own
// 128 accumulator rows.  No multicast loads are used anywhere.
//
// A and B may each be K-major (contraction index contiguous) or MN-major
// (row/column index contiguous); the transposed operands of the backward GEMMs
// are consumed in place, without a physical transpose.
#pragma once

#include "ptx.cuh"

namespace cb {

constexpr int kBlockM = 128;  // accumulator rows per CTA (= TMEM lanes)
constexpr int kBlockK = 64;   // bf16 elements per k-block = one 128-byte swizzle row
constexpr int kUmmaK = 16;    // contraction depth of one tcgen05.mma (bf16)
constexpr int kNumThreads = 192;
constexpr int kNumEpiWarps = 4;
constexpr int kSmemBudget = 227 * 1024;

struct GemmShape {
  int M, N, K;  // K = contraction length
  int tiles_m;  // number of (kBlockM * kCtaGroup)-row tiles
  int tiles_n;  // number of kBN-column tiles
  int group_m;  // raster: tiles of `group_m` consecutive row-tiles share their column sweep (L2 reuse)
  // Tail split (sk_split <= 1: off).  Tiles go to the clusters round-robin, so the last `sk_tail` tiles (fewer than
  // there are clusters) would keep only `sk_tail` clusters busy for a whole contraction.  With sk_split = s each of them is
  // cut into s equal ranges of k-blocks that run as separate items, accumulated in parts (see WorkItem).
  int sk_tail, sk_split;
  // Measurement aid (0 = off): while the mainloop of a tile runs, each epilogue warp issues this many bytes of
  // coalesced global loads from [probe_src, probe_src + probe_span) and of shared-memory stores per k-block, i.e. the
  // load/store-unit traffic an operand-transforming prologue would add, without changing any result.
  int probe_ld_bytes, probe_st_bytes;
  const void* probe_src;
  long long probe_span;
};

// Per-thread view of one accumulator tile handed to an epilogue.  `ring` and `slot` describe the warp's private
// staging ring in shared memory: output sub-tiles are written there and leave through TMA stores, so `slot` (and the
// bulk async-groups still in flight behind it) carries over from one tile to the next.
struct EpiCtx {
  int row;         // global row owned by this thread (may be >= M: loads still run, stores are clipped / predicated)
  int row0;        // global row of lane 0 of this warp (the y coordinate of the warp's TMA stores)
  int n0;          // first global column of the tile
  int tn;          // column-tile index
  int M, N;        // problem extents
  uint32_t taddr;  // TMEM address of (this warp's first lane, first column of the accumulator)
  int part_row0;   // -1: the accumulator is the whole contraction; else a partial sum, and this is the workspace row that
                   // lane 0's row goes to (tail split; only epilogues with kSplitTail are ever launched that way)
  int lane;
  uint32_t ring;   // shared-memory address of this warp's staging ring (kRingSlots slots of kRingSlotBytes)
  uint32_t slot;   // slot the next staged sub-tile goes to
  // Epilogues that read a second [M, N] operand fetch its sub-tiles by TMA into the warp's load slots:
  uint32_t ld_ring;   // shared-memory address of this warp's kLoadSlots load slots (kLoadSlotBytes each); 0 if none
  uint32_t ld_bar;    // shared-memory address of the warp's kLoadSlots mbarriers
  uint32_t ld_phase;  // bit s = parity the next wait on slot s expects
  volatile int* abort_word;
};

constexpr int kRingSlots = 2;
constexpr uint32_t kRingSlotBytes = 4096;  // 32 rows x 128 bytes: the widest sub-tile an epilogue stages at once
constexpr uint32_t kRingBytesPerWarp = kRingSlots * kRingSlotBytes;
constexpr int kLoadSlots = 2;
constexpr uint32_t kLoadSlotBytes = 4096;  // two 32 x 32 bf16 boxes
constexpr uint32_t kLoadRingBytesPerWarp = kLoadSlots * kLoadSlotBytes;
constexpr uint32_t kLoadBarOffset = 512;  // inside the control block: kNumEpiWarps x kLoadSlots mbarriers
constexpr uint32_t kRawBarOffset = 256;   // inside the control block: one mbarrier per stage for a prologue's raw tiles

// kEpiLoadBytes: bytes of operand load slots per epilogue warp (0 for epilogues without a second operand).
// kStageExtraBytes: bytes a prologue policy adds to every pipeline stage (the raw tile it transforms with).
template <int kCtaGroup, int kBN, uint32_t kEpiLoadBytes = 0, uint32_t kStageExtraBytes = 0>
struct GemmCfg {
  static constexpr int kBNcta = kBN / kCtaGroup;  // B rows loaded by one CTA
  static constexpr uint32_t kABytes = kBlockM * kBlockK * 2;
  static constexpr uint32_t kBBytes = kBNcta * kBlockK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes + kStageExtraBytes;
  static constexpr uint32_t kCtrlBytes = 1024;  // barriers, TMEM pointer, abort word
  static constexpr uint32_t kEpiScratch = kNumEpiWarps * (kRingBytesPerWarp + kEpiLoadBytes);  // staging rings (+ load slots) of the epilogue warps
  static constexpr int kStagesFit = (kSmemBudget - 1024 - kCtrlBytes - kEpiScratch) / kStageBytes;
  static constexpr int kStages = kStagesFit > 8 ? 8 : kStagesFit;
  static constexpr uint32_t kSmemBytes = 1024 + kStages * kStageBytes + kCtrlBytes + kEpiScratch;
  static constexpr uint32_t kTmemCols = 2 * kBN;  // two accumulator stages
  static_assert(kBN == 64 || kBN == 128 || kBN == 256, "tile width must be 64, 128 or 256");
  static_assert((kStages * kStageBytes + kCtrlBytes) % 1024 == 0, "the staging rings must start on a swizzle-atom boundary");
  static_assert(kStages >= 2, "need at least two pipeline stages");
};

__device__ __forceinline__ void tile_coords(const GemmShape& s, int tile, int& tm, int& tn) {
  const int per_group = s.group_m * s.tiles_n;
  const int g = tile / per_group;
  const int first_m = g * s.group_m;
  const int gsz = min(s.group_m, s.tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

// One pass of a role's loop: k-blocks [kb0, kb1) of `tile`.  slab < 0: the whole contraction, the epilogue writes the
// output.  Otherwise the item is one part of a tail tile, and its accumulator goes, as raw fp32, to slab `slab` of the
// workspace; a follow-up kernel adds a tile's parts in a fixed order (so results do not depend on timing), applies
// alpha and writes the output.
struct WorkItem {
  int tile, kb0, kb1, slab;
};

// Every role of a CTA walks the same item sequence, computed from the launch geometry alone: items
// cluster_id, cluster_id + num_clusters, ... of [whole tiles 0 .. F-1 | parts of the tail tiles], F = num_tiles - sk_tail.
// Tail items are ordered part-major (part 0 of every tail tile, then part 1, ...): the clusters that run concurrently
// then work on neighbouring tiles at the same depth of the contraction, which is what lets them share operand tiles
// through L2.
struct WorkSchedule {
  int num_kb, num_clusters, full, tail, split, total, next_item;

  __device__ WorkSchedule(const GemmShape& s, int cluster, int clusters, int tiles, int kbs)
      : num_kb(kbs), num_clusters(clusters), next_item(cluster) {
    split = s.sk_split > 1 ? s.sk_split : 1;
    tail = split > 1 ? s.sk_tail : 0;
    full = tiles - tail;
    total = full + tail * split;
  }
  __device__ bool next(WorkItem& w) {
    if (next_item >= total) return false;
    const int i = next_item;
    next_item += num_clusters;
    if (i < full) {
      w.tile = i;
      w.kb0 = 0;
      w.kb1 = num_kb;
      w.slab = -1;
    } else {
      const int j = i - full, part = j / tail;
      w.tile = full + (j - part * tail);
      w.kb0 = static_cast<int>(static_cast<long long>(part) * num_kb / split);
      w.kb1 = static_cast<int>(static_cast<long long>(part + 1) * num_kb / split);
      w.slab = j;
    }
    return true;
  }
};

// What-if traffic for the prologue-fusion study (see GemmShape): runs in an epilogue warp while it would otherwise
// spin on the accumulator barrier, stops as soon as the accumulator is complete.
__device__ __forceinline__ void probe_lsu_traffic(const GemmShape& shape, const EpiCtx& c, uint32_t bar, uint32_t parity, int num_kb,
                                                  int warp_slot) {
  if (c.lane == 0) tma_store_wait_read<0>();  // the staging ring doubles as the store target
  __syncwarp();
  const uint4* src = static_cast<const uint4*>(shape.probe_src);
  const long long n16 = shape.probe_span / 16;
  const int ld_iters = shape.probe_ld_bytes / 512, st_iters = shape.probe_st_bytes / 512;
  long long pos = (static_cast<long long>(blockIdx.x) * kNumEpiWarps + warp_slot) * 65536 % (n16 > 64 ? n16 - 64 : 1);
  uint4 acc = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll 1
  for (int kb = 0; kb < num_kb; ++kb) {
    if (mbar_test_wait(bar, parity)) break;
#pragma unroll 4
    for (int i = 0; i < ld_iters; ++i) {
      const uint4 v = __ldcg(src + pos + c.lane);
      acc.x ^= v.x; acc.y ^= v.y; acc.z ^= v.z; acc.w ^= v.w;
      pos += 32;
      if (pos + 32 >= n16) pos = 0;
    }
#pragma unroll 4
    for (int i = 0; i < st_iters; ++i) st_shared_v4(c.ring + ((i * 512 + c.lane * 16) & (kRingBytesPerWarp - 1)), acc.x, acc.y, acc.z, acc.w);
  }
  __syncwarp();
}

// ------------------------------------------------------------------ A-operand prologues
// A prologue policy replaces the TMA load of the A operand by "transform warps" (warps 6..9) that build each 128 x 64
// K-major A tile themselves and write it into the pipeline stage in the swizzle the MMA expects.
struct ProNone {
  static constexpr int kWarps = 0;
  static constexpr uint32_t kStageExtraBytes = 0;
  struct Params {};
};

// G = dout * out * (1 - out), the gradient of a sigmoid through its stored output, formed on the fly as the A operand
// of the input-gradient GEMM dx = G @ W (coda/kernels/functional/sigmoid.py:33-38 does this as a separate aten pass).
// TMA loads the `out` tile straight into the stage's A slot (it has the operand's layout already) and the `dout`
// tile into an extra slot of the stage; the transform warps multiply in place.  Math in packed bf16 (three roundings
// instead of one) to stay within the issue budget of four warps per k-block.  The CTAs of column tile 0 also store
// G, for the weight-gradient GEMM that follows.
struct ProDSigmoid {
  static constexpr int kWarps = 4;
  static constexpr uint32_t kStageExtraBytes = kBlockM * kBlockK * 2;  // the dout tile
  struct Params {
    alignas(64) CUtensorMap tm_dout;  // dout as [M, Kc], box 64 x 128, 128-byte swizzle (the A operand's geometry)
    __nv_bfloat16* G;                 // [M, Kc] written once
    long long ld_g;
  };
  // 8 consecutive elements (16 bytes) of out and dout -> 8 elements of G
  __device__ static uint4 transform(const uint4& o, const uint4& d) {
    const __nv_bfloat162 one = __float2bfloat162_rn(1.0f);
    const uint32_t ow[4] = {o.x, o.y, o.z, o.w}, dw[4] = {d.x, d.y, d.z, d.w};
    uint32_t r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __nv_bfloat162 ov = *reinterpret_cast<const __nv_bfloat162*>(&ow[j]);
      const __nv_bfloat162 dv = *reinterpret_cast<const __nv_bfloat162*>(&dw[j]);
      const __nv_bfloat162 g = __hmul2(__hmul2(dv, ov), __hsub2(one, ov));
      r[j] = *reinterpret_cast<const uint32_t*>(&g);
    }
    return make_uint4(r[0], r[1], r[2], r[3]);
  }
};

template <int kCtaGroup, int kBN, bool kAMn, bool kBMn, class Epi, class Pro = ProNone>
__global__ void __launch_bounds__(kNumThreads + Pro::kWarps * 32, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmShape shape,
            const __grid_constant__ typename Epi::Params ep, int* __restrict__ status,
            const __grid_constant__ typename Pro::Params pp) {
  using Cfg = GemmCfg<kCtaGroup, kBN, Epi::kLoadRingBytes, Pro::kStageExtraBytes>;
  constexpr bool kProlog = Pro::kWarps > 0;
  static_assert(!kProlog || !kAMn, "transform warps build a K-major A tile");
  constexpr int kStages = Cfg::kStages;
  constexpr int kBNcta = Cfg::kBNcta;
  constexpr uint32_t kABytes = Cfg::kABytes;
  constexpr uint32_t kStageBytes = Cfg::kStageBytes;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t smem_base = (raw_addr + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  uint8_t* smem_gen = smem_raw + (smem_base - raw_addr);

  const uint32_t ctrl = smem_base + kStages * kStageBytes;
  const uint32_t bar_full = ctrl;                        // [kStages]
  const uint32_t bar_empty = ctrl + 8 * kStages;         // [kStages]
  const uint32_t bar_acc_full = ctrl + 16 * kStages;     // [2]
  const uint32_t bar_acc_empty = bar_acc_full + 16;      // [2]
  const uint32_t tmem_slot = bar_acc_empty + 16;         // uint32
  volatile int* abort_word = reinterpret_cast<volatile int*>(smem_gen + kStages * kStageBytes + 16 * kStages + 40);
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + kStages * kStageBytes + 16 * kStages + 32);
  const uint32_t epi_rings = ctrl + Cfg::kCtrlBytes;  // 1024-byte aligned: kStageBytes and kCtrlBytes are multiples of 1024

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = (kCtaGroup == 2) ? cluster_ctarank() : 0u;
  const bool leader = (rank == 0);
  // shared::cluster address of the other CTA's abort word (valid until the cluster barrier of the teardown)
  const uint32_t peer_abort = (kCtaGroup == 2) ? mapa(ctrl + 16 * kStages + 40, rank ^ 1u) : 0u;
  const int cluster_id = blockIdx.x / kCtaGroup;
  const int num_clusters = gridDim.x / kCtaGroup;
  const int num_tiles = shape.tiles_m * shape.tiles_n;
  const int num_kb = (shape.K + kBlockK - 1) / kBlockK;

  // ---------------------------------------------------------------- setup
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1 + Pro::kWarps * kCtaGroup);  // the producer's expect_tx arrive + one per transform warp of the pair
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_acc_full + 8 * a, 1);
      mbar_init(bar_acc_empty + 8 * a, kNumEpiWarps * kCtaGroup);
    }
    if constexpr (Epi::kLoadRingBytes != 0) {
      for (int i = 0; i < kNumEpiWarps * kLoadSlots; ++i) mbar_init(ctrl + kLoadBarOffset + 8 * i, 1);
    }
    if constexpr (kProlog) {
      for (int i = 0; i < kStages; ++i) mbar_init(ctrl + kRawBarOffset + 8 * i, 1);  // this CTA's raw tiles have landed
    }
    *abort_word = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc<kCtaGroup>(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish<kCtaGroup>();
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (kCtaGroup == 2) {
    cluster_arrive();
    cluster_wait();
  }
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_gen;

  if (warp == 0) {
    // ============================================================ TMA producer
    if (lane == 0) {
      const uint32_t full_sig = (kCtaGroup == 2) ? mapa(bar_full, 0) : bar_full;  // the leader's barriers
      uint32_t s = 0, ph = 0;
      bool ok = true;
      WorkSchedule sched(shape, cluster_id, num_clusters, num_tiles, num_kb);
      WorkItem w;
      while (ok && sched.next(w)) {
        int tm, tn;
        tile_coords(shape, w.tile, tm, tn);
        const int a_row0 = tm * (kBlockM * kCtaGroup) + static_cast<int>(rank) * kBlockM;
        const int b_row0 = tn * kBN + static_cast<int>(rank) * kBNcta;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_word, kErrTimeoutEmpty)) {
            ok = false;
            break;
          }
          if (leader) mbar_arrive_expect_tx(bar_full + 8 * s, (kProlog ? Cfg::kBBytes : kStageBytes) * kCtaGroup);
          const uint32_t a_dst = smem_base + s * kStageBytes;
          const uint32_t b_dst = a_dst + kABytes;
          const uint32_t sig = full_sig + 8 * s;
          const int k0 = kb * kBlockK;
          if constexpr (kProlog) {
            // raw tiles for the transform warps: `out` into the A slot, `dout` into the stage's extra slot, both of this
            // CTA's own rows, signalled on this CTA's own barrier (plain loads, not the pair form)
            const uint32_t raw_bar = ctrl + kRawBarOffset + 8 * s;
            mbar_arrive_expect_tx(raw_bar, 2 * kABytes);
            tma_load_2d(a_dst, &tmap_a, raw_bar, k0, a_row0);
            tma_load_2d(a_dst + kABytes + Cfg::kBBytes, &pp.tm_dout, raw_bar, k0, a_row0);
          } else if constexpr (!kAMn) {
            if constexpr (kCtaGroup == 2) tma_load_2d_pair(a_dst, &tmap_a, sig, k0, a_row0);
            else tma_load_2d(a_dst, &tmap_a, sig, k0, a_row0);
          } else {
#pragma unroll
            for (int j = 0; j < kBlockM / 64; ++j) {
              if constexpr (kCtaGroup == 2) tma_load_2d_pair(a_dst + j * (kBlockK * 128), &tmap_a, sig, a_row0 + 64 * j, k0);
              else tma_load_2d(a_dst + j * (kBlockK * 128), &tmap_a, sig, a_row0 + 64 * j, k0);
            }
          }
          if constexpr (!kBMn) {
            if constexpr (kCtaGroup == 2) tma_load_2d_pair(b_dst, &tmap_b, sig, k0, b_row0);
            else tma_load_2d(b_dst, &tmap_b, sig, k0, b_row0);
          } else {
#pragma unroll
            for (int j = 0; j < kBNcta / 64; ++j) {
              if constexpr (kCtaGroup == 2) tma_load_2d_pair(b_dst + j * (kBlockK * 128), &tmap_b, sig, b_row0 + 64 * j, k0);
              else tma_load_2d(b_dst + j * (kBlockK * 128), &tmap_b, sig, b_row0 + 64 * j, k0);
            }
          }
          if (++s == kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
      // Tail: do not leave while commit-arrives for the last stages may still be
      // on their way to this CTA's barriers.
      for (int i = 0; i < kStages && ok; ++i) {
        ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_word, kErrTimeoutEmpty);
        if (++s == kStages) {
          s = 0;
          ph ^= 1u;
        }
      }
      if (!ok) abort_notify_and_drain(peer_abort, *abort_word);
    }
    __syncwarp();
  } else if (warp == 1) {
    // ============================================================ MMA issuer
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kBlockM * kCtaGroup, kBN, kAMn, kBMn);
      constexpr uint32_t lbo_mn = kBlockK * 128, sbo_mn = 1024u;
      // K-major: 8-row groups 1024 B apart, one MMA step = 32 B along the swizzled row.
      // MN-major: 64-element column blocks kBlockK*128 B apart, 8-k groups 1024 B apart, one MMA step = 2 groups.
      const uint32_t a_lbo = kAMn ? lbo_mn : 16u, a_sbo = kAMn ? sbo_mn : 1024u, a_step = kAMn ? 2048u : 32u;
      const uint32_t b_lbo = kBMn ? lbo_mn : 16u, b_sbo = kBMn ? sbo_mn : 1024u, b_step = kBMn ? 2048u : 32u;
      uint32_t s = 0, ph = 0, it = 0;
      bool ok = true;
      WorkSchedule sched(shape, cluster_id, num_clusters, num_tiles, num_kb);
      WorkItem w;
      for (; ok && sched.next(w); ++it) {
        const uint32_t acc = it & 1u, aph = (it >> 1) & 1u;
        if (!mbar_wait(bar_acc_empty + 8 * acc, aph ^ 1u, abort_word, kErrTimeoutAccEmpty)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(bar_full + 8 * s, ph, abort_word, kErrTimeoutFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_base + s * kStageBytes;
          const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint64_t adesc = make_smem_desc(a_addr + k * a_step, a_lbo, a_sbo);
            const uint64_t bdesc = make_smem_desc(b_addr + k * b_step, b_lbo, b_sbo);
            umma_bf16<kCtaGroup>(d_tmem, adesc, bdesc, idesc, (kb != w.kb0 || k != 0) ? 1u : 0u);
          }
          umma_commit<kCtaGroup>(bar_empty + 8 * s);  // frees the stage (in both CTAs) once these MMAs retire
          if (++s == kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (ok) umma_commit<kCtaGroup>(bar_acc_full + 8 * acc);
      }
      // Tail: wait until both accumulator stages have been drained, so that no
      // remote arrive can target this CTA's barriers after it has left.
      for (int i = 0; i < 2 && ok; ++i, ++it) {
        const uint32_t acc = it & 1u, aph = (it >> 1) & 1u;
        ok = mbar_wait(bar_acc_empty + 8 * acc, aph ^ 1u, abort_word, kErrTimeoutAccEmpty);
      }
      if (!ok) abort_notify_and_drain(peer_abort, *abort_word);
    }
    __syncwarp();
  } else if (kProlog && warp >= 2 + kNumEpiWarps) {
    // ============================================================ transform warps (A-operand prologue)
    if constexpr (kProlog) {
      const int t = warp - (2 + kNumEpiWarps);  // rows 32 t .. 32 t + 31 of the CTA's A tile
      const int piece = lane & 7;               // 16-byte piece = 8 contraction columns
      const int rsub = lane >> 3;               // 4 rows per access
      const uint32_t full_sig = (kCtaGroup == 2) ? mapa(bar_full, 0) : bar_full;  // the leader's barriers
      const int Kc = shape.K;
      uint32_t s = 0, ph = 0;
      bool ok = true;
      WorkSchedule sched(shape, cluster_id, num_clusters, num_tiles, num_kb);
      WorkItem w;
      while (ok && sched.next(w)) {
        int tm, tn;
        tile_coords(shape, w.tile, tm, tn);
        const int a_row0 = tm * (kBlockM * kCtaGroup) + static_cast<int>(rank) * kBlockM;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(ctrl + kRawBarOffset + 8 * s, ph, abort_word, kErrTimeoutFull)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + s * kStageBytes;
          const uint32_t x_dst = a_dst + kABytes + Cfg::kBBytes;
          const int k0 = kb * kBlockK;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r_in = 32 * t + 4 * i + rsub;
            const uint32_t off = r_in * 128 + ((piece ^ (r_in & 7)) << 4);  // the operand's 128-byte swizzle
            const uint4 g = Pro::transform(ld_shared_v4(a_dst + off), ld_shared_v4(x_dst + off));
            st_shared_v4(a_dst + off, g.x, g.y, g.z, g.w);  // in place: the A slot now holds G
            const int row = a_row0 + r_in, col = k0 + piece * 8;
            if (tn == 0 && row < shape.M && col < Kc) *reinterpret_cast<uint4*>(pp.G + static_cast<long long>(row) * pp.ld_g + col) = g;
          }
          fence_proxy_async_smem();  // the tensor core reads the tile through the async proxy
          __syncwarp();
          if (lane == 0) {
            if constexpr (kCtaGroup == 2) mbar_arrive_cluster(full_sig + 8 * s);
            else mbar_arrive(bar_full + 8 * s);
          }
          if (++s == kStages) {
            s = 0;
            ph ^= 1u;
          }
        }
      }
      if (!ok && lane == 0) abort_notify_and_drain(peer_abort, *abort_word);
      __syncwarp();
    }
  } else {
    // ============================================================ epilogue
    const int q = warp & 3;  // TMEM lane quadrant this warp may read
    const uint32_t acc_empty_sig = (kCtaGroup == 2) ? mapa(bar_acc_empty, 0) : bar_acc_empty;
    EpiCtx c;
    c.M = shape.M;
    c.N = shape.N;
    c.lane = lane;
    c.ring = epi_rings + static_cast<uint32_t>(warp - 2) * kRingBytesPerWarp;
    c.slot = 0;
    c.ld_ring = Epi::kLoadRingBytes != 0 ? epi_rings + kNumEpiWarps * kRingBytesPerWarp + static_cast<uint32_t>(warp - 2) * Epi::kLoadRingBytes : 0u;
    c.ld_bar = ctrl + kLoadBarOffset + static_cast<uint32_t>(warp - 2) * (8 * kLoadSlots);
    c.ld_phase = 0;
    c.abort_word = abort_word;
    uint32_t it = 0;
    WorkSchedule sched(shape, cluster_id, num_clusters, num_tiles, num_kb);
    WorkItem w;
    for (; sched.next(w); ++it) {
      int tm, tn;
      tile_coords(shape, w.tile, tm, tn);
      const uint32_t acc = it & 1u, aph = (it >> 1) & 1u;
      if (shape.probe_ld_bytes + shape.probe_st_bytes != 0) probe_lsu_traffic(shape, c, bar_acc_full + 8 * acc, aph, w.kb1 - w.kb0, warp - 2);
      bool ok = mbar_wait(bar_acc_full + 8 * acc, aph, abort_word, kErrTimeoutAccFull);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) abort_notify_and_drain(peer_abort, *abort_word);
        __syncwarp();
        break;
      }
      tc_fence_after();
      c.row0 = tm * (kBlockM * kCtaGroup) + static_cast<int>(rank) * kBlockM + q * 32;
      c.row = c.row0 + lane;
      c.n0 = tn * kBN;
      c.tn = tn;
      c.taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * kBN;
      c.part_row0 = w.slab < 0 ? -1 : w.slab * (kBlockM * kCtaGroup) + static_cast<int>(rank) * kBlockM + q * 32;
      Epi::template run<kBN>(ep, c);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kCtaGroup == 2) mbar_arrive_cluster(acc_empty_sig + 8 * acc);
        else mbar_arrive(bar_acc_empty + 8 * acc);
      }
    }
    // Staged sub-tiles still on their way out: the shared memory they are read from and the global writes themselves
    // must be finished before the CTA exits.
    if (lane == 0) tma_store_wait_all();
    __syncwarp();
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if constexpr (kCtaGroup == 2) {
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<kCtaGroup>(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0) {
    report_status(status, *abort_word);
  }
}

}  // namespace cb
