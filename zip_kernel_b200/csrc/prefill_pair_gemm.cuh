// Kernel 2b: the many-token tensor-core kernel on CTA PAIRS (tcgen05 cta_group::2).
//
// Same arithmetic, roles and pipeline as prefill_gemm.cuh (read its header first); what changes is the
// tile.  Two CTAs of a thread-block cluster own two adjacent block-rows (2 x 128 weight rows = MMA
// M = 256) and SHARE a tile of 128 tokens (MMA N): each CTA loads its own 128 weight rows and only ITS
// HALF of the tokens (64 x 128 bytes per K-step); the pair's tensor cores read the other half from the
// peer's shared memory.  Per 128 x 128 x 128 multiply-accumulates a CTA then pulls 16 KB (8 + 8) over
// the L2 -> SM fabric instead of 24 KB (8 + 16): the unpaired kernel runs at the fabric's limit
// (~27 bytes per clock and SM), so this is where its time goes.  One thread of the pair's leader CTA
// (cluster rank 0) issues every MMA for both CTAs; accumulators, widened weights and the zero-point
// accumulator live at the same tensor-memory addresses in both CTAs, each CTA folds and stores its own
// 128 rows x 128 tokens.  No load in this file is a multicast load: every CTA fetches its own bytes.
//
// Synchronisation across the pair.  The leader's MMA thread waits on ONE "ready" barrier per step in the
// LEADER's shared memory; everything either CTA contributes to the step arrives there - the leader's
// own activation copy (transaction bytes), its unpack and fold warps, and from the peer: a relay thread
// (the peer's otherwise idle MMA warp waits for the peer's copies on a local barrier and forwards one
// arrival), the peer's unpack warps and fold warps (remote mbarrier arrivals, release at cluster scope).
// Completion of a step's MMAs is committed to the "done" barriers of BOTH CTAs.  Residual blocks: the
// pair walks the union of the block columns of its two block-rows; a CTA without a block in a column
// loads its peer's block instead (uniform control flow, finite data) and skips the fold of that step.
// Every wait is bounded; both CTAs meet at a cluster barrier before tensor memory is released.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "prefill_gemm.cuh"

namespace w4a4 {
namespace pp {

using pre::A_BUFS;
using pre::A_COLS;
using pre::ROWS;
using pre::SZ_CHUNK;
using pre::TMEM_COLS;
using pre::TN;
using pre::ZT_BYTES;
constexpr int TH = TN / 2;                      // tokens a CTA loads per step (its half of the pair's tile)
constexpr int XH_BYTES = TH * BCOL;             // 8192
constexpr int MAX_UNION = 512;                  // residual columns of a row pair that the step list can hold

constexpr int WARP_TMA = 0, WARP_MMA = 1, WARP_UNPACK0 = 2, N_UNPACK_WARPS = 4, WARP_FOLD0 = 6, N_FOLD_WARPS = 8;
constexpr int THREADS = (WARP_FOLD0 + N_FOLD_WARPS) * 32;
constexpr int FOLD_THREADS = N_FOLD_WARPS * 32;
constexpr int COLS_PER_FOLD = TN / (N_FOLD_WARPS / 4);

enum : int {
  SITE_PP_WEMPTY = 48, SITE_PP_WFULL, SITE_PP_AEMPTY, SITE_PP_ZFULL, SITE_PP_XEMPTY, SITE_PP_READY,
  SITE_PP_ZDONE, SITE_PP_ACCFULL, SITE_PP_DUMP, SITE_PP_LANDED
};

template <bool PREP>
struct TmemLayout {
  static constexpr int ACC_BUFS = PREP ? 3 : 2;
  static constexpr int A_COL0 = ACC_BUFS * TN;
  static constexpr int Z_COL0 = A_COL0 + (PREP ? 0 : A_BUFS * A_COLS);
  static_assert(Z_COL0 + TN <= TMEM_COLS, "tensor memory capacity");
};

template <bool PREP>
struct SmemLayout {
  static constexpr int W_STAGES = PREP ? 6 : 8;
  static constexpr int X_STAGES = PREP ? 6 : 8;
  static constexpr int WP_BYTES = PREP ? ROWS * BCOL : ROWS * GROUP_BYTES;
  static_assert(W_STAGES == X_STAGES, "the pair kernel walks one ring index for both copies of a step");
  static constexpr size_t wp = 0;
  static constexpr size_t x = wp + (size_t)W_STAGES * WP_BYTES;
  static constexpr size_t sz = x + (size_t)X_STAGES * XH_BYTES;
  static constexpr size_t zb = sz + (size_t)SZ_CHUNK * ROWS * 4;               // tf32 [2][TH tokens][32]: this CTA's tokens' group sums
  static constexpr size_t za = zb + (size_t)2 * (ZT_BYTES / 2);                // tf32 [128 rows][32]
  static constexpr size_t raw = za + (size_t)ZT_BYTES;
  static constexpr size_t sxs = raw + (size_t)2 * ROWS * 32;
  static constexpr size_t ulist = sxs + (size_t)TN * 4;                         // int [MAX_UNION][2]: (column, my block or ~peer's block)
  static constexpr size_t bars = ulist + (size_t)MAX_UNION * 8;
  static constexpr size_t total = bars + 512;
};
inline size_t smem_bytes(bool prep) { return 1024 + (prep ? SmemLayout<true>::total : SmemLayout<false>::total); }
inline bool supported(int T, int K, int N) { return T >= 1 && K >= 128 && N >= 1 && K / 128 <= MAX_UNION / 2; }

// ---------------------------------------------------------------- cluster / pair helpers
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `p` (a pointer into this CTA's shared memory) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(smem_u32(p)), "r"(rank));
  return a;
}
// Arrival on a barrier of any CTA of the cluster.  Default semantics (release at CTA scope), like the
// barrier itself: what crosses the pair here is tensor-memory state, ordered by the tcgen05 fences around
// the arrival, and shared-memory operand tiles that were already made visible to the asynchronous proxy by
// fence.proxy.async - a cluster-scope release on every arrival costs a fence per warp and step (measured:
// it halved the kernel's throughput).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, int site, bool relaxed) {
  return relaxed ? mbar_wait_relaxed(bar, parity, site) : mbar_wait(bar, parity, site);
}

// ---------------------------------------------------------------- tcgen05, cta_group::2 forms
__device__ __forceinline__ void tmem_alloc2(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// M = 256 over the pair (128 rows per CTA), N = TN tokens (half from each CTA's shared memory)
constexpr uint32_t IDESC2_I8 = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)((2 * ROWS) >> 4) << 24);
constexpr uint32_t IDESC2_F8 = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)((2 * ROWS) >> 4) << 24);
constexpr uint32_t IDESC2_TF32 = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)((2 * ROWS) >> 4) << 24);
__device__ __forceinline__ void umma2_i8_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(IDESC2_I8), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma2_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(IDESC2_F8), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma2_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(IDESC2_TF32), "r"(accumulate) : "memory");
}
// one arrival on the barrier at this shared-memory offset in BOTH CTAs of the pair once every MMA issued
// so far by this thread has completed (a commit, not a load: no data is multicast)
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}

template <bool DUMP, bool F8, bool PREP>
__global__ void __launch_bounds__(THREADS, 1)
prefill_pair_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_wh,
                         const pre::Params p) {
  static_assert(F8 == PREP, "packed weights take integer MMAs, prepared weights fp8 MMAs");
  using SmemLayout = pp::SmemLayout<PREP>;
  using namespace pre;      // tcgen05.ld / st wrappers, descriptors, fences
  constexpr int STAGES = SmemLayout::X_STAGES, WP_BYTES = SmemLayout::WP_BYTES;
  constexpr int ACC_BUFS = pp::TmemLayout<PREP>::ACC_BUFS, A_COL0 = pp::TmemLayout<PREP>::A_COL0, Z_COL0 = pp::TmemLayout<PREP>::Z_COL0;
  static_assert(ACC_BUFS < STAGES, "the fold warps' arrival for step n + ACC_BUFS must fall into that step's barrier phase");
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* wp_ring = sm + SmemLayout::wp;
  unsigned char* x_ring = sm + SmemLayout::x;
  float* szs = reinterpret_cast<float*>(sm + SmemLayout::sz);
  unsigned char* zb_tiles = sm + SmemLayout::zb;
  unsigned char* za_tile = sm + SmemLayout::za;
  float* sxs = reinterpret_cast<float*>(sm + SmemLayout::sxs);
  int2* ulist = reinterpret_cast<int2*>(sm + SmemLayout::ulist);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + SmemLayout::bars);
  uint64_t* w_full = bars;                    // [STAGES] this CTA's packed weight tile has landed (unpack warps wait)
  uint64_t* w_empty = w_full + STAGES;        // [STAGES] ... and has been widened
  uint64_t* ready = w_empty + STAGES;         // [STAGES] LEADER's copy is used: everything step n's MMAs need, from both CTAs
  uint64_t* done = ready + STAGES;            // [STAGES] the MMAs of step n have completed (committed to both CTAs)
  uint64_t* landed = done + STAGES;           // [STAGES] PEER only: its copies of step n have landed (relayed to the leader)
  uint64_t* z_full = landed + STAGES;         // LEADER's copy is used
  uint64_t* z_done = z_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(z_done + 1);
  int* n_res_slot = reinterpret_cast<int*>(tmem_slot + 1);

  grid_launch_dependents();
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t rank = cluster_rank();         // 0 = leader of the pair
  const bool leader = rank == 0;
  // pairs are dispatched in bands of `band` token tiles, token tile first (see prefill_gemm.cuh)
  const int n_pairs = gridDim.x >> 1;
  const int lin = (blockIdx.x >> 1) + blockIdx.y * n_pairs;
  const int per_band = n_pairs * p.band;
  const int band_i = lin / per_band, band_rem = lin - band_i * per_band;
  const int band_h = min(p.band, (int)gridDim.y - band_i * p.band);
  const int pr = band_rem / band_h;             // pair of block-rows
  const int r = 2 * pr + (int)rank;             // this CTA's block-row (may lie beyond the last one: nothing is stored then)
  const int row0 = r * ROWS;
  const int tokp = (band_i * p.band + band_rem % band_h) * TN;    // first token of the pair's tile
  const int tokh = tokp + (int)rank * TH;                            // first token this CTA loads
  const int nbr = (p.N + ROWS - 1) / ROWS;

  if (tid == 0) {
    const uint32_t n_ready = PREP ? (2 + N_FOLD_WARPS) + (1 + N_FOLD_WARPS) : 2 * (1 + N_UNPACK_WARPS + N_FOLD_WARPS);
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&w_full[i], 1);
      mbar_init(&w_empty[i], N_UNPACK_WARPS);
      mbar_init(&ready[i], n_ready);
      mbar_init(&done[i], 1);
      mbar_init(&landed[i], PREP ? 2 : 1);
    }
    mbar_init(z_full, 2 * N_FOLD_WARPS);
    mbar_init(z_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_wh);
    // Residual K-steps of the pair: the union of the block columns of its two block-rows, ascending.  Entry =
    // (column, block to load): this CTA's own block when it has one in that column, else ~(the peer's block).
    int n = 0;
    if (p.sparse_on) {
      const int ra = 2 * pr, rb = 2 * pr + 1;
      int a = ra < nbr ? ld_plain(p.hp_row_offsets + ra) : 0, a_hi = ra < nbr ? ld_plain(p.hp_row_offsets + ra + 1) : 0;
      int b = rb < nbr ? ld_plain(p.hp_row_offsets + rb) : 0, b_hi = rb < nbr ? ld_plain(p.hp_row_offsets + rb + 1) : 0;
      while ((a < a_hi || b < b_hi) && n < MAX_UNION) {
        const int ca = a < a_hi ? ld_plain(p.hp_col_indices + a) : 0x7fffffff;
        const int cb = b < b_hi ? ld_plain(p.hp_col_indices + b) : 0x7fffffff;
        const int c = min(ca, cb);
        const int blk_a = ca == c ? a++ : -1, blk_b = cb == c ? b++ : -1;
        const int mine = leader ? blk_a : blk_b, other = leader ? blk_b : blk_a;
        ulist[n++] = make_int2(c, mine >= 0 ? mine : ~other);
      }
    }
    *n_res_slot = n;
  }
  if (warp == WARP_MMA) tmem_alloc2(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();         // both CTAs' barriers are initialised before either one arrives on the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int n_res = *n_res_slot;
  const int n_steps = p.nd + n_res;
  const int n_windows = (p.nd + SZ_CHUNK - 1) / SZ_CHUNK;
  // the leader's barriers, as addresses any CTA of the pair can arrive on
  const uint32_t ready_l = map_to_cta(ready, 0), z_full_l = map_to_cta(z_full, 0);

  if (warp == WARP_TMA) {
    // ------------------------------------------------------------ copy thread (one per CTA)
    if (lane == 0) {
      bool ok = true;
      const int n_pre = min(STAGES, n_steps);
      // The leader's copies report straight to the step's readiness barrier; the peer's to its local
      // `landed` barrier, which its relay thread forwards.  Packed tiles go to the unpack warps first.
      auto issue_w = [&](int n, int st) {
        uint64_t* bar = PREP ? (leader ? &ready[st] : &landed[st]) : &w_full[st];
        mbar_arrive_expect_tx(bar, WP_BYTES);
        if (n < p.nd) {
          tma_load_2d(wp_ring + st * WP_BYTES, &tm_w, n * (PREP ? BCOL : GROUP_BYTES), row0, bar);
        } else {
          const int e = ulist[n - p.nd].y;
          tma_load_2d(wp_ring + st * WP_BYTES, &tm_wh, 0, (e >= 0 ? e : ~e) * BROW, bar);
        }
      };
      for (int n = 0; n < n_pre; ++n) issue_w(n, n);       // weights do not depend on the preceding kernel
      grid_dependency_wait_for_async_reads();
      int st = 0;
      uint32_t wph = 1;
      for (int n = 0; n < n_steps && ok; ++n) {
        if (n >= n_pre) {
          ok = PREP ? mbar_wait_relaxed(&done[st], ((n - STAGES) / STAGES) & 1, SITE_PP_WEMPTY)
                    : mbar_wait_relaxed(&w_empty[st], wph, SITE_PP_WEMPTY);
          if (!ok) break;
          issue_w(n, st);
        }
        // the activation slot is free once the MMAs of step n - STAGES have completed
        if (n >= STAGES) ok = mbar_wait_relaxed(&done[st], ((n - STAGES) / STAGES) & 1, SITE_PP_XEMPTY);
        if (!ok) break;
        const int g = n < p.nd ? n : ulist[n - p.nd].x;
        uint64_t* xbar = leader ? &ready[st] : &landed[st];
        mbar_arrive_expect_tx(xbar, XH_BYTES);
        bulk_load_1d(x_ring + st * XH_BYTES, p.XE + ((size_t)g * p.t_pad + tokh) * BCOL, XH_BYTES, xbar);
        if (++st == STAGES) { st = 0; wph ^= 1; }
      }
    }
  } else if (warp == WARP_MMA) {
    if (lane == 0 && !leader) {
      // ---------------------------------------------------------- peer: relay "my copies have landed" to the leader
      bool ok = true;
      for (int n = 0; n < n_steps && ok; ++n) {
        const int st = n % STAGES;
        ok = mbar_wait_relaxed(&landed[st], (n / STAGES) & 1, SITE_PP_LANDED);
        if (ok) mbar_arrive_cluster(ready_l + st * 8);
      }
    } else if (lane == 0) {
      // ---------------------------------------------------------- leader: MMA issuer for the pair
      bool ok = true;
      int st = 0;
      uint32_t ph = 0;
      int z_next = 0;
      auto issue_zero_term = [&](int k) {
        if (!mbar_wait_cluster(z_full, k & 1, SITE_PP_ZFULL, true)) return false;
        tc_fence_after();
        const uint64_t za_desc = smem_desc_sw128(za_tile);
        const uint64_t zb_desc = smem_desc_sw128(zb_tiles + (k & 1) * (ZT_BYTES / 2));
#pragma unroll
        for (int j = 0; j < 4; ++j) umma2_tf32(tmem_base + Z_COL0, za_desc + j * 2, zb_desc + j * 2, (k > 0 || j > 0) ? 1u : 0u);
        umma2_commit_both(z_done);
        return true;
      };
      int buf = 0, ab = 0;
      const uint64_t bdesc0 = smem_desc_sw128(x_ring), adesc0 = smem_desc_sw128(wp_ring);
      const uint32_t d0 = tmem_base, a0 = tmem_base + A_COL0;
      const bool with_z = p.Y != nullptr && n_windows > 0;
      int z_due = ACC_BUFS;
      for (int n = 0; n < n_steps && ok; ++n) {
        if (with_z && n == z_due && z_next < n_windows) {
          ok = issue_zero_term(z_next++);
          z_due += SZ_CHUNK;
          if (!ok) break;
        }
        if (!mbar_wait_cluster(&ready[st], ph, SITE_PP_READY, PREP)) { ok = false; break; }
        tc_fence_after();
        const uint64_t bdesc = bdesc0 + (uint64_t)(st * (XH_BYTES >> 4));
        const uint32_t d = d0 + buf * TN, a = a0 + ab * A_COLS;
        if (PREP) {
          const uint64_t adesc = adesc0 + (uint64_t)(st * (WP_BYTES >> 4));
          umma2_f8(d, adesc, bdesc, 0);
          umma2_f8(d, adesc + 2, bdesc + 2, 1);
          umma2_f8(d, adesc + 4, bdesc + 4, 1);
          umma2_f8(d, adesc + 6, bdesc + 6, 1);
        } else {
          umma2_i8_ta(d, a, bdesc, 0);
          umma2_i8_ta(d, a + 8, bdesc + 2, 1);
          umma2_i8_ta(d, a + 16, bdesc + 4, 1);
          umma2_i8_ta(d, a + 24, bdesc + 6, 1);
        }
        umma2_commit_both(&done[st]);
        if (++st == STAGES) { st = 0; ph ^= 1; }
        if (++buf == ACC_BUFS) buf = 0;
        ab ^= 1;
      }
      while (ok && p.Y != nullptr && z_next < n_windows) ok = issue_zero_term(z_next++);
    }
  } else if (warp < WARP_FOLD0) {
    // ------------------------------------------------------------ unpack warps (packed weights only)
    const int urow = (warp & 3) * 32 + lane;
    const uint32_t wp_a = smem_u32(wp_ring);
    const uint32_t a_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + A_COL0;
    bool ok = true;
    int st = 0;
    uint32_t ph = 0;
    for (int n = 0; n < (PREP ? 0 : n_steps); ++n) {
      const int buf = n % A_BUFS;
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait_relaxed(&w_full[st], ph, SITE_PP_WFULL));
      // the A buffer was last read by the MMAs of step n - 2
      if (ok && n >= A_BUFS)
        ok = __all_sync(0xffffffffu, mbar_wait_relaxed(&done[(n - A_BUFS) % STAGES], ((n - A_BUFS) / STAGES) & 1, SITE_PP_AEMPTY));
      if (ok) {
        tc_fence_after();
        const uint32_t src = wp_a + st * WP_BYTES + urow * GROUP_BYTES;
        uint4 w[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) w[c] = lds_v4(src + ((c ^ ((urow >> 1) & 3)) << 4));
        uint32_t v[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t q[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            v[(c * 4 + e) * 2] = nib_lo_x16(q[e]);
            v[(c * 4 + e) * 2 + 1] = nib_hi_x16(q[e]);
          }
        }
        tmem_st32(a_lane + buf * A_COLS, v);
        tc_fence_before();
      }
      __syncwarp();
      if (ok && lane == 0) {
        mbar_arrive(&w_empty[st]);
        mbar_arrive_cluster(ready_l + st * 8);
      }
      if (++st == STAGES) { st = 0; ph ^= 1; }
    }
  } else {
    // ------------------------------------------------------------ fold warps: this CTA's 128 rows x the pair's 128 tokens
    const int ft = tid - WARP_FOLD0 * 32;        // 0..255
    const int quarter = warp & 3;
    const int chalf = (warp - WARP_FOLD0) >> 2;
    const int rl = quarter * 32 + lane;
    const int row = row0 + rl;
    const int c0 = chalf * COLS_PER_FOLD;
    const uint32_t szs_a = smem_u32(szs), zb_a = smem_u32(zb_tiles), za_a = smem_u32(za_tile);
    grid_dependency_wait();
    for (int i = ft; i < TN; i += FOLD_THREADS)
      sxs[i] = (tokp + i < p.T && p.scale_x) ? __half2float(ld_plain(p.scale_x + tokp + i)) : 0.f;
    asm volatile("bar.sync 1, %0;" ::"n"(FOLD_THREADS) : "memory");

    f32x2_t y2[COLS_PER_FOLD / 2];
#pragma unroll
    for (int i = 0; i < COLS_PER_FOLD / 2; ++i) y2[i] = 0ull;

    const int lrow = ft >> 1, lhalf = ft & 1;
    constexpr int SUMS_PER_THREAD = SZ_CHUNK * TH / FOLD_THREADS;     // group sums of THIS CTA's half of the tokens
    const uint32_t raw_a = smem_u32(sm + SmemLayout::raw) + ft * 32;
    auto issue_window = [&](int gwin, int sel) {
#pragma unroll
      for (int k = 0; k < SUMS_PER_THREAD; ++k) {
        const int i = ft + k * FOLD_THREADS;
        const int gl = i / TH, t = i - gl * TH;
        const int g = gwin + gl, tok = tokh + t;
        const uint32_t rowa = zb_a + sel * (ZT_BYTES / 2) + t * 128 + (gl & 3) * 4;
        const uint32_t d0 = rowa + ((((gl >> 2)) ^ (t & 7)) << 4), d1 = rowa + ((((gl >> 2) + 4) ^ (t & 7)) << 4);
        if (p.sumxf && g < p.ng && tok < p.T) {
          const float* src = p.sumxf + ((size_t)(tok >> 4) * p.ng + g) * 16 + (tok & 15);
          cp_async_4(d0, src);
          cp_async_4(d1, src);
        } else {
          sts_f1(d0, 0.f);
          sts_f1(d1, 0.f);
        }
      }
      {
        const int grow = row0 + lrow;
        const int g = gwin + lhalf * 8;
        const bool live = p.scale_u4 != nullptr && grow < p.N && g < p.ng;
        const __half* srow = p.scale_u4 + (size_t)grow * p.ng;
        const __half* zrow = p.zero_u4 ? p.zero_u4 + (size_t)grow * p.ng : nullptr;
        if (live && p.sz_vec) {
          cp_async_16(raw_a, srow + g);
          if (zrow) cp_async_16(raw_a + 16, zrow + g);
          else sts_v4(raw_a + 16, make_uint4(0, 0, 0, 0));
        } else {
          __align__(16) __half hs[8], hz[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            hs[i] = (live && g + i < p.ng) ? srow[g + i] : __float2half(0.f);
            hz[i] = (live && g + i < p.ng && zrow) ? zrow[g + i] : __float2half(0.f);
          }
          sts_v4(raw_a, *reinterpret_cast<uint4*>(&hs[0]));
          sts_v4(raw_a + 16, *reinterpret_cast<uint4*>(&hz[0]));
        }
      }
      cp_async_commit();
    };
    auto park_window = [&]() {
      const uint4 ps = lds_v4(raw_a), pz = lds_v4(raw_a + 16);
      const __half2* hs = reinterpret_cast<const __half2*>(&ps);
      const __half2* hz = reinterpret_cast<const __half2*>(&pz);
      float chi[8], clo[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 s2 = __half22float2(hs[i]), z2 = __half22float2(hz[i]);
        sts_f1(szs_a + ((lhalf * 8 + 2 * i) * ROWS + lrow) * 4, s2.x * (F8 ? 1.f : 0.0625f));
        sts_f1(szs_a + ((lhalf * 8 + 2 * i + 1) * ROWS + lrow) * 4, s2.y * (F8 ? 1.f : 0.0625f));
        const float c0_ = s2.x * z2.x, c1_ = s2.y * z2.y;
        chi[2 * i] = __uint_as_float(__float_as_uint(c0_) & 0xFFFFE000u);
        chi[2 * i + 1] = __uint_as_float(__float_as_uint(c1_) & 0xFFFFE000u);
        clo[2 * i] = c0_ - chi[2 * i];
        clo[2 * i + 1] = c1_ - chi[2 * i + 1];
      }
      const uint32_t rowa = za_a + lrow * 128;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        sts_v4(rowa + (((lhalf * 2 + q) ^ (lrow & 7)) << 4),
               make_uint4(__float_as_uint(chi[4 * q]), __float_as_uint(chi[4 * q + 1]), __float_as_uint(chi[4 * q + 2]), __float_as_uint(chi[4 * q + 3])));
        sts_v4(rowa + (((4 + lhalf * 2 + q) ^ (lrow & 7)) << 4),
               make_uint4(__float_as_uint(clo[4 * q]), __float_as_uint(clo[4 * q + 1]), __float_as_uint(clo[4 * q + 2]), __float_as_uint(clo[4 * q + 3])));
      }
    };

    bool ok = true;
    if (p.nd > 0) issue_window(0, 0);
    // the accumulator buffers start out free: this warp's share of the first steps' readiness
    if (lane == 0)
      for (int i = 0; i < ACC_BUFS && i < n_steps; ++i) mbar_arrive_cluster(ready_l + (i % STAGES) * 8);
    for (int n = 0; n < n_steps; ++n) {
      const bool is_dense = n < p.nd;
      if (is_dense && (n % SZ_CHUNK) == 0) {
        const int k = n / SZ_CHUNK;
        cp_async_wait_all();
        if (ok && k > 0 && p.Y != nullptr) ok = __all_sync(0xffffffffu, mbar_wait(z_done, (k - 1) & 1, SITE_PP_ZDONE));
        asm volatile("bar.sync 1, %0;" ::"n"(FOLD_THREADS) : "memory");
        park_window();
        fence_proxy_async_smem();
        if (n + SZ_CHUNK < p.nd) issue_window(n + SZ_CHUNK, (k + 1) & 1);
        asm volatile("bar.sync 1, %0;" ::"n"(FOLD_THREADS) : "memory");
        if (lane == 0) mbar_arrive_cluster(z_full_l);
      }
      float f = 0.f;
      int blk = -1;
      bool active = true;
      if (is_dense) {
        f = lds_f1(szs_a + ((n % SZ_CHUNK) * ROWS + rl) * 4);
      } else {
        const int2 e = ulist[n - p.nd];
        blk = e.y;
        active = blk >= 0;          // without a block in this column the step's accumulator is not this CTA's business
        if (active && p.scale_u4 && row < p.N)
          f = __half2float(ld_plain(p.scale_u4 + (size_t)row * p.ng + e.x)) * (F8 ? 1.f : 0.0625f) * p.sparse_weight;
      }
      const int buf = n % ACC_BUFS;
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&done[n % STAGES], (n / STAGES) & 1, SITE_PP_ACCFULL));
      if (!ok) continue;
      tc_fence_after();
      if (active) {
        const f32x2_t f2 = pack_f32x2(f, f);
#pragma unroll
        for (int cc = 0; cc < COLS_PER_FOLD; cc += 32) {
          uint32_t a[32];
          tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * TN + c0 + cc, a);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            f32x2_t v;
            if (F8) asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(a[i]), "r"(a[i + 1]));
            else v = cvt_s32x2_f32x2(a[i], a[i + 1]);
            y2[(cc + i) >> 1] = fma_f32x2(v, f2, y2[(cc + i) >> 1]);
          }
          if (DUMP) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int tok = tokp + c0 + cc + i;
              if (tok >= p.T) continue;
              if (is_dense) {
                const size_t idx = ((size_t)n * p.N + row) * p.T + tok;
                if (p.acc_dump && row < p.N) {
                  if (idx < (size_t)p.ng * p.N * p.T) p.acc_dump[idx] = F8 ? (int)__uint_as_float(a[i]) : ((int)a[i]) >> 4;
                  else record_error(SITE_PP_DUMP, 1);
                }
              } else if (p.acc_hi_dump) {
                const size_t idx = ((size_t)blk * BROW + rl) * p.T + tok;
                if (blk < p.nnz && idx < (size_t)p.nnz * BROW * p.T) p.acc_hi_dump[idx] = F8 ? (int)__uint_as_float(a[i]) : ((int)a[i]) >> 4;
                else record_error(SITE_PP_DUMP, 2);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0 && n + ACC_BUFS < n_steps) mbar_arrive_cluster(ready_l + ((n + ACC_BUFS) % STAGES) * 8);
    }

    // y -= Z, the tensor core's sum over all groups of (scale * zero) * sumX
    if (p.Y != nullptr && n_windows > 0) {
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(z_done, (n_windows - 1) & 1, SITE_PP_ZDONE));
      if (ok) {
        tc_fence_after();
        const f32x2_t minus1 = pack_f32x2(-1.f, -1.f);
#pragma unroll
        for (int cc = 0; cc < COLS_PER_FOLD; cc += 32) {
          uint32_t z[32];
          tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + Z_COL0 + c0 + cc, z);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            f32x2_t zz;
            asm("mov.b64 %0, {%1, %2};" : "=l"(zz) : "r"(z[i]), "r"(z[i + 1]));
            y2[(cc + i) >> 1] = fma_f32x2(zz, minus1, y2[(cc + i) >> 1]);
          }
        }
      }
    }

    // epilogue: y * scale_x -> fp16
    if (ok && p.Y != nullptr && row < p.N) {
      const bool vec = (p.y_stride_t == 1) && ((p.y_stride_n & 7) == 0) && ((tokp + c0) % 8 == 0) &&
                       ((reinterpret_cast<uintptr_t>(p.Y) & 15) == 0) && (tokp + c0 + COLS_PER_FOLD <= p.T);
      if (vec) {
        __half* dst = p.Y + (size_t)row * p.y_stride_n + tokp + c0;
#pragma unroll
        for (int i = 0; i < COLS_PER_FOLD; i += 8) {
          __align__(16) __half2 h[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 v = unpack_f32x2(y2[(i >> 1) + k]);
            h[k] = __floats2half2_rn(v.x * sxs[c0 + i + 2 * k], v.y * sxs[c0 + i + 2 * k + 1]);
          }
          *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<uint4*>(h);
        }
      } else {
#pragma unroll
        for (int i = 0; i < COLS_PER_FOLD; ++i) {
          const int tok = tokp + c0 + i;
          if (tok < p.T)
            p.Y[(size_t)row * p.y_stride_n + (size_t)tok * p.y_stride_t] =
                __float2half_rn(((i & 1) ? unpack_f32x2(y2[i >> 1]).y : unpack_f32x2(y2[i >> 1]).x) * sxs[c0 + i]);
        }
      }
    }
  }

  // Common exit.  Every role of both CTAs falls through to here; neither CTA may retire (and neither may
  // release tensor memory) while the other could still arrive on its barriers or its MMAs are in flight.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, TMEM_COLS);
  }
}

}  // namespace pp
}  // namespace w4a4
