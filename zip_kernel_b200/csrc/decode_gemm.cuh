// Kernel 3: weight-streaming stream-K fused GEMM for small token counts (16
// tokens per CTA pass).  Replaces the reference's dp4a GEMV family
// (cuda_kernel/csrc/fused_dense_sparse/fused_gemv_decode.cu:54-191,
// fused_gemv_smallT.cu:47-221) and the split-K branch of its MMA kernel
// (fused_dense_sparse_mma_int4.cu:1597-1722, reduce :116-129).
//
//   Y[n,t] = fp16( sx[t] * ( sum_g s[n,g] * (acc[g,n,t] - z[n,g] * sumX[t,g])
//                            + w * sum_{blk in block-row} s[n,bc] * acc_hi[blk,n,t] ) )
//
// Work decomposition.  One "step" is a 128-row x 128-column tile of packed
// nibbles (8 KB): a group of the dense weights of one block-row, or one residual
// block.  All steps of the layer form one line, block-row after block-row, dense
// groups first and the row's residual blocks behind them:
//   first_step(r) = r * ng + hp_row_offsets[r].
// The line is cut into equal contiguous ranges, one per CTA, so every CTA
// streams the same number of bytes however N, K and the residual mask fall
// relative to the SM count.  A CTA that owns a whole block-row writes it out
// directly; a block-row shared by several CTAs meets in an fp32 workspace, and
// the CTA that arrives last at the row's counter adds the pieces in K order,
// applies scale_x and writes fp16.  Nothing ever waits for another CTA.
//
// Data flow per CTA.  A producer warp walks the range and, per step, issues
// three non-multicast asynchronous copies into one slot of an 8-deep
// shared-memory ring guarded by mbarriers: the weight tile (TMA, 8 KB), the
// matching 128-byte slice of the expanded activation codes of up to 16 tokens
// (TMA, 128-byte swizzle so fragment reads are conflict-free) and the 16 group
// sums (bulk copy).  Eight consumer warps (16 rows each) read their fragments
// with 128-bit loads, expand nibbles to s8 lanes scaled by 16 with three logic
// ops per word, run mma.sync m16n8k32 s8 (element order inside a group is
// permuted identically on both operands), and fold each group's int32
// accumulator in fp32 with the group's scale and zero, which every thread
// fetches with plain loads issued ahead of the slot wait.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace w4a4 {
namespace dec {

constexpr int ROWS = 128;
constexpr int CONSUMER_WARPS = 8;
constexpr int CONSUMER_THREADS = CONSUMER_WARPS * 32;
constexpr int THREADS = CONSUMER_THREADS + 32;
constexpr int STAGES = 8;
constexpr int TOK = 16;                           // tokens per CTA pass
constexpr int W_TILE_BYTES = ROWS * GROUP_BYTES;  // 8192
constexpr int X_TILE_BYTES = TOK * BCOL;          // 2048 (16 tokens x 128 codes)
constexpr int SUMX_BYTES = TOK * 4;               // 64
constexpr int STAGE_BYTES = W_TILE_BYTES + X_TILE_BYTES + 1024;
constexpr int MAX_ROW_TILES_SMEM = 2048;          // block-row offsets cached in shared memory

enum : int { SITE_DEC_FULL = 1, SITE_DEC_EMPTY = 2, SITE_DEC_DRAIN = 3, SITE_DEC_DUMP = 4 };

struct Params {
  const int* hp_row_offsets;
  const int* hp_col_indices;
  const __half* scale_u4;   // (N, ng)
  const __half* zero_u4;    // (N, ng) or nullptr
  const float* sumxf;       // [tok tiles][ng][16] or nullptr
  const __half* scale_x;    // (T)
  __half* Y;
  long long y_stride_n, y_stride_t;
  float* partial;           // [tok tiles][ctas + row tiles][128][16] fp32
  int* counters;            // [tok tiles][row tiles], zero between launches
  int* acc_dump;            // optional (ng, N, T) int32
  int* acc_hi_dump;         // optional (nnz, 128, T) int32
  int T, K, N, ng, nnz;
  int row_tiles;
  int nd;                   // dense steps per block-row (ng, or 0 when the dense part is off)
  int sparse_on;
  int steps_total;
  int steps_per_cta;        // 0: one whole block-row per CTA (no shared rows, no workspace)
  float sparse_weight;      // 16 (fused) or 1 (sparse-only op)
};

inline size_t smem_bytes() { return 1024 + (size_t)STAGES * STAGE_BYTES + (MAX_ROW_TILES_SMEM + 1) * 4 + 256; }

template <int NT, bool DUMP>
__global__ void __launch_bounds__(THREADS, 2)
decode_gemm_kernel(const __grid_constant__ CUtensorMap tm_low, const __grid_constant__ CUtensorMap tm_high,
                   const __grid_constant__ CUtensorMap tm_x, const Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* stage_buf = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  int* row_off = reinterpret_cast<int*>(stage_buf + STAGES * STAGE_BYTES);      // first_step(r), r = 0..row_tiles
  uint64_t* full = reinterpret_cast<uint64_t*>(row_off + MAX_ROW_TILES_SMEM + 2);
  uint64_t* empty = full + STAGES;
  int* misc = reinterpret_cast<int*>(empty + STAGES);     // [0] = last-arriver flag, [1] = a wait gave up

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int cta = blockIdx.x;
  const int tt = blockIdx.y;
  const int tok0 = tt * TOK;
  const int L = p.steps_per_cta;

  if (tid == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], CONSUMER_WARPS);
    }
    mbar_fence_init();
    misc[0] = 0;
    misc[1] = 0;
    tma_prefetch_desc(&tm_low);
    tma_prefetch_desc(&tm_high);
    tma_prefetch_desc(&tm_x);
  }
  // first_step(r) for every block-row (weights only: valid before the dependency wait)
  for (int r = tid; r <= p.row_tiles; r += THREADS)
    row_off[r] = r * p.nd + (p.sparse_on ? ld_plain(p.hp_row_offsets + r) : 0);
  __syncthreads();

  const int lo = L ? cta * L : row_off[cta];
  const int hi = L ? min(p.steps_total, lo + L) : row_off[cta + 1];
  // block-row that contains step `lo`: largest r with first_step(r) <= lo
  int r_first = cta;
  if (L) {
    int a = 0, b = p.row_tiles;            // invariant: row_off[a] <= lo < row_off[b] (lo < steps_total)
    while (b - a > 1) {
      const int m = (a + b) >> 1;
      if (row_off[m] <= lo) a = m; else b = m;
    }
    r_first = a;
  }

  if (warp == CONSUMER_WARPS) {
    // ------------------------------------------------------------ producer
    if (lane == 0 && lo < hi) {
      const bool with_sums = p.sumxf != nullptr;
      bool ok = true;
      int issued = 0;
      // Step `pos` of block-row r -> the slot's three copies.  The weight tile does
      // not depend on the preceding kernel in the stream, the other two do.
      auto issue = [&](int pos, int r, int n, bool weights, bool acts) {
        const int st = n % STAGES;
        unsigned char* slot = stage_buf + st * STAGE_BYTES;
        const int j = pos - row_off[r];
        const bool dense = j < p.nd;
        int blk = 0, g = j;
        if (!dense) {
          blk = ld_plain(p.hp_row_offsets + r) + j - p.nd;
          g = ld_plain(p.hp_col_indices + blk);
        }
        if (weights) {
          const uint32_t bytes = W_TILE_BYTES + NT * 8 * BCOL + ((dense && with_sums) ? SUMX_BYTES : 0);
          mbar_arrive_expect_tx(&full[st], bytes);
          if (dense) tma_load_2d(slot, &tm_low, g * GROUP_BYTES, r * ROWS, &full[st]);
          else       tma_load_2d(slot, &tm_high, 0, blk * BROW, &full[st]);
        }
        if (acts) {
          tma_load_2d(slot + W_TILE_BYTES, &tm_x, g * BCOL, tok0, &full[st]);
          if (dense && with_sums)
            bulk_load_1d(slot + W_TILE_BYTES + X_TILE_BYTES, p.sumxf + ((size_t)tt * p.ng + g) * TOK, SUMX_BYTES,
                         &full[st]);
        }
      };
      // ring fill: weight tiles first, then wait for the activations' producer kernel
      const int n_pre = min(STAGES, hi - lo);
      {
        int r = r_first;
        for (int n = 0; n < n_pre; ++n) {
          const int pos = lo + n;
          while (pos >= row_off[r + 1]) ++r;
          issue(pos, r, n, true, false);
        }
      }
      grid_dependency_wait();
      int r = r_first;
      for (int pos = lo; pos < hi; ++pos, ++issued) {
        while (pos >= row_off[r + 1]) ++r;
        if (issued < n_pre) {
          issue(pos, r, issued, false, true);
        } else {
          ok = mbar_wait(&empty[issued % STAGES], ((issued / STAGES) & 1) ^ 1, SITE_DEC_EMPTY);
          if (!ok) break;
          issue(pos, r, issued, true, true);
        }
      }
      if (!ok) {
        misc[1] = 1;
        // let copies already in flight land before the CTA may retire
        for (int i = max(0, issued - STAGES); i < issued; ++i)
          mbar_wait(&full[i % STAGES], (i / STAGES) & 1, SITE_DEC_DRAIN);
      }
    }
  } else if (lo < hi) {
    // ------------------------------------------------------------ consumers
    const int gid = lane >> 2;
    const int tig = lane & 3;
    const int r_a = warp * 16 + gid;      // local rows of this thread's fragments
    const int r_b = r_a + 8;
    grid_dependency_wait();               // scale_x, and the workspace of earlier launches

    float y[NT][4];
    bool ok = true;
    int consumed = 0;
    int pos = lo;
    // A wait that gives up clears `ok` for the whole warp; the loops still run to
    // their end (skipping the work) so that every named barrier below is reached.
    for (int r = r_first; pos < hi; ++r) {
      const int row_lo = row_off[r], row_hi = row_off[r + 1];
      const int seg_hi = min(hi, row_hi);
      if (seg_hi <= pos) continue;        // block-row without steps
      const int row0 = r * ROWS;
      const int blk0 = p.sparse_on ? ld_plain(p.hp_row_offsets + r) : 0;
      const size_t sz_a = (size_t)(row0 + r_a) * p.ng, sz_b = (size_t)(row0 + r_b) * p.ng;
      const bool live_a = row0 + r_a < p.N && p.scale_u4 != nullptr;
      const bool live_b = row0 + r_b < p.N && p.scale_u4 != nullptr;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) y[nt][i] = 0.f;

      for (; pos < seg_hi; ++pos, ++consumed) {
        const int j = pos - row_lo;
        const bool is_dense = j < p.nd;
        const int blk = blk0 + j - p.nd;
        const int g = is_dense ? j : ld_plain(p.hp_col_indices + blk);
        // group scale / zero of this thread's two rows, requested ahead of the slot wait
        float s_a = 0.f, s_b = 0.f, z_a = 0.f, z_b = 0.f;
        if (live_a) {
          s_a = __half2float(ld_plain(p.scale_u4 + sz_a + g));
          if (is_dense && p.zero_u4) z_a = __half2float(ld_plain(p.zero_u4 + sz_a + g));
        }
        if (live_b) {
          s_b = __half2float(ld_plain(p.scale_u4 + sz_b + g));
          if (is_dense && p.zero_u4) z_b = __half2float(ld_plain(p.zero_u4 + sz_b + g));
        }
        const int st = consumed % STAGES;
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&full[st], (consumed / STAGES) & 1, SITE_DEC_FULL));
        if (!ok) continue;
        const unsigned char* slot = stage_buf + st * STAGE_BYTES;
        const uint4 wa = *reinterpret_cast<const uint4*>(slot + r_a * GROUP_BYTES + tig * 16);
        const uint4 wb = *reinterpret_cast<const uint4*>(slot + r_b * GROUP_BYTES + tig * 16);
        uint4 q0[NT], q1[NT];
        float2 sx[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int xr = nt * 8 + gid;     // token row of the activation tile (128-byte swizzle)
          const unsigned char* xrow = slot + W_TILE_BYTES + xr * BCOL;
          q0[nt] = *reinterpret_cast<const uint4*>(xrow + (((2 * tig) ^ (xr & 7)) << 4));
          q1[nt] = *reinterpret_cast<const uint4*>(xrow + (((2 * tig + 1) ^ (xr & 7)) << 4));
          sx[nt] = (is_dense && p.sumxf)
                       ? *reinterpret_cast<const float2*>(slot + W_TILE_BYTES + X_TILE_BYTES + (nt * 8 + tig * 2) * 4)
                       : make_float2(0.f, 0.f);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);

        int acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[nt][i] = 0;
        const uint32_t wa_[4] = {wa.x, wa.y, wa.z, wa.w};
        const uint32_t wb_[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const uint32_t b0_[4] = {q0[nt].x, q0[nt].z, q1[nt].x, q1[nt].z};
          const uint32_t b1_[4] = {q0[nt].y, q0[nt].w, q1[nt].y, q1[nt].w};
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            mma_m16n8k32_s8(acc[nt], nib_lo_x16(wa_[jj]), nib_lo_x16(wb_[jj]), nib_hi_x16(wa_[jj]),
                            nib_hi_x16(wb_[jj]), b0_[jj], b1_[jj]);
        }

        // fold: accumulators carry a factor 16 from the weight expansion
        const float w = is_dense ? 0.0625f : 0.0625f * p.sparse_weight;
        const float fa = s_a * w, fb = s_b * w;
        const float ca = s_a * z_a, cb = s_b * z_b;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          y[nt][0] = fmaf((float)acc[nt][0], fa, fmaf(-ca, sx[nt].x, y[nt][0]));
          y[nt][1] = fmaf((float)acc[nt][1], fa, fmaf(-ca, sx[nt].y, y[nt][1]));
          y[nt][2] = fmaf((float)acc[nt][2], fb, fmaf(-cb, sx[nt].x, y[nt][2]));
          y[nt][3] = fmaf((float)acc[nt][3], fb, fmaf(-cb, sx[nt].y, y[nt][3]));
        }
        if (DUMP) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int rl = (i & 2) ? r_b : r_a;
              const int tok = tok0 + nt * 8 + tig * 2 + (i & 1);
              if (tok >= p.T) continue;
              // parity aid, not a hot path: every store is range-checked
              if (is_dense) {
                const size_t idx = ((size_t)g * p.N + row0 + rl) * p.T + tok;
                if (p.acc_dump && row0 + rl < p.N) {
                  if (g >= 0 && g < p.ng && idx < (size_t)p.ng * p.N * p.T) p.acc_dump[idx] = acc[nt][i] >> 4;
                  else record_error(SITE_DEC_DUMP, 1);
                }
              } else if (p.acc_hi_dump) {
                const size_t idx = ((size_t)blk * BROW + rl) * p.T + tok;
                if (blk >= 0 && blk < p.nnz && idx < (size_t)p.nnz * BROW * p.T) p.acc_hi_dump[idx] = acc[nt][i] >> 4;
                else record_error(SITE_DEC_DUMP, 2);
              }
            }
        }
      }

      // ---------------------------------------------------------- block-row done
      if (p.Y == nullptr) continue;
      const bool whole = (L == 0) || ((lo <= row_lo) && (row_hi <= hi));
      if (whole) {
        if (ok) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int row = row0 + ((i & 2) ? r_b : r_a);
              const int tok = tok0 + nt * 8 + tig * 2 + (i & 1);
              if (row < p.N && tok < p.T) {
                const float sxs = __half2float(ld_plain(p.scale_x + tok));
                p.Y[(size_t)row * p.y_stride_n + (size_t)tok * p.y_stride_t] = __float2half_rn(y[nt][i] * sxs);
              }
            }
        }
      } else {
        // shared block-row: park this CTA's piece, the last arriver adds them up
        const int first_cta = row_lo / L;
        const int n_pieces = (row_hi - 1) / L - first_cta + 1;
        const size_t tile = (size_t)ROWS * TOK;
        float* base = p.partial + (size_t)tt * (gridDim.x + p.row_tiles) * tile;
        float* dst = base + (size_t)(cta + r) * tile;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          *reinterpret_cast<float2*>(dst + r_a * TOK + nt * 8 + tig * 2) = make_float2(y[nt][0], y[nt][1]);
          *reinterpret_cast<float2*>(dst + r_b * TOK + nt * 8 + tig * 2) = make_float2(y[nt][2], y[nt][3]);
        }
        __threadfence();
        asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");
        if (tid == 0) {
          int* ctr = p.counters + tt * p.row_tiles + r;
          const int prev = atomicAdd(ctr, 1);
          const int last = (prev == n_pieces - 1);
          if (last) *ctr = 0;
          misc[0] = last;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");
        if (misc[0] && ok) {
          __threadfence();
          constexpr int NCOL = NT * 8;
          const float* src = base + (size_t)(first_cta + r) * tile;
          for (int i = tid; i < ROWS * NCOL; i += CONSUMER_THREADS) {
            const int rl = i / NCOL, col = i - rl * NCOL;
            const int row = row0 + rl, tok = tok0 + col;
            if (row >= p.N || tok >= p.T) continue;
            float v = 0.f;
            for (int c = 0; c < n_pieces; ++c) v += __ldcg(src + (size_t)c * tile + rl * TOK + col);
            v *= __half2float(ld_plain(p.scale_x + tok));
            p.Y[(size_t)row * p.y_stride_n + (size_t)tok * p.y_stride_t] = __float2half_rn(v);
          }
        }
      }
    }
    if (!ok) misc[1] = 1;
  }
}

}  // namespace dec
}  // namespace w4a4
