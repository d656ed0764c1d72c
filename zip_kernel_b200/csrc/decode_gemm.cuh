// Kernel 3: weight-streaming split-K fused GEMM for small token counts (M <= 16
// per CTA pass).  Replaces the reference's dp4a GEMV family
// (cuda_kernel/csrc/fused_dense_sparse/fused_gemv_decode.cu:54-191,
// fused_gemv_smallT.cu:47-221) and the split-K branch of its MMA kernel
// (fused_dense_sparse_mma_int4.cu:1597-1722, reduce :116-129).
//
//   Y[n,t] = fp16( sx[t] * ( sum_g s[n,g] * (acc[g,n,t] - z[n,g] * sumX[t,g])
//                            + w * sum_{blk in block-row} s[n,bc] * acc_hi[blk,n,t] ) )
//
// Data flow per CTA (128 output rows = one block-row, one K slice of S groups,
// 16 tokens):
//   * a producer warp streams 128x64-byte tiles of packed nibbles (one group of
//     the dense weights, then the residual blocks of this block-row whose
//     column falls in the slice) through an 8-stage shared-memory ring with
//     non-multicast TMA and mbarriers - 64 KB in flight per CTA keeps HBM busy;
//   * 8 consumer warps (16 rows each) read their fragments with conflict-free
//     128-bit loads, expand nibbles to s8 lanes scaled by 16 with three logic
//     ops per word, and issue mma.sync m16n8k32 s8 against the activation
//     codes, which were expanded to s8 once into shared memory; element order
//     inside a group is permuted identically on both operands;
//   * each group's int32 accumulator is folded in fp32 with the group's scale and
//     zero; K slices meet in an fp32 workspace and the CTA that arrives last at
//     the row tile's counter adds them in slice order, applies scale_x and
//     writes fp16.  Nothing spins on another CTA.
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
constexpr int STAGE_BYTES = ROWS * GROUP_BYTES;   // 8192
constexpr int TOK = 16;                           // tokens per CTA
constexpr int S_MAX = 16;                         // groups per K slice

enum : int { SITE_DEC_FULL = 1, SITE_DEC_EMPTY = 2, SITE_DEC_DRAIN = 3 };

struct Params {
  const int* hp_row_offsets;
  const int* hp_col_indices;
  const int8_t* X_s4;       // (T, K/2)
  const __half* scale_u4;   // (N, ng)
  const __half* zero_u4;    // (N, ng)
  const int* sum_X;         // (T, ng)
  const __half* scale_x;    // (T)
  __half* Y;
  long long y_stride_n, y_stride_t;
  float* partial;           // [tok tiles][split_k][row tiles*128][16] fp32
  int* counters;            // [tok tiles][row tiles], zero between launches
  int* acc_dump;            // optional (ng, N, T) int32
  int* acc_hi_dump;         // optional (nnz, 128, T) int32
  int T, K, N, ng, nnz;
  int S;                    // groups per K slice (<= S_MAX)
  int split_k;              // CTAs along K; each walks slices_per_cta consecutive slices
  int slices_per_cta;
  int do_dense;
  float sparse_weight;      // 16 (fused), 1 (sparse-only op), 0 = residual off
};

__host__ __device__ inline int x_row_stride(int S) { return S * BCOL + 16; }

inline size_t smem_bytes(int S) {
  return 1024 /*align slack*/ + (size_t)STAGES * STAGE_BYTES + (size_t)TOK * x_row_stride(S) +
         (size_t)S * ROWS * sizeof(float2) + (size_t)S * TOK * sizeof(float) + 256;
}

template <int NT, bool DUMP>
__global__ void __launch_bounds__(THREADS)
decode_gemm_kernel(const __grid_constant__ CUtensorMap tm_low,
                   const __grid_constant__ CUtensorMap tm_high, const Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* stage_buf = base;
  unsigned char* xs = stage_buf + STAGES * STAGE_BYTES;
  const int xstride = x_row_stride(p.S);
  float2* szs = reinterpret_cast<float2*>(xs + TOK * xstride);          // (s/16, s*z)
  float* sumxs = reinterpret_cast<float*>(szs + p.S * ROWS);
  uint64_t* full = reinterpret_cast<uint64_t*>(sumxs + p.S * TOK);
  uint64_t* empty = full + STAGES;
  int* misc = reinterpret_cast<int*>(empty + STAGES);                    // [2]=last arriver [3]=a wait gave up

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int br = blockIdx.x;
  const int kpart = blockIdx.y;
  const int tt = blockIdx.z;
  const int row0 = br * ROWS;
  const int tok0 = tt * TOK;
  const int n_slices = (p.ng + p.S - 1) / p.S;
  const int slice_begin = kpart * p.slices_per_cta;
  const int slice_end = min(n_slices, slice_begin + p.slices_per_cta);
  const bool sparse_on = p.sparse_weight != 0.f && p.nnz > 0;
  const int blk_begin = sparse_on ? __ldg(p.hp_row_offsets + br) : 0;
  const int blk_end = sparse_on ? __ldg(p.hp_row_offsets + br + 1) : 0;

  if (tid == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], CONSUMER_WARPS);
    }
    mbar_fence_init();
    misc[2] = 0;
    misc[3] = 0;
    tma_prefetch_desc(&tm_low);
    tma_prefetch_desc(&tm_high);
  }
  __syncthreads();

  if (warp == CONSUMER_WARPS) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int issued = 0;
      bool ok = true;
      int blk = blk_begin;
      for (int sl = slice_begin; sl < slice_end && ok; ++sl) {
        const int g0 = sl * p.S, g1 = min(p.ng, g0 + p.S);
        const int n_dense = p.do_dense ? (g1 - g0) : 0;
        // residual blocks of this block-row whose column lies in [g0, g1)
        while (blk < blk_end && __ldg(p.hp_col_indices + blk) < g0) ++blk;
        int b_hi = blk;
        while (b_hi < blk_end && __ldg(p.hp_col_indices + b_hi) < g1) ++b_hi;
        const int nsteps = n_dense + (b_hi - blk);
        for (int step = 0; step < nsteps; ++step, ++issued) {
          const int st = issued % STAGES;
          ok = mbar_wait(&empty[st], ((issued / STAGES) & 1) ^ 1, SITE_DEC_EMPTY);
          if (!ok) break;
          mbar_arrive_expect_tx(&full[st], STAGE_BYTES);
          if (step < n_dense)
            tma_load_2d(stage_buf + st * STAGE_BYTES, &tm_low, (g0 + step) * GROUP_BYTES, row0, &full[st]);
          else
            tma_load_2d(stage_buf + st * STAGE_BYTES, &tm_high, 0, (blk + step - n_dense) * BROW, &full[st]);
        }
        blk = b_hi;
      }
      if (!ok) {
        misc[3] = 1;
        // let copies already in flight land before the CTA may retire
        for (int i = max(0, issued - STAGES); i < issued; ++i)
          mbar_wait(&full[i % STAGES], (i / STAGES) & 1, SITE_DEC_DRAIN);
      }
    }
    __syncwarp();
    grid_dependency_wait();   // this warp joins the slice reduction below
  } else {
    // ------------------------------------------------------------ consumers
    const int gid = lane >> 2;
    const int tig = lane & 3;
    const int r_a = warp * 16 + gid;      // local rows of this thread's fragments
    const int r_b = r_a + 8;

    float y[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) y[nt][i] = 0.f;

    bool ok = true;
    int consumed = 0;
    int blk_cursor = blk_begin;
    // A wait that gives up clears `ok` for the whole warp; the loops still run to
    // their end (skipping the work) so that every named barrier below is reached.
    for (int sl = slice_begin; sl < slice_end; ++sl) {
      const int g0 = sl * p.S, g1 = min(p.ng, g0 + p.S);
      const int n_dense = p.do_dense ? (g1 - g0) : 0;
      while (blk_cursor < blk_end && __ldg(p.hp_col_indices + blk_cursor) < g0) ++blk_cursor;
      const int b_lo = blk_cursor;
      while (blk_cursor < blk_end && __ldg(p.hp_col_indices + blk_cursor) < g1) ++blk_cursor;
      const int nsteps = n_dense + (blk_cursor - b_lo);

      // every consumer is done with the previous slice's shared operands
      if (sl != slice_begin) asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");

      // weights-side prologue: (s/16, s*z) per (group, row) of the slice
      if (tid < ROWS) {
        const int row = row0 + tid;
        for (int gl = 0; gl < g1 - g0; ++gl) {
          float s = 0.f, z = 0.f;
          if (row < p.N && p.scale_u4) {
            s = __half2float(__ldg(p.scale_u4 + (size_t)row * p.ng + g0 + gl));
            z = p.zero_u4 ? __half2float(__ldg(p.zero_u4 + (size_t)row * p.ng + g0 + gl)) : 0.f;
          }
          szs[gl * ROWS + tid] = make_float2(s * 0.0625f, s * z);
        }
      }
      // activations come from the preceding kernel in the stream
      if (sl == slice_begin) grid_dependency_wait();
      {
        const int words_per_row = (g1 - g0) * 16;
        const int total = TOK * words_per_row;
        for (int wi = tid; wi < total; wi += CONSUMER_THREADS) {
          const int tok = wi / words_per_row;
          const int w_in = wi - tok * words_per_row;
          uint32_t w = 0;
          if (tok0 + tok < p.T)
            w = __ldg(reinterpret_cast<const uint32_t*>(p.X_s4 + (size_t)(tok0 + tok) * (p.K >> 1) +
                                                        (size_t)g0 * GROUP_BYTES) + w_in);
          *reinterpret_cast<uint2*>(xs + tok * xstride + w_in * 8) = make_uint2(nib_lo_s8(w), nib_hi_s8(w));
        }
        for (int i = tid; i < (g1 - g0) * TOK; i += CONSUMER_THREADS) {
          const int gl = i / TOK, tok = i - gl * TOK;
          float v = 0.f;
          if (p.sum_X && tok0 + tok < p.T) v = (float)__ldg(p.sum_X + (size_t)(tok0 + tok) * p.ng + g0 + gl);
          sumxs[i] = v;
        }
      }
      asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");

      for (int step = 0; step < nsteps; ++step, ++consumed) {
        const int st = consumed % STAGES;
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&full[st], (consumed / STAGES) & 1, SITE_DEC_FULL));
        if (!ok) continue;
        const unsigned char* sA = stage_buf + st * STAGE_BYTES;
        const uint4 wa = *reinterpret_cast<const uint4*>(sA + r_a * GROUP_BYTES + tig * 16);
        const uint4 wb = *reinterpret_cast<const uint4*>(sA + r_b * GROUP_BYTES + tig * 16);
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);

        const bool is_dense = step < n_dense;
        const int blk = b_lo + step - n_dense;
        const int gl = is_dense ? step : (__ldg(p.hp_col_indices + blk) - g0);

        int acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[nt][i] = 0;

        const uint32_t wa_[4] = {wa.x, wa.y, wa.z, wa.w};
        const uint32_t wb_[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const unsigned char* xb = xs + (nt * 8 + gid) * xstride + gl * BCOL + tig * 32;
          const uint4 q0 = *reinterpret_cast<const uint4*>(xb);
          const uint4 q1 = *reinterpret_cast<const uint4*>(xb + 16);
          const uint32_t b0_[4] = {q0.x, q0.z, q1.x, q1.z};
          const uint32_t b1_[4] = {q0.y, q0.w, q1.y, q1.w};
#pragma unroll
          for (int j = 0; j < 4; ++j)
            mma_m16n8k32_s8(acc[nt], nib_lo_x16(wa_[j]), nib_lo_x16(wb_[j]), nib_hi_x16(wa_[j]),
                            nib_hi_x16(wb_[j]), b0_[j], b1_[j]);
        }

        const float2 sz_a = szs[gl * ROWS + r_a];
        const float2 sz_b = szs[gl * ROWS + r_b];
        if (is_dense) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const float2 sx = *reinterpret_cast<const float2*>(sumxs + gl * TOK + nt * 8 + tig * 2);
            y[nt][0] = fmaf((float)acc[nt][0], sz_a.x, fmaf(-sz_a.y, sx.x, y[nt][0]));
            y[nt][1] = fmaf((float)acc[nt][1], sz_a.x, fmaf(-sz_a.y, sx.y, y[nt][1]));
            y[nt][2] = fmaf((float)acc[nt][2], sz_b.x, fmaf(-sz_b.y, sx.x, y[nt][2]));
            y[nt][3] = fmaf((float)acc[nt][3], sz_b.x, fmaf(-sz_b.y, sx.y, y[nt][3]));
          }
        } else {
          const float wa_s = sz_a.x * p.sparse_weight, wb_s = sz_b.x * p.sparse_weight;
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            y[nt][0] = fmaf((float)acc[nt][0], wa_s, y[nt][0]);
            y[nt][1] = fmaf((float)acc[nt][1], wa_s, y[nt][1]);
            y[nt][2] = fmaf((float)acc[nt][2], wb_s, y[nt][2]);
            y[nt][3] = fmaf((float)acc[nt][3], wb_s, y[nt][3]);
          }
        }
        if (DUMP) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int rl = (i & 2) ? r_b : r_a;
              const int tok = tok0 + nt * 8 + tig * 2 + (i & 1);
              if (tok >= p.T) continue;
              if (is_dense) {
                if (p.acc_dump && row0 + rl < p.N)
                  p.acc_dump[((size_t)(g0 + gl) * p.N + row0 + rl) * p.T + tok] = acc[nt][i] >> 4;
              } else if (p.acc_hi_dump) {
                p.acc_hi_dump[((size_t)blk * BROW + rl) * p.T + tok] = acc[nt][i] >> 4;
              }
            }
        }
      }
    }
    if (!ok) misc[3] = 1;

    // ---------------------------------------------------------- epilogue
    if (ok && p.Y) {
      if (p.split_k == 1) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int row = row0 + ((i & 2) ? r_b : r_a);
            const int tok = tok0 + nt * 8 + tig * 2 + (i & 1);
            if (row < p.N && tok < p.T) {
              const float sx = __half2float(__ldg(p.scale_x + tok));
              p.Y[(size_t)row * p.y_stride_n + (size_t)tok * p.y_stride_t] = __float2half_rn(y[nt][i] * sx);
            }
          }
      } else {
        float* dst = p.partial + ((size_t)(tt * p.split_k + kpart) * gridDim.x * ROWS + row0) * TOK;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          *reinterpret_cast<float2*>(dst + r_a * TOK + nt * 8 + tig * 2) = make_float2(y[nt][0], y[nt][1]);
          *reinterpret_cast<float2*>(dst + r_b * TOK + nt * 8 + tig * 2) = make_float2(y[nt][2], y[nt][3]);
        }
      }
    }
  }

  if (p.split_k > 1) {
    // last CTA to arrive at this row tile's counter folds the slices in order
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      int* ctr = p.counters + tt * gridDim.x + br;
      const int prev = atomicAdd(ctr, 1);
      const int last = (prev == p.split_k - 1);
      if (last) *ctr = 0;
      misc[2] = last;
    }
    __syncthreads();
    if (misc[2] && !misc[3]) {
      __threadfence();
      const size_t slice_stride = (size_t)gridDim.x * ROWS * TOK;
      const float* src = p.partial + ((size_t)tt * p.split_k * gridDim.x * ROWS + row0) * TOK;
      constexpr int NCOL = NT * 8;
      for (int i = tid; i < ROWS * NCOL; i += THREADS) {
        const int rl = i / NCOL, col = i - rl * NCOL;
        const int row = row0 + rl, tok = tok0 + col;
        if (row >= p.N || tok >= p.T) continue;
        float v = 0.f;
        for (int s = 0; s < p.split_k; ++s) v += __ldcg(src + s * slice_stride + rl * TOK + col);
        v *= __half2float(__ldg(p.scale_x + tok));
        p.Y[(size_t)row * p.y_stride_n + (size_t)tok * p.y_stride_t] = __float2half_rn(v);
      }
    }
  }
}

}  // namespace dec
}  // namespace w4a4
