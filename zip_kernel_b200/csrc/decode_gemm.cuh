// Kernel 3: weight-streaming split-K fused GEMM for small token counts (16
// tokens per CTA pass).  Replaces the reference's dp4a GEMV family
// (cuda_kernel/csrc/fused_dense_sparse/fused_gemv_decode.cu:54-191,
// fused_gemv_smallT.cu:47-221) and the split-K branch of its MMA kernel
// (fused_dense_sparse_mma_int4.cu:1597-1722, reduce :116-129).
//
//   Y[n,t] = fp16( sx[t] * ( sum_g s[n,g] * (acc[g,n,t] - z[n,g] * sumX[t,g])
//                            + w * sum_{blk in block-row} s[n,bc] * acc_hi[blk,n,t] ) )
//
// Work decomposition.  One "step" is a tile of packed nibbles of one block-row
// (128 rows): two adjacent groups of the dense weights (128 x 128 bytes = 16 KB,
// so every TMA row is a full 128-byte line), or one residual block (8 KB,
// contiguous).  A block-row is owned by a thread-block cluster of S CTAs
// (S = 1..8, chosen so that the grid fills the SMs about twice): CTA k of the
// cluster takes the k-th share of the row's dense steps - known without reading
// memory, so its first weight copies leave at once - and the k-th share of the
// row's residual blocks.  When the row is finished the S partial tiles meet in
// distributed shared memory: every CTA parks its 128 x 16 fp32 tile in its own
// shared memory, the cluster synchronises, and CTA k adds rows
// [k*128/S, (k+1)*128/S) of all S tiles in rank order, applies scale_x and
// writes fp16.  No global-memory round trip, counter or workspace is involved,
// and nothing waits on a CTA outside its own cluster.
//
// Data flow per CTA.  A producer warp walks the range and, per step, issues
// non-multicast asynchronous copies into one slot of a 4-deep shared-memory
// ring guarded by mbarriers: the weight tile (TMA, or a plain bulk copy for a
// residual block), the expanded activation codes of up to 16 tokens for the same
// groups (one contiguous bulk copy per group; the layout is pre-swizzled so
// fragment reads are conflict-free) and the group sums (bulk copy).  Eight consumer warps (16 rows each) read
// their fragments with 128-bit loads, expand nibbles to s8 lanes scaled by 16
// with three logic ops per word, run mma.sync m16n8k32 s8 on the two groups as
// independent chains (element order inside a group is permuted identically on
// both operands), and fold each group's int32 accumulator in fp32 with the
// group's scale and zero using packed f32x2 FMAs.  Scales and zeros of the
// CTA's 128 rows are staged in shared memory 16 groups at a time with 128-bit
// loads that are issued one span ahead and parked in registers, so the loop
// never waits on a scattered 2-byte load.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace w4a4 {
namespace dec {

constexpr int ROWS = 128;
constexpr int CONSUMER_WARPS = 8;
constexpr int CONSUMER_THREADS = CONSUMER_WARPS * 32;
constexpr int THREADS = CONSUMER_THREADS + 32;
constexpr int W_TILE_BYTES = ROWS * 2 * GROUP_BYTES;   // 16384: 128 rows x two groups
constexpr int BLK_BYTES = BROW * GROUP_BYTES;     // 8192: one residual block
constexpr int MAX_STAGES = 4;
// Tile geometry of an instantiation: NT = 8-token MMA tiles per CTA pass.  Up to
// 16 tokens a pass covers 16 tokens and the ring is 4 deep; NT = 4 covers 32
// tokens per pass (weights are streamed once for up to 32 tokens) with a 3-deep
// ring so that two CTAs still share an SM.
template <int NT>
struct Tile {
  static constexpr int TOK = NT > 2 ? 32 : 16;            // tokens per CTA pass
  static constexpr int STAGES = NT > 2 ? 3 : 4;
  static constexpr int NTH = NT > 2 ? 2 : NT;             // MMA tiles handled together (register pressure)
  static constexpr int HALVES = NT / NTH;
  static constexpr int X_TILE_BYTES = TOK * BCOL;         // per group
  static constexpr int SUMX_BYTES = TOK * 4;              // per group: one 64-byte piece per 16 tokens
  static constexpr int STAGE_BYTES = W_TILE_BYTES + 2 * X_TILE_BYTES;   // group sums live in a ring of their own
  static constexpr size_t SMEM = 1024 + (size_t)STAGES * STAGE_BYTES + STAGES * 2 * SUMX_BYTES + 16 * ROWS * 8 + 256;
};
constexpr int MAX_CLUSTER = 8;                    // portable cluster size limit
constexpr int SZ_CHUNK = 16;                      // groups of scale/zero staged per span
constexpr int SZ_BYTES = SZ_CHUNK * ROWS * 8;     // float2 (scale/16, scale*zero) per (group, row)

enum : int { SITE_DEC_FULL = 1, SITE_DEC_EMPTY = 2, SITE_DEC_DRAIN = 3, SITE_DEC_DUMP = 4 };

struct Params {
  const int* hp_row_offsets;
  const int* hp_col_indices;
  const int8_t* W_high;     // (nnz, 128, 64) residual blocks
  const int8_t* XE;         // expanded activation codes, group-major [ng][t_pad][128]
  int t_pad;
  const __half* scale_u4;   // (N, ng)
  const __half* zero_u4;    // (N, ng) or nullptr
  const float* sumxf;       // [tok tiles][ng][16] or nullptr
  const __half* scale_x;    // (T)
  __half* Y;
  long long y_stride_n, y_stride_t;
  int* acc_dump;            // optional (ng, N, T) int32
  int* acc_hi_dump;         // optional (nnz, 128, T) int32
  int T, K, N, ng, nnz;
  int row_tiles;
  int nd;                   // dense steps per block-row (ceil(ng/2), or 0 when the dense part is off)
  int sparse_on;
  int sz_vec;               // scale/zero rows may be read with 128-bit loads
  int split;                // CTAs per block-row (= cluster size along x)
  float sparse_weight;      // 16 (fused) or 1 (sparse-only op)
};

inline size_t smem_bytes(int nt) { return nt > 2 ? Tile<4>::SMEM : Tile<1>::SMEM; }
inline int tokens_per_pass(int nt) { return nt > 2 ? Tile<4>::TOK : Tile<1>::TOK; }

// ---- thread-block cluster helpers (no multicast; plain distributed-shared-memory loads)
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// All threads of all CTAs of the cluster arrive; hardware barrier, not a spin loop.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_dsmem_f32(const void* own_smem_ptr, uint32_t peer_rank) {
  uint32_t remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(own_smem_ptr)), "r"(peer_rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// d = a * b + c on two packed fp32 lanes
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(*reinterpret_cast<unsigned long long*>(&d))
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return d;
}

// D(16x8,s32) = A(16x32,s8,row) * B(32x8,s8,col) with a zero accumulator input
__device__ __forceinline__ void mma_m16n8k32_s8_first(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                      uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// The A fragments of one group of one warp (16 rows x 128 codes): nibbles widened to s8 lanes x 16.
struct AFrag { uint32_t a[4][4]; };
__device__ __forceinline__ AFrag unpack_a(const uint4& wa, const uint4& wb) {
  const uint32_t wa_[4] = {wa.x, wa.y, wa.z, wa.w};
  const uint32_t wb_[4] = {wb.x, wb.y, wb.z, wb.w};
  AFrag f;
#pragma unroll
  for (int jj = 0; jj < 4; ++jj) {
    f.a[jj][0] = nib_lo_x16(wa_[jj]);
    f.a[jj][1] = nib_lo_x16(wb_[jj]);
    f.a[jj][2] = nib_hi_x16(wa_[jj]);
    f.a[jj][3] = nib_hi_x16(wb_[jj]);
  }
  return f;
}
// One group of one warp against NT*8 tokens.
template <int NT>
__device__ __forceinline__ void group_mma(int (&acc)[NT][4], const AFrag& f, const uint4 (&q0)[NT], const uint4 (&q1)[NT]) {
#pragma unroll
  for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const uint32_t b0_[4] = {q0[nt].x, q0[nt].z, q1[nt].x, q1[nt].z};
      const uint32_t b1_[4] = {q0[nt].y, q0[nt].w, q1[nt].y, q1[nt].w};
      if (jj == 0) mma_m16n8k32_s8_first(acc[nt], f.a[jj][0], f.a[jj][1], f.a[jj][2], f.a[jj][3], b0_[jj], b1_[jj]);
      else         mma_m16n8k32_s8(acc[nt], f.a[jj][0], f.a[jj][1], f.a[jj][2], f.a[jj][3], b0_[jj], b1_[jj]);
    }
  }
}

// y += acc * f - c * sumx   for the thread's two rows (a: acc[0..1], b: acc[2..3])
template <int NT>
__device__ __forceinline__ void group_fold(float2 (*y)[2], const int (&acc)[NT][4], float fa, float fb, float ca,
                                           float cb, const float2 (&sx)[NT]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const float2 ta = fma2(make_float2(-ca, -ca), sx[nt], y[nt][0]);
    const float2 tb = fma2(make_float2(-cb, -cb), sx[nt], y[nt][1]);
    y[nt][0] = fma2(make_float2(__int2float_rn(acc[nt][0]), __int2float_rn(acc[nt][1])), make_float2(fa, fa), ta);
    y[nt][1] = fma2(make_float2(__int2float_rn(acc[nt][2]), __int2float_rn(acc[nt][3])), make_float2(fb, fb), tb);
  }
}

template <int NT, bool DUMP>
__global__ void __launch_bounds__(THREADS, 2)
decode_gemm_kernel(const __grid_constant__ CUtensorMap tm_low, const Params p) {
  using TL = Tile<NT>;
  constexpr int TOK = TL::TOK, STAGES = TL::STAGES, NTH = TL::NTH, HALVES = TL::HALVES;
  constexpr int X_TILE_BYTES = TL::X_TILE_BYTES, SUMX_BYTES = TL::SUMX_BYTES, STAGE_BYTES = TL::STAGE_BYTES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* stage_buf = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sumx_ring = stage_buf + STAGES * STAGE_BYTES;
  float2* szs = reinterpret_cast<float2*>(sumx_ring + STAGES * 2 * SUMX_BYTES);   // [16 groups][128 rows] (s/16, s*z)
  uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(szs) + SZ_BYTES);
  uint64_t* empty = full + MAX_STAGES;
  int* misc = reinterpret_cast<int*>(empty + MAX_STAGES);     // [1] = a wait gave up

  // the next kernel in the stream may be scheduled as soon as every CTA got here;
  // it waits for this grid's completion before it touches anything we use
  grid_launch_dependents();
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int S = p.split;
  const int rank = S > 1 ? (int)cluster_ctarank() : 0;   // == blockIdx.x % S
  const int r = blockIdx.x / S;                            // block-row of this cluster
  const int tt = blockIdx.y;
  const int tok0 = tt * TOK;
  const int row0 = r * ROWS;
  constexpr int XG_BYTES = NT * 8 * BCOL;     // activation bytes actually copied per group
  // this CTA's share of the dense steps of the block-row: needs no memory access
  const int d_lo = (int)((long long)rank * p.nd / S), d_hi = (int)((long long)(rank + 1) * p.nd / S);

  if (tid == 0) {
    for (int i = 0; i < STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], CONSUMER_WARPS);
    }
    mbar_fence_init();
    misc[1] = 0;
    tma_prefetch_desc(&tm_low);
  }
  __syncthreads();

  if (warp == CONSUMER_WARPS) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      const bool with_sums = p.sumxf != nullptr;
      // the sums table is cut into 16-token tiles; a pass covers TOK / 16 of them (the last pass maybe fewer)
      const int tiles16 = (p.T + 15) >> 4;
      const int n_u = with_sums ? min(TOK / 16, tiles16 - tt * (TOK / 16)) : 0;
      bool ok = true;
      // The weight copy of a step does not depend on the preceding kernel in the
      // stream, the activation copies do.  Dense step j covers groups 2j, 2j+1.
      // the tokens' codes of one group are one contiguous run in the expanded layout
      auto x_src = [&](int g) { return p.XE + ((size_t)g * p.t_pad + tok0) * BCOL; };
      auto dense_w = [&](int j, int st) {
        const int n_grp = (2 * j + 1 < p.ng) ? 2 : 1;
        mbar_arrive_expect_tx(&full[st], W_TILE_BYTES + n_grp * XG_BYTES + n_u * n_grp * 64);
        tma_load_2d(stage_buf + st * STAGE_BYTES, &tm_low, 2 * j * GROUP_BYTES, row0, &full[st]);
      };
      auto dense_x = [&](int j, int st) {
        unsigned char* xt = stage_buf + st * STAGE_BYTES + W_TILE_BYTES;
        bulk_load_1d(xt, x_src(2 * j), XG_BYTES, &full[st]);
        if (2 * j + 1 < p.ng) bulk_load_1d(xt + X_TILE_BYTES, x_src(2 * j + 1), XG_BYTES, &full[st]);
        // slot layout of the sums: [16-token tile][group of the step][16 tokens]
        for (int u = 0; u < n_u; ++u)
          bulk_load_1d(sumx_ring + st * 2 * SUMX_BYTES + u * 128,
                       p.sumxf + ((size_t)(tt * (TOK / 16) + u) * p.ng + 2 * j) * 16,
                       ((2 * j + 1 < p.ng) ? 2 : 1) * 64, &full[st]);
      };
      // ring fill: weight tiles first, then wait for the activations' producer kernel
      const int n_dense = d_hi - d_lo;
      const int n_pre = min(STAGES, n_dense);
      for (int n = 0; n < n_pre; ++n) dense_w(d_lo + n, n);
      // this CTA's share of the residual blocks of the block-row
      int b_lo = 0, b_hi = 0;
      if (p.sparse_on) {
        const int o0 = ld_plain(p.hp_row_offsets + r), o1 = ld_plain(p.hp_row_offsets + r + 1);
        b_lo = o0 + (int)((long long)rank * (o1 - o0) / S);
        b_hi = o0 + (int)((long long)(rank + 1) * (o1 - o0) / S);
      }
      grid_dependency_wait_for_async_reads();
      int st = 0, n = 0;
      uint32_t ph = 1;                     // parity the empty barrier is waited on
      for (int j = d_lo; j < d_hi && ok; ++j, ++n) {
        if (n >= n_pre) {
          ok = mbar_wait(&empty[st], ph, SITE_DEC_EMPTY);
          if (!ok) break;
          dense_w(j, st);
        }
        dense_x(j, st);
        if (++st == STAGES) { st = 0; ph ^= 1; }
      }
      for (int blk = b_lo; blk < b_hi && ok; ++blk, ++n) {
        ok = mbar_wait(&empty[st], ph, SITE_DEC_EMPTY);
        if (!ok) break;
        unsigned char* slot = stage_buf + st * STAGE_BYTES;
        mbar_arrive_expect_tx(&full[st], BLK_BYTES + XG_BYTES);
        bulk_load_1d(slot, p.W_high + (size_t)blk * BLK_BYTES, BLK_BYTES, &full[st]);
        bulk_load_1d(slot + W_TILE_BYTES, x_src(ld_plain(p.hp_col_indices + blk)), XG_BYTES, &full[st]);
        if (++st == STAGES) { st = 0; ph ^= 1; }
      }
      if (!ok) {
        misc[1] = 1;
        // let copies already in flight land before the CTA may retire
        for (int i = max(0, n - STAGES); i < n; ++i)
          mbar_wait(&full[i % STAGES], (i / STAGES) & 1, SITE_DEC_DRAIN);
      }
    }
  } else {
    // ------------------------------------------------------------ consumers
    const int gid = lane >> 2;
    const int tig = lane & 3;
    // Local rows of this thread's fragments.  Which weight row feeds MMA row `gid` is free (the epilogue
    // writes row r_a), so the two rows a quarter-warp reads together are chosen to differ in bit 0 and in
    // bit 2: a dense tile (128-byte rows, 16-byte chunks stored at chunk ^ (row & 7) by the tensor map's
    // 128-byte swizzle) and a residual block (64-byte rows, unswizzled) are then both read without bank
    // conflicts - rows 0,5 | 1,4 | 2,7 | 3,6.
    const int r_a = warp * 16 + ((0x63724150u >> (4 * gid)) & 7);
    const int r_b = r_a + 8;
    // group 2j of a dense step; group 2j + 1 sits at chunk (4 + tig) ^ (r_a & 7): the same address with bit 6 flipped
    const int w_off = r_a * (2 * GROUP_BYTES) + ((tig ^ (r_a & 7)) << 4);

    // Per-thread constant offsets inside a slot.  An activation tile is a stack of
    // 128-byte lines (one per token) whose 16-byte chunks sit at chunk ^ (token & 7);
    // a dense step holds one tile per group, X_TILE_BYTES apart.
    // token nt * 8 + gid: (token & 7) == gid for every nt, so MMA tile nt sits 8 lines further on
    const int xs0 = W_TILE_BYTES + gid * BCOL + (((2 * tig) ^ gid) << 4);
    const int xs1 = W_TILE_BYTES + gid * BCOL + (((2 * tig + 1) ^ gid) << 4);
    constexpr int XNT = 8 * BCOL;         // bytes between consecutive MMA tiles of tokens

    const uint32_t stage_a = smem_u32(stage_buf), sumx_a = smem_u32(sumx_ring), szs_a = smem_u32(szs);

    const uint32_t runtime_zero = (uint32_t)p.ng >> 31;      // 0, unknown to the compiler (see the slot hand-back)
    float2 y[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) y[nt][0] = y[nt][1] = make_float2(0.f, 0.f);
    bool ok = true;
    int consumed = 0;
    int b_lo = 0, b_hi = 0;
    if (p.sparse_on) {
      const int o0 = ld_plain(p.hp_row_offsets + r), o1 = ld_plain(p.hp_row_offsets + r + 1);
      b_lo = o0 + (int)((long long)rank * (o1 - o0) / S);
      b_hi = o0 + (int)((long long)(rank + 1) * (o1 - o0) / S);
    }

    // The dense share is walked in spans that lie inside one aligned window of 16
    // groups (8 steps); the residual blocks form a last span.
    struct Span { int j0, j1, dense; };
    auto walk = [&](int& j, int& did_sparse, Span& sp) -> bool {
      if (j < d_hi) {
        sp.j0 = j;
        sp.j1 = min(d_hi, (j / (SZ_CHUNK / 2) + 1) * (SZ_CHUNK / 2));
        sp.dense = 1;
        j = sp.j1;
        return true;
      }
      if (!did_sparse && b_lo < b_hi) {
        did_sparse = 1;
        sp.j0 = b_lo;
        sp.j1 = b_hi;
        sp.dense = 0;
        return true;
      }
      return false;
    };
    // Scale/zero window of a dense span: thread t fetches 8 groups of row t/2
    // (one 128-bit load from each array when rows are 16-byte aligned) and parks
    // them as (scale/16, scale*zero): the accumulators carry a factor 16 from the
    // weight expansion.
    const int lrow = tid >> 1, lhalf = tid & 1;
    uint4 ps, pz;
    auto fetch_sz = [&](const Span& sp) {
      ps = pz = make_uint4(0, 0, 0, 0);
      if (!sp.dense || p.scale_u4 == nullptr) return;
      const int row = row0 + lrow;
      if (row >= p.N) return;
      const int g = (2 * sp.j0 / SZ_CHUNK) * SZ_CHUNK + lhalf * 8;
      if (g >= p.ng) return;
      const __half* srow = p.scale_u4 + (size_t)row * p.ng;
      const __half* zrow = p.zero_u4 ? p.zero_u4 + (size_t)row * p.ng : nullptr;
      if (p.sz_vec) {
        ps = *reinterpret_cast<const uint4*>(srow + g);
        if (zrow) pz = *reinterpret_cast<const uint4*>(zrow + g);
      } else {
        __half hs[8], hz[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          hs[i] = (g + i < p.ng) ? srow[g + i] : __float2half(0.f);
          hz[i] = (g + i < p.ng && zrow) ? zrow[g + i] : __float2half(0.f);
        }
        ps = *reinterpret_cast<uint4*>(&hs[0]);
        pz = *reinterpret_cast<uint4*>(&hz[0]);
      }
    };
    auto park_sz = [&]() {
      const __half2* hs = reinterpret_cast<const __half2*>(&ps);
      const __half2* hz = reinterpret_cast<const __half2*>(&pz);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 s2 = __half22float2(hs[i]), z2 = __half22float2(hz[i]);
        sts_f2(szs_a + ((lhalf * 8 + 2 * i) * ROWS + lrow) * 8, make_float2(s2.x * 0.0625f, s2.x * z2.x));
        sts_f2(szs_a + ((lhalf * 8 + 2 * i + 1) * ROWS + lrow) * 8, make_float2(s2.y * 0.0625f, s2.y * z2.y));
      }
    };

    int j_w = d_lo, did_sparse = 0;
    Span cur, nxt;
    bool have = walk(j_w, did_sparse, cur);
    // weights' scales and zeros do not depend on the preceding kernel: their first
    // window is on its way before this warp waits for that kernel
    if (have) fetch_sz(cur);
    grid_dependency_wait();               // scale_x (read in the epilogue) is written by the preceding kernel
    // activation scales of this thread's output columns, fetched now so that the epilogue does not wait for them
    float sxv[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int tok = tok0 + nt * 8 + tig * 2 + h;
        sxv[nt][h] = (S == 1 && p.scale_x && tok < p.T) ? __half2float(ld_plain(p.scale_x + tok)) : 0.f;
      }
    // A wait that gives up clears `ok` for the whole warp; the loops still run to
    // their end (skipping the work) so that every barrier below is reached.
    while (have) {
      const bool have_next = walk(j_w, did_sparse, nxt);
      asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");   // previous span's window is free
      if (cur.dense) park_sz();
      if (have_next) fetch_sz(nxt);
      asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");

      if (cur.dense) {
        for (int j = cur.j0; j < cur.j1; ++j, ++consumed) {
          const int g = 2 * j;
          const bool two = g + 1 < p.ng;
          const int st = consumed % STAGES;
          if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&full[st], (consumed / STAGES) & 1, SITE_DEC_FULL));
          if (!ok) continue;
          const uint32_t slot = stage_a + st * STAGE_BYTES;
          const uint32_t wrow[2] = {slot + w_off, (slot + w_off) ^ GROUP_BYTES};     // row b: eight rows (1 KB) further on
          const uint32_t sums = sumx_a + st * 2 * SUMX_BYTES;
          // the wide instantiation (four MMA tiles per pass) reads a group's weight fragments when it gets to
          // the group: both groups' fragments at once do not fit its register budget
          constexpr bool LATE_W = NT > 2;
          uint4 wa[2], wb[2];
#pragma unroll
          for (int h = 0; h < (LATE_W ? 1 : 2); ++h) {
            wa[h] = lds_v4(wrow[h]);
            wb[h] = lds_v4(wrow[h] + 8 * 2 * GROUP_BYTES);
          }
          const float2 sza0 = lds_f2(szs_a + ((g & (SZ_CHUNK - 1)) * ROWS + r_a) * 8);
          const float2 szb0 = lds_f2(szs_a + ((g & (SZ_CHUNK - 1)) * ROWS + r_b) * 8);
          const float2 sza1 = lds_f2(szs_a + (((g + 1) & (SZ_CHUNK - 1)) * ROWS + r_a) * 8);
          const float2 szb1 = lds_f2(szs_a + (((g + 1) & (SZ_CHUNK - 1)) * ROWS + r_b) * 8);
          // group gg of the step, MMA tiles of tokens in bunches of NTH: A fragments are widened once per group
#pragma unroll
          for (int gg = 0; gg < 2; ++gg) {
            if (LATE_W && gg == 1) {
              wa[0] = lds_v4(wrow[1]);
              wb[0] = lds_v4(wrow[1] + 8 * 2 * GROUP_BYTES);
            }
            const AFrag fa = LATE_W ? unpack_a(wa[0], wb[0]) : unpack_a(wa[gg], wb[gg]);
            const float2 sza = gg ? sza1 : sza0, szb = gg ? szb1 : szb0;
#pragma unroll
            for (int hh = 0; hh < HALVES; ++hh) {
              uint4 q0[NTH], q1[NTH];
              float2 sx[NTH];
#pragma unroll
              for (int nt = 0; nt < NTH; ++nt) {
                const int xo = gg * X_TILE_BYTES + (hh * NTH + nt) * XNT;
                q0[nt] = lds_v4(slot + xo + xs0);
                q1[nt] = lds_v4(slot + xo + xs1);
                // sums slot: [16-token tile][group][16]; tokens of bunch hh lie in tile (hh * NTH * 8) / 16
                const int t_in = (hh * NTH + nt) * 8 + tig * 2;
                sx[nt] = (p.sumxf && (gg == 0 || two)) ? lds_f2(sums + (((t_in >> 4) * 2 + gg) * 16 + (t_in & 15)) * 4)
                                                      : make_float2(0.f, 0.f);
              }
              if (gg == 1 && hh == HALVES - 1) {
                // Hand the slot back - but only once the loads from it have RETURNED.  Issuing them first is
                // not enough: the arrival overtook shared-memory loads still in flight, the producer's next
                // copy then landed under them, and about one launch in ten of a long, two-CTAs-per-SM shape
                // folded one group with the group sums of four steps on (seen as 16-row x 16-token patches
                // off by a fraction of a step; found by matching the error against candidate operands).  The
                // arrival's address therefore depends on the last registers loaded from the slot (`dep & 0`
                // with a zero the compiler cannot see): it issues when they are ready, and a warp's earlier
                // shared-memory loads have returned by then.  (The slot's next writer is the copy engine - another
                // proxy - so a release by this thread orders nothing for it; fence.proxy.async before the
                // arrival also cures it and costs 4 % of the decode sweep, this costs 1.5 %.)
                const uint32_t dep = q1[NTH - 1].w ^ __float_as_uint(sx[NTH - 1].y);     // the loads issued last
                __syncwarp();
                if (lane == 0) mbar_arrive_after(&empty[st], dep, runtime_zero);
              }
              int acc[NTH][4];
              group_mma<NTH>(acc, fa, q0, q1);
              group_fold<NTH>(y + hh * NTH, acc, sza.x, szb.x, sza.y, szb.y, sx);
              if (DUMP && p.acc_dump) {
#pragma unroll
                for (int nt = 0; nt < NTH; ++nt)
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const int rl = (i & 2) ? r_b : r_a;
                    const int tok = tok0 + (hh * NTH + nt) * 8 + tig * 2 + (i & 1);
                    if (tok >= p.T || g + gg >= p.ng || row0 + rl >= p.N) continue;
                    // parity aid, not a hot path: every store is range-checked
                    const size_t idx = ((size_t)(g + gg) * p.N + row0 + rl) * p.T + tok;
                    if (idx < (size_t)p.ng * p.N * p.T) p.acc_dump[idx] = acc[nt][i] >> 4;
                    else record_error(SITE_DEC_DUMP, 1);
                  }
              }
            }
          }
        }
      } else {
        for (int blk = cur.j0; blk < cur.j1; ++blk, ++consumed) {
          const int g = ld_plain(p.hp_col_indices + blk);
          // a residual block's column is anywhere in the row: fetch the two scales directly
          float s_a = 0.f, s_b = 0.f;
          if (p.scale_u4) {
            if (row0 + r_a < p.N) s_a = __half2float(ld_plain(p.scale_u4 + (size_t)(row0 + r_a) * p.ng + g));
            if (row0 + r_b < p.N) s_b = __half2float(ld_plain(p.scale_u4 + (size_t)(row0 + r_b) * p.ng + g));
          }
          const int st = consumed % STAGES;
          if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&full[st], (consumed / STAGES) & 1, SITE_DEC_FULL));
          if (!ok) continue;
          const uint32_t slot = stage_a + st * STAGE_BYTES;
          const uint4 wa = lds_v4(slot + r_a * GROUP_BYTES + tig * 16);
          const uint4 wb = lds_v4(slot + r_b * GROUP_BYTES + tig * 16);
          const AFrag fa = unpack_a(wa, wb);
          const float w = 0.0625f * p.sparse_weight;
#pragma unroll
          for (int hh = 0; hh < HALVES; ++hh) {
            uint4 q0[NTH], q1[NTH];
            float2 sx[NTH];
#pragma unroll
            for (int nt = 0; nt < NTH; ++nt) {
              q0[nt] = lds_v4(slot + (hh * NTH + nt) * XNT + xs0);
              q1[nt] = lds_v4(slot + (hh * NTH + nt) * XNT + xs1);
              sx[nt] = make_float2(0.f, 0.f);
            }
            if (hh == HALVES - 1) {
              const uint32_t dep = q1[NTH - 1].w;                                       // as in the dense branch
              __syncwarp();
              if (lane == 0) mbar_arrive_after(&empty[st], dep, runtime_zero);
            }
            int acc[NTH][4];
            group_mma<NTH>(acc, fa, q0, q1);
            group_fold<NTH>(y + hh * NTH, acc, s_a * w, s_b * w, 0.f, 0.f, sx);
            if (DUMP && p.acc_hi_dump) {
#pragma unroll
              for (int nt = 0; nt < NTH; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const int rl = (i & 2) ? r_b : r_a;
                  const int tok = tok0 + (hh * NTH + nt) * 8 + tig * 2 + (i & 1);
                  if (tok >= p.T) continue;
                  const size_t idx = ((size_t)blk * BROW + rl) * p.T + tok;
                  if (blk >= 0 && blk < p.nnz && idx < (size_t)p.nnz * BROW * p.T) p.acc_hi_dump[idx] = acc[nt][i] >> 4;
                  else record_error(SITE_DEC_DUMP, 2);
                }
            }
          }
        }
      }

      cur = nxt;
      have = have_next;
    }
    if (!ok) misc[1] = 1;

    // ---------------------------------------------------------- block-row share done
    if (p.Y != nullptr && S == 1) {
      if (ok) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int row = row0 + ((i & 2) ? r_b : r_a);
            const int tok = tok0 + nt * 8 + tig * 2 + (i & 1);
            if (row < p.N && tok < p.T) {
              const float v = (i & 1) ? y[nt][i >> 1].y : y[nt][i >> 1].x;
              p.Y[(size_t)row * p.y_stride_n + (size_t)tok * p.y_stride_t] = __float2half_rn(v * sxv[nt][i & 1]);
            }
          }
      }
    } else if (p.Y != nullptr) {
      // park this CTA's 128 x 16 partial tile in its own shared memory (the ring is
      // drained: every copy that was issued has been consumed)
      asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_THREADS) : "memory");   // nobody still reads the last slot
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        sts_f2(stage_a + (r_a * TOK + nt * 8 + tig * 2) * 4, y[nt][0]);
        sts_f2(stage_a + (r_b * TOK + nt * 8 + tig * 2) * 4, y[nt][1]);
      }
    }
  }

  if (p.Y != nullptr && S > 1) {
    // Every thread of every CTA of the cluster reaches both barriers: no path
    // above returns early.  CTA k then owns rows [k*128/S, (k+1)*128/S) of the tile.
    __syncwarp();
    constexpr int NCOL = NT * 8;
    static_assert(THREADS % NCOL == 0, "a thread keeps one output column through the reduction loop");
    // the column's activation scale travels while the cluster gathers (most of the
    // producer warp has not passed the dependency wait, so it waits here: a no-op by now)
    const int col = tid % NCOL;
    if (warp == CONSUMER_WARPS) grid_dependency_wait();
    const float sxs = (p.scale_x && tok0 + col < p.T) ? __half2float(ld_plain(p.scale_x + tok0 + col)) : 0.f;
    cluster_sync_all();
    const float* red = reinterpret_cast<const float*>(stage_buf);
    const int rl_lo = rank * ROWS / S, rl_hi = (rank + 1) * ROWS / S;
    for (int i = tid; i < (rl_hi - rl_lo) * NCOL; i += THREADS) {
      const int rl = rl_lo + i / NCOL;
      const int row = row0 + rl, tok = tok0 + col;
      if (row >= p.N || tok >= p.T) continue;
      float v = 0.f;
#pragma unroll 8
      for (int c = 0; c < S; ++c) v += ld_dsmem_f32(red + rl * TOK + col, (uint32_t)c);
      p.Y[(size_t)row * p.y_stride_n + (size_t)tok * p.y_stride_t] = __float2half_rn(v * sxs);
    }
    cluster_sync_all();     // peers may not retire while their tiles are still being read
  }
}

}  // namespace dec
}  // namespace w4a4
