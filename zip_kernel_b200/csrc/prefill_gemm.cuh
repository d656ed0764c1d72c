// Kernel 2: tensor-core fused GEMM for many tokens (prefill), tcgen05 / TMEM.
// Replaces the reference's mma.sync m16n8k64 s4 kernels
// (cuda_kernel/csrc/fused_dense_sparse/fused_dense_sparse_mma_int4.cu:184-1190,
// dense_gemm/dense_gemm_mma_int4.cu:39-431, sparse_gemm/sparse_gemm_mma_int4.cu:25-253).
//
//   Y[n,t] = fp16( sx[t] * ( sum_g s[n,g] * (acc[g,n,t] - z[n,g] * sumX[t,g])
//                            + w * sum_{blk in block-row} s[n,bc] * acc_hi[blk,n,t] ) )
//
// sm_100a tensor cores have no 4-bit integer MMA, so nibbles are widened to s8 on
// the way: a CTA owns 128 weight rows (one block-row = MMA M) x TN tokens (MMA N).
// Per K-group of 128 (and per residual block of the block-row, which is just one
// more K-step):
//   * the producer warp issues two non-multicast asynchronous copies: the packed
//     weight tile (TMA, 128 x 64 bytes, 64-byte swizzle so that a thread can read
//     its whole row without bank conflicts) and the tokens' expanded codes (one
//     bulk copy of TN x 128 bytes: the expanded layout is group-major and
//     pre-swizzled, i.e. already the K-major operand layout tcgen05 reads);
//   * four unpack warps widen the weight tile (s8 lanes scaled by 16, three logic
//     ops per 8 codes, same element permutation as the activations) and store it
//     straight into TENSOR MEMORY with tcgen05.st: thread = weight row = TMEM
//     lane, 32 columns of four s8 each.  The MMA takes its A operand from there,
//     so the widened weights never touch shared memory: per K-step shared memory
//     carries 24 KB of copies, 8 KB of unpack reads and 16 KB of B-operand reads
//     instead of 96 KB, and shared-memory bandwidth is what a 128 x 128 tile
//     runs out of first;
//   * one thread issues four tcgen05.mma kind::i8 (K = 32 each, A from TMEM, B
//     from shared memory) into a fresh int32 accumulator in TMEM (two accumulator
//     buffers alternate).  It waits on ONE "ready" mbarrier per step, on which the
//     activation copy, the unpack warps and the fold warps (accumulator buffer
//     folded) all arrive, and commits ONCE to a ring of "step done" mbarriers that
//     the fold warps (accumulator ready), the unpack warps (A buffer free again)
//     and the producer (activation slot free again) wait on: its loop is a chain
//     of dependent instructions of a single thread that competes for issue slots
//     with twelve busy warps, so it is kept as short as it can be;
//   * eight fold warps read the accumulator with tcgen05.ld and fold it in fp32:
//     y += acc * (s/16), keeping y (128 x TN fp32) in registers as packed pairs;
//   * the zero-point term  Z[n,t] = sum_g (s*z)[n,g] * sumX[t,g]  is a small GEMM of
//     its own and runs on the tensor core too: per window of 16 groups the fold
//     warps lay out (s*z) - exact in fp32, split into two 11-bit halves - and the
//     tokens' group sums (below 2^11) as tf32 operand tiles, the MMA thread issues
//     four tcgen05.mma kind::tf32 into a third, fp32 accumulator, and the epilogue
//     subtracts it once.  The conversions and FMAs of the fold issue at half rate
//     on this part and saturate the SM's schedulers long before the tensor pipe is
//     busy, so every operation taken out of the per-group fold counts.
// Epilogue: y * scale_x -> fp16 -> Y.  Every mbarrier wait is bounded; a wait
// that gives up records an error, all roles fall through to the common exit and
// the TMEM allocation is released.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace w4a4 {
namespace pre {

constexpr int ROWS = 128;                 // MMA M
constexpr int TN = 128;                   // tokens per CTA = MMA N
constexpr int A_BUFS = 2;                 // widened weight tiles in flight (the paired kernel, and the e4m3 tiles in shared memory)
#ifndef W4A4_A_BUFS_TMEM
#define W4A4_A_BUFS_TMEM 4
#endif
// Widened s8 tiles in tensor memory (integer instantiation).  A tile is free again only once the MMAs that read
// it have COMPLETED - hundreds of clocks after they were issued while the fold warps keep the SM busy - so
// with two tiles the unpack warps and the tensor pipe took turns: four tiles let the unpack warps run ahead.
constexpr int A_BUFS_TMEM = W4A4_A_BUFS_TMEM;
constexpr int X_BYTES = TN * BCOL;                // 16384
constexpr int MAX_STAGES = 6;
constexpr int SZ_CHUNK = 16;                      // groups of scale/zero/sums staged at a time
constexpr int A_COLS = BCOL / 4;                  // 32 TMEM columns hold one widened row of 128 s8
constexpr int TMEM_COLS = 512;                    // the whole tensor memory of the SM (one CTA per SM)
// Tensor-memory columns.  Accumulator buffers first (the MMAs run that many steps ahead of the fold), then
// the widened weight tiles (integer instantiation only), then the fp32 accumulator of the zero-point term.
// The fp8 instantiations read A from shared memory and have room for a third accumulator buffer.
template <bool A_TMEM>
struct TmemLayout {
  static constexpr int ACC_BUFS = A_TMEM ? 2 : 3;
  static constexpr int A_COL0 = ACC_BUFS * TN;
  static constexpr int Z_COL0 = A_COL0 + (A_TMEM ? A_BUFS_TMEM * A_COLS : 0);
  static_assert(Z_COL0 + TN <= TMEM_COLS, "tensor memory capacity");
};
constexpr int ZT_BYTES = ROWS * 128;              // one tf32 operand tile of the zero-point term: 128 rows x 32 values

#ifndef W4A4_FOLD_WARPS
#define W4A4_FOLD_WARPS 8
#endif
constexpr int WARP_TMA = 0, WARP_MMA = 1, WARP_UNPACK0 = 2, N_UNPACK_WARPS = 4, WARP_FOLD0 = 6;
constexpr int N_FOLD_WARPS = W4A4_FOLD_WARPS;     // a multiple of 4: a warp reads only its quarter of the TMEM lanes
constexpr int WARP_TMAX = WARP_FOLD0 + N_FOLD_WARPS;   // the activation copies have an issuing thread of their own
constexpr int WARP_MMA2 = WARP_TMAX + 1;               // ... and the odd steps' MMAs too
constexpr int THREADS = (WARP_MMA2 + 1) * 32;
static_assert(A_BUFS % 2 == 0 && A_BUFS_TMEM % 2 == 0, "an issuing thread takes every other step");
constexpr int FOLD_THREADS = N_FOLD_WARPS * 32;
constexpr int COLS_PER_FOLD = TN / (N_FOLD_WARPS / 4);   // a fold thread owns one row and this many tokens
static_assert(N_FOLD_WARPS % 4 == 0 && COLS_PER_FOLD % 32 == 0, "fold warps tile the accumulator in 32-lane x 32-column pieces");

enum : int {
  SITE_PRE_WEMPTY = 16, SITE_PRE_WFULL, SITE_PRE_AEMPTY, SITE_PRE_AFULL, SITE_PRE_XEMPTY, SITE_PRE_XFULL,
  SITE_PRE_ACCEMPTY, SITE_PRE_ACCFULL, SITE_PRE_DUMP
};

struct Params {
  const int* hp_row_offsets;
  const int* hp_col_indices;
  const int8_t* XE;         // expanded activation codes, group-major [ng][t_pad][128]
  int t_pad;
  const __half* scale_u4;   // (N, ng)
  const __half* zero_u4;    // (N, ng) or nullptr
  const float* sumxf;       // [ceil(T/16)][ng][16] or nullptr
  const __half* scale_x;    // (T)
  __half* Y;
  long long y_stride_n, y_stride_t;
  int* acc_dump;            // optional (ng, N, T) int32
  int* acc_hi_dump;         // optional (nnz, 128, T) int32
  int T, K, N, ng, nnz;
  int nd;                   // dense K-steps (ng, or 0 when the dense part is off)
  int sparse_on;
  int sz_vec;
  int band;                 // token tiles per band of the CTA order (>= 1)
  float sparse_weight;
#ifdef W4A4_TRACE
  long long* trace;         // [16 events][64 steps] clock stamps of one CTA
  int trace_cta;
#endif
};
#ifdef W4A4_TRACE
#define TRACE(ev, n) do { if (lin == p.trace_cta && (n) < 64) p.trace[(ev) * 64 + (n)] = clock64(); } while (0)
#else
#define TRACE(ev, n) do { } while (0)
#endif

inline bool supported(int T, int K, int N) { return T >= 1 && K >= 128 && N >= 1; }

// Three instantiations.  <F8 = false, PREP = false>: packed nibbles are copied in (8 KB per step), widened to
// s8 on the SM, integer MMAs (kind::i8) - for activation codes the caller expanded as s8, and for calls
// without activation group sums.  <F8 = true, PREP = false>: the same packed copies and the same three logic
// operations per 8 codes, but the bytes the unpack warps write are read as e4m3 numbers: a nibble with bit 3
// flipped, alone in its byte, is the e4m3 value (code + 8) * 2^-9 (nib_lo_off8), the activation codes are
// e4m3 integers in the same even/odd order, and the MMA is kind::f8f6f4 with fp32 accumulators that hold
// 2^-9 * (acc + 8 * sumX) exactly.  The fold then needs no int -> float conversion - the instruction that
// bounds the integer instantiation - and the offset 8 * sumX leaves with the zero-point term, which already
// is a product with sumX on the tensor core (dense groups), or with one extra FMA per element (the few
// residual steps).  <F8 = true, PREP = true>: the caller supplies weights prepared once as e4m3 bytes (16 KB
// per step, the A operand as it lands): no unpack work either.
template <bool F8, bool PREP>
struct SmemLayout {
  static constexpr bool OFF8 = F8 && !PREP;                   // packed weights widened into e4m3 operand tiles in shared memory
  static constexpr int W_STAGES = PREP ? 5 : (F8 ? 4 : 6);    // weight tiles in flight
  static constexpr int X_STAGES = PREP ? 5 : (F8 ? 5 : 6);    // activation tiles in flight = depth of the "ready" / "step done" rings
  static constexpr int WP_BYTES = PREP ? ROWS * BCOL : ROWS * GROUP_BYTES;
  static constexpr int AT_BYTES = ROWS * BCOL;                // one widened weight tile as an MMA operand
  static_assert(!PREP || W_STAGES == X_STAGES, "with prepared weights both copies of a step share a ring slot index");
  static constexpr size_t wp = 0;
  static constexpr size_t x = wp + (size_t)W_STAGES * WP_BYTES;
  static constexpr size_t at = x + (size_t)X_STAGES * X_BYTES;                  // e4m3 [A_BUFS][128 rows][128]: widened weights (K-major, swizzled)
  static constexpr size_t sz = at + (size_t)(OFF8 ? A_BUFS * AT_BYTES : 0);     // float [SZ_CHUNK][128]: scale (/16 for int8 accumulators)
  static constexpr size_t zb = sz + (size_t)SZ_CHUNK * ROWS * 4;                // tf32 [2][TN tokens][32]: group sums, twice (K-major, swizzled)
  static constexpr size_t za = zb + (size_t)2 * ZT_BYTES;                       // tf32 [128 rows][32]: high and low half of scale * zero
  static constexpr size_t za2 = za + (size_t)ZT_BYTES;                          // tf32 [128 rows][32]: 8 * scale in the first 16 values
  static constexpr size_t raw = za2 + (size_t)(OFF8 ? ZT_BYTES : 0);            // 2 x 16 bytes per (row, half): fp16 scales, zeros
  static constexpr size_t sxs = raw + (size_t)2 * ROWS * 32;                    // float  [TN]
  static constexpr size_t bars = sxs + (size_t)TN * 4;
  static constexpr size_t total = bars + 256;
  static_assert(1024 + total <= 232448, "shared memory of one SM");
};
inline size_t smem_bytes(bool f8, bool prep) {
  return 1024 + (prep ? SmemLayout<true, true>::total : f8 ? SmemLayout<true, false>::total : SmemLayout<false, false>::total);
}

// ---------------------------------------------------------------- tcgen05 wrappers
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// K-major operand tile of 128-byte rows under the 128-byte swizzle: 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(const void* tile) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);        // start address, 16-byte units
  d |= (uint64_t)1 << 16;                                  // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;                        // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                                  // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                                  // SWIZZLE_128B
  return d;
}
// kind::i8, s8 x s8 -> s32, both operands K-major, M = 128, N = TN
constexpr uint32_t IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
// kind::f8f6f4, e4m3 x e4m3 -> f32, both operands K-major in shared memory, M = 128, N = TN (K = 32 per instruction)
constexpr uint32_t IDESC_F8 = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(IDESC_F8), "r"(accumulate)
      : "memory");
}
// kind::tf32, tf32 x tf32 -> f32, both operands K-major, M = 128, N = TN (K = 8 per instruction)
constexpr uint32_t IDESC_TF32 = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(IDESC_TF32), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(IDESC), "r"(accumulate)
      : "memory");
}
// the same with the A operand in tensor memory (row = lane, four s8 per 32-bit column)
__device__ __forceinline__ void umma_i8_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(IDESC), "r"(accumulate)
      : "memory");
}
// 32 consecutive 32-bit columns of the calling thread's TMEM lane
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,"
      "%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Sum of the 128 integer-valued e4m3 codes of one (group, token) line of the expanded activations (parity dump only).
__device__ __forceinline__ int e4m3_line_sum(const int8_t* line) {
  int s = 0;
  for (int i = 0; i < BCOL; ++i) {
    const uint32_t b = (uint8_t)line[i], e = (b >> 3) & 15u, m = b & 7u;
    const int mag = e == 0 ? 0 : (int)(((8u | m) << e) >> 10);
    s += (b & 0x80u) ? -mag : mag;
  }
  return s;
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

template <bool DUMP, bool F8, bool PREP>
__global__ void __launch_bounds__(THREADS, 1)
prefill_gemm_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_wh,
                    const Params p) {
  static_assert(F8 || !PREP, "prepared weights are e4m3 bytes");
  using SmemLayout = pre::SmemLayout<F8, PREP>;
  constexpr int W_STAGES = SmemLayout::W_STAGES, X_STAGES = SmemLayout::X_STAGES, WP_BYTES = SmemLayout::WP_BYTES;
  constexpr int ACC_BUFS = TmemLayout<!F8>::ACC_BUFS, A_COL0 = TmemLayout<!F8>::A_COL0, Z_COL0 = TmemLayout<!F8>::Z_COL0;
  constexpr int AT_BYTES = SmemLayout::AT_BYTES;
  constexpr int N_A = F8 ? A_BUFS : A_BUFS_TMEM;           // widened weight tiles in flight
  static_assert(N_A < X_STAGES, "the completion barrier of the step a tile was last read in must not have been reused");
  static_assert(ACC_BUFS < X_STAGES, "the fold warps' arrival for step n + ACC_BUFS must fall into that step's barrier phase");
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* wp_ring = sm + SmemLayout::wp;
  unsigned char* x_ring = sm + SmemLayout::x;
  float* szs = reinterpret_cast<float*>(sm + SmemLayout::sz);
  unsigned char* zb_tiles = sm + SmemLayout::zb;
  unsigned char* za_tile = sm + SmemLayout::za;
  unsigned char* za2_tile = sm + SmemLayout::za2;
  unsigned char* a_tiles = sm + SmemLayout::at;
  // packed nibbles read as e4m3 numbers: accumulators carry the offset 8 * sumX and the unit 2^-9
  constexpr bool OFF8 = F8 && !PREP;
  float* sxs = reinterpret_cast<float*>(sm + SmemLayout::sxs);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + SmemLayout::bars);
  uint64_t* w_full = bars;                      // [W_STAGES]
  uint64_t* w_empty = w_full + W_STAGES;        // [W_STAGES]
  // ready[n % X_STAGES]: everything step n's MMAs need is in place - the activation tile has landed (1
  // arrival + its bytes), the widened weights are in tensor memory (one arrival per unpack warp) and the
  // accumulator buffer has been folded (one arrival per fold warp).  The issuing thread is a single
  // thread competing for issue slots with twelve busy warps: one wait per step instead of three.
  uint64_t* ready = w_empty + W_STAGES;         // [X_STAGES]
  uint64_t* done = ready + X_STAGES;            // [X_STAGES] the MMAs of step n (slot n % X_STAGES) have completed
  uint64_t* z_full = done + X_STAGES;           // operand tiles of a window's zero-point term are in shared memory
  uint64_t* z_done = z_full + 1;                // ... and its MMAs have completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(z_done + 1);

  grid_launch_dependents();
  const int tid = threadIdx.x;
#ifdef W4A4_TRACE
  const long long t_start = clock64();
#endif
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // CTAs are dispatched in the order of their linear index.  Bands of `band` token tiles are walked
  // token tile first, so the CTAs resident at one time cover a compact patch of (block-rows x token
  // tiles) whose weight and activation tiles stay in L2 while they are shared.
  const int lin = blockIdx.x + blockIdx.y * gridDim.x;
  const int per_band = gridDim.x * p.band;
  const int band_i = lin / per_band, band_rem = lin - band_i * per_band;
  const int band_h = min(p.band, (int)gridDim.y - band_i * p.band);
  const int r = band_rem / band_h;              // block-row
  const int row0 = r * ROWS;
  const int tok0 = (band_i * p.band + band_rem % band_h) * TN;

  if (tid == 0) {
    for (int i = 0; i < W_STAGES; ++i) { mbar_init(&w_full[i], 1); mbar_init(&w_empty[i], N_UNPACK_WARPS); }
    // arrivals per step: the activation copy, then either the four unpack warps or the weight copy, then the fold warps
    for (int i = 0; i < X_STAGES; ++i) { mbar_init(&ready[i], (PREP ? 2 : 1 + N_UNPACK_WARPS) + N_FOLD_WARPS); mbar_init(&done[i], 1); }
    mbar_init(z_full, N_FOLD_WARPS);
    mbar_init(z_done, 1);
    mbar_fence_init();
    tma_prefetch_desc(&tm_w);
    tma_prefetch_desc(&tm_wh);
  }
  if (warp == WARP_MMA) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // K-steps of this CTA: the dense groups, then the residual blocks of the block-row
  int b_lo = 0, b_hi = 0;
  if (p.sparse_on) {
    b_lo = ld_plain(p.hp_row_offsets + r);
    b_hi = ld_plain(p.hp_row_offsets + r + 1);
  }
  const int n_steps = p.nd + (b_hi - b_lo);
  const int n_windows = (p.nd + SZ_CHUNK - 1) / SZ_CHUNK;     // zero-point term: one small tf32 MMA batch per window of 16 groups

  if (warp == WARP_TMA) {
    // ------------------------------------------------------------ weight copies
    // One thread's wait / expect / copy sequence takes 300-400 clk in this kernel (a lone thread among polling
    // warps), more than the MMAs of a step: weights and activations each have an issuing thread of their own.
    if (lane == 0) {
      bool ok = true;
      int ws = 0;
      uint32_t wph = 1;
      for (int n = 0; n < n_steps && ok; ++n) {
        if (n >= W_STAGES) {
          // packed tiles are released by the unpack warps, prepared tiles by the completion of the MMAs that read them
          ok = PREP ? mbar_wait(&done[ws], wph, SITE_PRE_WEMPTY) : mbar_wait(&w_empty[ws], wph, SITE_PRE_WEMPTY);
          if (!ok) break;
        }
        // prepared weights are the A operand as it is: the copy reports to the step's readiness barrier
        uint64_t* bar = PREP ? &ready[ws] : &w_full[ws];
        mbar_arrive_expect_tx(bar, WP_BYTES);
        if (n < p.nd) tma_load_2d(wp_ring + ws * WP_BYTES, &tm_w, n * (PREP ? BCOL : GROUP_BYTES), row0, bar);
        else          tma_load_2d(wp_ring + ws * WP_BYTES, &tm_wh, 0, (b_lo + n - p.nd) * BROW, bar);
        TRACE(0, n);
        if (++ws == W_STAGES) { ws = 0; wph ^= 1; }
      }
    }
  } else if (warp == WARP_TMAX) {
    // ------------------------------------------------------------ activation copies
    if (lane == 0) {
      bool ok = true;
      int xs = 0;
      uint32_t xph = 1;
      grid_dependency_wait_for_async_reads();                 // the expanded codes are written by the preceding kernel
      const int8_t* src0 = p.XE + (size_t)tok0 * BCOL;
      const size_t gstride = (size_t)p.t_pad * BCOL;
      for (int n = 0; n < n_steps && ok; ++n) {
        // the slot is free once the MMAs of step n - X_STAGES have completed
        if (n >= X_STAGES) ok = mbar_wait(&done[xs], xph, SITE_PRE_XEMPTY);
        if (!ok) break;
        const int g = n < p.nd ? n : ld_plain(p.hp_col_indices + b_lo + n - p.nd);
        mbar_arrive_expect_tx(&ready[xs], X_BYTES);
        // TN consecutive tokens of one group: contiguous and already in operand layout
        bulk_load_1d(x_ring + xs * X_BYTES, src0 + g * gstride, X_BYTES, &ready[xs]);
        TRACE(1, n);
        if (++xs == X_STAGES) { xs = 0; xph ^= 1; }
      }
    }
  } else if (warp == WARP_MMA || warp == WARP_MMA2) {
    // ------------------------------------------------------------ MMA issuers
    // Two issuing threads take the even and the odd steps.  An issuing thread is stalled while the tensor
    // pipe's queue is full and then needs 200-300 clk for its own loop (a lone thread among polling warps):
    // with one thread the pipe drained in between.  Steps are independent of one another - each has an
    // accumulator buffer, operand slots and a completion barrier of its own - so their MMAs need no order.
    if (lane == 0) {
      bool ok = true;
      const int par = warp == WARP_MMA ? 0 : 1;
      int xs = par % X_STAGES;
      uint32_t xph = 0;
      int z_next = 0;
      // Z[n, t] += sum over the window's 16 groups of (scale * zero)[n, g] * sumX[t, g]: both factors
      // as tf32 (the product of two fp16 values split into two 11-bit halves; sums below 2^11 are
      // exact), four MMAs of K = 8 over the 32 values of an operand row
      auto issue_zero_term = [&](int k) {
        bool zok = mbar_wait_relaxed(z_full, k & 1, SITE_PRE_AFULL);
        if (!zok) return false;
        tc_fence_after();
        const uint64_t za_desc = smem_desc_sw128(za_tile);
        const uint64_t zb_desc = smem_desc_sw128(zb_tiles + (k & 1) * ZT_BYTES);
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_tf32(tmem_base + Z_COL0, za_desc + j * 2, zb_desc + j * 2, (k > 0 || j > 0) ? 1u : 0u);
        if (OFF8) {
          // + sum over the window of (8 * scale)[n, g] * sumX[t, g]: the offset of the weights' e4m3 form
          const uint64_t za2_desc = smem_desc_sw128(za2_tile);
#pragma unroll
          for (int j = 0; j < 2; ++j) umma_tf32(tmem_base + Z_COL0, za2_desc + j * 2, zb_desc + j * 2, 1u);
        }
        umma_commit(z_done);
        return true;
      };
      int buf = par % ACC_BUFS;
      int ab = par;                   // widened weight tile of the step: step % N_A
      const uint64_t bdesc0 = smem_desc_sw128(x_ring), adesc0 = smem_desc_sw128(wp_ring), atdesc0 = smem_desc_sw128(a_tiles);
      const uint32_t d0 = tmem_base, a0 = tmem_base + A_COL0;
      const bool with_z = p.Y != nullptr && n_windows > 0;
      int z_due = ACC_BUFS;          // step at which the next window's zero-point MMAs are issued
      for (int n = par; n < n_steps && ok; n += 2) {
        // a window's tiles are ready once the fold warps have passed its boundary, which they
        // have when they return the accumulator of the window's first step (the even thread issues them)
        if (par == 0 && with_z && n >= z_due && z_next < n_windows) {
          ok = issue_zero_term(z_next++);
          z_due += SZ_CHUNK;
          if (!ok) break;
        }
        if (!(PREP ? mbar_wait_relaxed(&ready[xs], xph, SITE_PRE_XFULL) : mbar_wait(&ready[xs], xph, SITE_PRE_XFULL))) { ok = false; break; }
        tc_fence_after();
        TRACE(2, n);
        const uint64_t bdesc = bdesc0 + (uint64_t)(xs * (X_BYTES >> 4));
        const uint32_t d = d0 + buf * TN, a = a0 + ab * A_COLS;
        if (PREP) {
          const uint64_t adesc = adesc0 + (uint64_t)(xs * (WP_BYTES >> 4));
          umma_f8(d, adesc, bdesc, 0);                 // K = 32 each: 32 bytes of A and of B
          umma_f8(d, adesc + 2, bdesc + 2, 1);
          umma_f8(d, adesc + 4, bdesc + 4, 1);
          umma_f8(d, adesc + 6, bdesc + 6, 1);
        } else if (F8) {
          const uint64_t adesc = atdesc0 + (uint64_t)(ab * (AT_BYTES >> 4));
          umma_f8(d, adesc, bdesc, 0);
          umma_f8(d, adesc + 2, bdesc + 2, 1);
          umma_f8(d, adesc + 4, bdesc + 4, 1);
          umma_f8(d, adesc + 6, bdesc + 6, 1);
        } else {
          umma_i8_ta(d, a, bdesc, 0);
          umma_i8_ta(d, a + 8, bdesc + 2, 1);
          umma_i8_ta(d, a + 16, bdesc + 4, 1);
          umma_i8_ta(d, a + 24, bdesc + 6, 1);
        }
        umma_commit(&done[xs]);
        TRACE(3, n);
        xs += 2;
        if (xs >= X_STAGES) { xs -= X_STAGES; xph ^= 1; }
        buf += 2;
        if (buf >= ACC_BUFS) buf -= ACC_BUFS;
        ab += 2;
        if (ab >= N_A) ab -= N_A;
      }
      while (par == 0 && ok && p.Y != nullptr && z_next < n_windows) ok = issue_zero_term(z_next++);
    }
  } else if (warp < WARP_FOLD0) {
    // ------------------------------------------------------------ unpack warps
    // thread = weight row = TMEM lane: warp w may touch lanes 32 * (w % 4) .. + 31
    const int urow = (warp & 3) * 32 + lane;
    const uint32_t wp_a = smem_u32(wp_ring);
    const uint32_t a_lane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + A_COL0;
    bool ok = true;
    int ws = 0;
    uint32_t wph = 0;
    for (int n = 0; n < (PREP ? 0 : n_steps); ++n) {     // prepared weights need no widening
      const int buf = n % N_A;
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait_relaxed(&w_full[ws], wph, SITE_PRE_WFULL));
      if (warp == WARP_UNPACK0 && lane == 0) TRACE(6, n);
      // the A buffer was last read by the MMAs of step n - 2
      if (ok && n >= N_A)
        ok = __all_sync(0xffffffffu, mbar_wait_relaxed(&done[(n - N_A) % X_STAGES], ((n - N_A) / X_STAGES) & 1, SITE_PRE_AEMPTY));
      if (ok) {
        tc_fence_after();
        // the row's 64 packed bytes: four 16-byte chunks, stored at chunk ^ ((row >> 1) & 3) by the 64-byte swizzle
        const uint32_t src = wp_a + ws * WP_BYTES + urow * GROUP_BYTES;
        uint4 w[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) w[c] = lds_v4(src + ((c ^ ((urow >> 1) & 3)) << 4));
        uint32_t v[32];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint32_t q[4] = {w[c].x, w[c].y, w[c].z, w[c].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (F8) {
              v[(c * 4 + e) * 2] = nib_lo_off8(q[e]);                                 // even codes + 8, then odd ones + 8
              v[(c * 4 + e) * 2 + 1] = nib_hi_off8(q[e]);
            } else {
              v[(c * 4 + e) * 2] = nib_lo_x16(q[e]);                                  // even codes, then odd ones
              v[(c * 4 + e) * 2 + 1] = nib_hi_x16(q[e]);
            }
          }
        }
        if (F8) {
          // the widened row as an fp8 MMA operand row: 16-byte chunk c at c ^ (row & 7) (128-byte swizzle)
          const uint32_t dst = smem_u32(a_tiles) + buf * AT_BYTES + urow * BCOL;
#pragma unroll
          for (int c = 0; c < 8; ++c)
            sts_v4(dst + ((c ^ (urow & 7)) << 4), make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]));
          fence_proxy_async_smem();                  // this thread's row -> visible to the tensor core
        } else {
          tmem_st32(a_lane + buf * A_COLS, v);
          tc_fence_before();
        }
      }
      __syncwarp();
      if (ok && lane == 0) {
        mbar_arrive(&w_empty[ws]);
        mbar_arrive(&ready[n % X_STAGES]);
      }
      if (warp == WARP_UNPACK0 && lane == 0) TRACE(7, n);
      if (++ws == W_STAGES) { ws = 0; wph ^= 1; }
    }
  } else {
    // ------------------------------------------------------------ fold warps
    const int ft = tid - WARP_FOLD0 * 32;        // 0..255
    const int quarter = warp & 3;                // TMEM lanes this warp may read: 32*quarter .. +31
    const int chalf = (warp - WARP_FOLD0) >> 2;  // which share of the tokens
    const int rl = quarter * 32 + lane;          // local row
    const int row = row0 + rl;
    const int c0 = chalf * COLS_PER_FOLD;
    const uint32_t szs_a = smem_u32(szs), zb_a = smem_u32(zb_tiles), za_a = smem_u32(za_tile), za2_a = smem_u32(za2_tile);
    // scale factor of an accumulator: 1/16 undoes the s8 widening, 512 the unit of the e4m3 bytes
    constexpr float ACC_UNIT = OFF8 ? 512.f : (F8 ? 1.f : 0.0625f);
    grid_dependency_wait();
    for (int i = ft; i < TN; i += FOLD_THREADS)
      sxs[i] = (tok0 + i < p.T && p.scale_x) ? __half2float(ld_plain(p.scale_x + tok0 + i)) : 0.f;
    asm volatile("bar.sync 1, %0;" ::"n"(FOLD_THREADS) : "memory");

    // The thread's row x COLS_PER_FOLD tokens.  On prepared weights the accumulators arrive as floats in single
    // registers and the fold is one scalar FMA per element: pairing them up for fma.rn.f32x2 costs two register
    // moves per pair, as many issue slots as the FMAs (measured: -15 % kernel time without them).  The
    // integer instantiation converts two accumulators at a time into a register pair anyway and keeps the
    // packed FMAs (scalar ones: +6 %).
    constexpr bool SCALAR_FOLD = PREP;
    float yf[SCALAR_FOLD ? COLS_PER_FOLD : 1];
    f32x2_t y2[SCALAR_FOLD ? 1 : COLS_PER_FOLD / 2];      // two tokens per register pair
    if (SCALAR_FOLD) {
#pragma unroll
      for (int i = 0; i < COLS_PER_FOLD; ++i) yf[i] = 0.f;
    } else {
#pragma unroll
      for (int i = 0; i < COLS_PER_FOLD / 2; ++i) y2[i] = 0ull;
    }

    // Scale/zero/sums windows of 16 groups.  The next window travels as cp.async
    // copies while the current one is folded, so it occupies no registers: thread ft
    // copies the fp16 scales and zeros of 8 groups of row ft/2 into a staging slot of
    // its own, and 4-byte pieces of the tokens' group sums straight into the other
    // half of the double-buffered sums table.  At the window boundary each thread
    // turns its slot into (scale/16, scale*zero) pairs of the shared table.
    const int lrow = ft >> 1, lhalf = ft & 1;
    constexpr int SUMS_PER_THREAD = SZ_CHUNK * TN / FOLD_THREADS;
    const uint32_t raw_a = smem_u32(sm + SmemLayout::raw) + ft * 32;
    auto issue_window = [&](int gwin, int sel) {
#pragma unroll
      for (int k = 0; k < SUMS_PER_THREAD; ++k) {
        const int i = ft + k * FOLD_THREADS;
        const int gl = i / TN, t = i - gl * TN;
        const int g = gwin + gl, tok = tok0 + t;
        // operand row = token, value gl and again gl + 16 (for the low half of scale * zero); 16-byte chunks swizzled by row
        const uint32_t rowa = zb_a + sel * ZT_BYTES + t * 128 + (gl & 3) * 4;
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
      if (ft < 2 * ROWS) {
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
      if (ft >= 2 * ROWS) return;
      const uint4 ps = lds_v4(raw_a), pz = lds_v4(raw_a + 16);
      const __half2* hs = reinterpret_cast<const __half2*>(&ps);
      const __half2* hz = reinterpret_cast<const __half2*>(&pz);
      float chi[8], clo[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 s2 = __half22float2(hs[i]), z2 = __half22float2(hz[i]);
        // int8 path: the accumulators carry the factor 16 of the widened nibbles
        sts_f1(szs_a + ((lhalf * 8 + 2 * i) * ROWS + lrow) * 4, s2.x * ACC_UNIT);
        sts_f1(szs_a + ((lhalf * 8 + 2 * i + 1) * ROWS + lrow) * 4, s2.y * ACC_UNIT);
        // scale * zero is exact in fp32 (two 11-bit significands); its upper 11 bits and the exact rest are both tf32 values
        const float c0_ = s2.x * z2.x, c1_ = s2.y * z2.y;
        chi[2 * i] = __uint_as_float(__float_as_uint(c0_) & 0xFFFFE000u);
        chi[2 * i + 1] = __uint_as_float(__float_as_uint(c1_) & 0xFFFFE000u);
        clo[2 * i] = c0_ - chi[2 * i];
        clo[2 * i + 1] = c1_ - chi[2 * i + 1];
      }
      if (OFF8) {
        // 8 * scale, exact: values lhalf * 8 .. + 7 of the row (the MMAs read the first 16 values only)
        const uint32_t rowb = za2_a + lrow * 128;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const float2 sa = __half22float2(hs[2 * q]), sb = __half22float2(hs[2 * q + 1]);
          sts_v4(rowb + (((lhalf * 2 + q) ^ (lrow & 7)) << 4),
                 make_uint4(__float_as_uint(8.f * sa.x), __float_as_uint(8.f * sa.y), __float_as_uint(8.f * sb.x), __float_as_uint(8.f * sb.y)));
        }
      }
      // operand row = weight row: values lhalf * 8 .. + 7 (upper halves) and 16 + lhalf * 8 .. (rests)
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
      for (int i = 0; i < ACC_BUFS && i < n_steps; ++i) mbar_arrive(&ready[i % X_STAGES]);
    for (int n = 0; n < n_steps; ++n) {
      const bool is_dense = n < p.nd;
      if (is_dense && (n % SZ_CHUNK) == 0) {
        const int k = n / SZ_CHUNK;
        cp_async_wait_all();                                                // this thread's pieces of the window have landed
        // the previous window's zero-point MMAs read the weight-side tile and the sums tile that is refilled next
        if (ok && k > 0 && p.Y != nullptr) ok = __all_sync(0xffffffffu, mbar_wait(z_done, (k - 1) & 1, SITE_PRE_AEMPTY));
        asm volatile("bar.sync 1, %0;" ::"n"(FOLD_THREADS) : "memory");   // previous window no longer read
        park_window();
        fence_proxy_async_smem();                                           // this thread's tile pieces -> visible to the tensor core
        if (n + SZ_CHUNK < p.nd) issue_window(n + SZ_CHUNK, (k + 1) & 1);
        asm volatile("bar.sync 1, %0;" ::"n"(FOLD_THREADS) : "memory");   // table of this window visible to all
        if (lane == 0) mbar_arrive(z_full);
      }
      float f = 0.f;
      int blk = 0, gcol = n;
      if (is_dense) {
        f = lds_f1(szs_a + ((n % SZ_CHUNK) * ROWS + rl) * 4);
      } else {
        blk = b_lo + n - p.nd;
        gcol = ld_plain(p.hp_col_indices + blk);
        if (p.scale_u4 && row < p.N)
          f = __half2float(ld_plain(p.scale_u4 + (size_t)row * p.ng + gcol)) * ACC_UNIT * p.sparse_weight;
      }
      const int buf = n % ACC_BUFS;
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&done[n % X_STAGES], (n / X_STAGES) & 1, SITE_PRE_ACCFULL));
      if (!ok) continue;
      tc_fence_after();
      if (ft == 0) TRACE(4, n);
      const f32x2_t f2 = pack_f32x2(f, f);
#pragma unroll
      for (int cc = 0; cc < COLS_PER_FOLD; cc += 32) {
        uint32_t a[32];
        tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * TN + c0 + cc, a);
        // y += acc * (scale / 16): the zero-point term is accumulated by the tensor core (see the MMA thread)
#pragma unroll
        if (OFF8 && (!is_dense || DUMP)) {
          // A residual step is outside the zero-point windows: take its offset 8 * sumX out here, exactly
          // (accumulator and sum are small multiples of 2^-9).  The parity dump does the same on every step.
          const int tile0 = (tok0 + c0 + cc) >> 4, n_tiles = (p.T + 15) >> 4;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (tile0 + h >= n_tiles || gcol >= p.ng) continue;
            float sv[16];
            if (p.sumxf != nullptr) {
              const float4* line = reinterpret_cast<const float4*>(p.sumxf + ((size_t)(tile0 + h) * p.ng + gcol) * 16);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float4 s4 = ld_plain(line + q);
                sv[q * 4] = s4.x; sv[q * 4 + 1] = s4.y; sv[q * 4 + 2] = s4.z; sv[q * 4 + 3] = s4.w;
              }
            } else {
              // only a dump launch comes without the sums: add up the group's codes (any order)
#pragma unroll 1
              for (int e = 0; e < 16; ++e) sv[e] = (float)e4m3_line_sum(p.XE + ((size_t)gcol * p.t_pad + (tile0 + h) * 16 + e) * BCOL);
            }
#pragma unroll
            for (int e = 0; e < 16; ++e)
              a[h * 16 + e] = __float_as_uint(__fmaf_rn(sv[e], -8.f * OFF8_UNIT, __uint_as_float(a[h * 16 + e])));
          }
        }
        if (!(OFF8 && DUMP && is_dense)) {       // (a dump launch writes no output: its dense steps keep the corrected values for the dump only)
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            if (SCALAR_FOLD) {
              yf[cc + i] = __fmaf_rn(__uint_as_float(a[i]), f, yf[cc + i]);                  // fp32 accumulators: the integers as floats
              yf[cc + i + 1] = __fmaf_rn(__uint_as_float(a[i + 1]), f, yf[cc + i + 1]);
            } else {
              f32x2_t v;
              if (F8) asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(a[i]), "r"(a[i + 1]));
              else v = cvt_s32x2_f32x2(a[i], a[i + 1]);
              y2[(cc + i) >> 1] = fma_f32x2(v, f2, y2[(cc + i) >> 1]);
            }
          }
        }
        if (DUMP) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int tok = tok0 + c0 + cc + i;
            if (tok >= p.T) continue;
            // parity aid, not a hot path: every store is range-checked
            if (is_dense) {
              const size_t idx = ((size_t)n * p.N + row) * p.T + tok;
              if (p.acc_dump && row < p.N) {
                if (idx < (size_t)p.ng * p.N * p.T) p.acc_dump[idx] = F8 ? (int)(__uint_as_float(a[i]) * (OFF8 ? 512.f : 1.f)) : ((int)a[i]) >> 4;
                else record_error(SITE_PRE_DUMP, 1);
              }
            } else if (p.acc_hi_dump) {
              const size_t idx = ((size_t)blk * BROW + rl) * p.T + tok;
              if (blk < p.nnz && idx < (size_t)p.nnz * BROW * p.T) p.acc_hi_dump[idx] = F8 ? (int)(__uint_as_float(a[i]) * (OFF8 ? 512.f : 1.f)) : ((int)a[i]) >> 4;
              else record_error(SITE_PRE_DUMP, 2);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      // the buffer is free again: it will be written by step n + ACC_BUFS
      if (lane == 0 && n + ACC_BUFS < n_steps) mbar_arrive(&ready[(n + ACC_BUFS) % X_STAGES]);
      if (ft == 0) TRACE(5, n);
    }

    // ---------------------------------------------------------- zero-point term
    // y -= Z, the tensor core's sum over all groups of (scale * zero) * sumX (every lane takes part in the TMEM reads)
    if (p.Y != nullptr && n_windows > 0) {
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(z_done, (n_windows - 1) & 1, SITE_PRE_ACCFULL));
      if (ok) {
        tc_fence_after();
        const f32x2_t minus1 = pack_f32x2(-1.f, -1.f);
#pragma unroll
        for (int cc = 0; cc < COLS_PER_FOLD; cc += 32) {
          uint32_t z[32];
          tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + Z_COL0 + c0 + cc, z);
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            if (SCALAR_FOLD) {
              yf[cc + i] = __fsub_rn(yf[cc + i], __uint_as_float(z[i]));
              yf[cc + i + 1] = __fsub_rn(yf[cc + i + 1], __uint_as_float(z[i + 1]));
            } else {
              f32x2_t zz;
              asm("mov.b64 %0, {%1, %2};" : "=l"(zz) : "r"(z[i]), "r"(z[i + 1]));
              y2[(cc + i) >> 1] = fma_f32x2(zz, minus1, y2[(cc + i) >> 1]);
            }
          }
        }
      }
    }

    // ---------------------------------------------------------- epilogue
    if (ok && p.Y != nullptr && row < p.N) {
      const bool vec = (p.y_stride_t == 1) && ((p.y_stride_n & 7) == 0) && ((tok0 + c0) % 8 == 0) &&
                       ((reinterpret_cast<uintptr_t>(p.Y) & 15) == 0) && (tok0 + c0 + COLS_PER_FOLD <= p.T);
      if (vec) {
        __half* dst = p.Y + (size_t)row * p.y_stride_n + tok0 + c0;
#pragma unroll
        for (int i = 0; i < COLS_PER_FOLD; i += 8) {
          __align__(16) __half2 h[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 v = SCALAR_FOLD ? make_float2(yf[i + 2 * k], yf[i + 2 * k + 1]) : unpack_f32x2(y2[(i >> 1) + k]);
            h[k] = __floats2half2_rn(v.x * sxs[c0 + i + 2 * k], v.y * sxs[c0 + i + 2 * k + 1]);
          }
          *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<uint4*>(h);
        }
      } else {
#pragma unroll
        for (int i = 0; i < COLS_PER_FOLD; ++i) {
          const int tok = tok0 + c0 + i;
          if (tok < p.T)
            p.Y[(size_t)row * p.y_stride_n + (size_t)tok * p.y_stride_t] =
                __float2half_rn((SCALAR_FOLD ? yf[i] : (i & 1) ? unpack_f32x2(y2[i >> 1]).y : unpack_f32x2(y2[i >> 1]).x) * sxs[c0 + i]);
        }
      }
    }
  }

  // common exit: every role falls through to here, then the allocating warp frees TMEM
  tc_fence_before();
  __syncthreads();
#ifdef W4A4_TRACE
  if (tid == 0) { TRACE(8, 0); if (lin == p.trace_cta) p.trace[8 * 64 + 1] = t_start; }
#endif
  if (warp == WARP_MMA) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace pre
}  // namespace w4a4
