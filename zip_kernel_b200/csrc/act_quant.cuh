// Kernel 1: per-token symmetric s4 activation quantisation.
//
// Contract (reference: cuda_kernel/csrc/activation_quant/activation_quant.cu:6-12,
// oracle tools/parity/quant_reference.py:82-112):
//   Xp = X[t, perm[:]];  scale_x[t] = fp16(max|Xp| / 7);  s = fp32(scale_x[t])
//   q  = clamp(rint(Xp / s), -8, 7)  (all zero when s == 0)
//   X_s4 packs two codes per byte (even element in the low nibble)
//   sum_X[t, g] = sum of the 128 codes of group g
// The division is the IEEE one (div.rn) and rint is round-half-even: codes are
// bit-identical to the oracle.  The reference's optimised kernel deviates here
// with an approximate division (activation_quant.cu:76-92); its naive kernel and
// its oracle do not (csrc_naive/activation_quant_naive.cu:132-133).
//
// A token is handled by a thread-block cluster of C CTAs (C = 1 for long
// prompts, up to 8 when only a few tokens are in flight and one CTA per token
// would leave the GPU idle).  Each CTA reads its K/C slice of the row from HBM
// exactly once with 128-bit loads (or gathered through perm), parks it in shared
// memory as fp16 while it reduces max|x| with warp shuffles, pushes its maximum
// into the shared memory of every CTA of the cluster and meets them at one
// cluster barrier; then it quantises its slice from shared memory.  A thread
// owns 8 consecutive codes = one 32-bit packed word, and 16 neighbouring lanes
// own one group, so sum_X is a 4-step shuffle reduction.
#pragma once

#include "common.cuh"

namespace w4a4 {

constexpr int QUANT_THREADS = 256;
constexpr size_t QUANT_MAX_SMEM = 200 * 1024;   // dynamic shared memory the kernel may ask for (one row slice)

struct QuantParams {
  const __half* X;        // (T, K) fp16, row stride ldx elements
  long long ldx;
  const int* perm;        // (K) or nullptr for identity
  int8_t* X_s4;           // (T, K/2) or nullptr
  __half* scale_x;        // (T)
  int* sum_X;             // (T, K/128) or nullptr
  int8_t* XE;             // optional expanded codes, group-major (see xe_offset), or nullptr
  float* sumxf;           // optional [ceil(T/16)][K/128][16] float group sums, or nullptr
  int T, K;
  int t_pad;              // tokens rounded up to 16: row pitch of the expanded layout
  int vec_ok;             // 1 when every row start is 16-byte aligned
  int C;                  // CTAs (cluster size) per token; divides K/128
  int stage_row;          // 1: perm given, C == 1: the dynamic shared memory holds the raw row, gathered while quantising
  int fmt;                // bytes of XE: 0 = s8 codes (even/odd order), 1 = e4m3 in natural order, 2 = e4m3 in even/odd order (see expand_word)
  // Fused prologues (SRC template parameter of the kernel): the value that is quantised is a function of the input row.
  const __half* norm_w;   // SRC_RMSNORM: (K) fp16 weight of the normalisation
  float eps;              // SRC_RMSNORM: added to the mean square
};

// What the quantiser reads.  SRC_PLAIN: X itself.  SRC_RMSNORM: fp16(fp16(x * r) * w[k]) with
// r = 1 / sqrt(mean(x^2) + eps) - the fp16 RMSNorm of a decoder layer, so that normalisation and
// quantisation are one launch and the normalised activations never travel through memory.
// SRC_SILU_MUL: the row holds [gate (K) | up (K)] (row stride ldx >= 2K) and the value is
// fp16(fp16(silu(gate)) * up) - the gated activation that feeds the down projection.
enum : int { SRC_PLAIN = 0, SRC_RMSNORM = 1, SRC_SILU_MUL = 2 };

// silu(x) = x / (1 + exp(-x)), rounded once to fp32 and then to fp16 - the value a double-precision
// evaluation gives, so that a CPU restatement with a correctly rounded exp produces the same fp16 bits.
// Fast path: single precision (expf is accurate to 2 ulp, the sum and the IEEE quotient add half an ulp
// each: relative error below 4e-7).  If the fp16 roundings of s (1 - 1e-6) and s (1 + 1e-6) agree, every
// value in between - the exact one included - rounds to that fp16 and the answer is known.  They differ
// for about one element in 250; those take the double-precision path below.
__device__ __forceinline__ double silu_f64(double x) {
  // exp(-x) = 2^n * exp(r), |r| <= ln2 / 2, Taylor polynomial of degree 11 (truncation below 2^-46)
  double t = fmin(fmax(-x, -60.0), 60.0);       // beyond +-60 the fp16 result no longer changes
  const double n = rint(t * 1.4426950408889634);
  const double r = fma(n, -1.9082149292705877e-10, fma(n, -0.6931471803691238, t));
  double p = 2.505210838544172e-8;               // 1 / 11!
  p = fma(p, r, 2.755731922398589e-7);
  p = fma(p, r, 2.7557319223985893e-6);
  p = fma(p, r, 2.48015873015873e-5);
  p = fma(p, r, 1.984126984126984e-4);
  p = fma(p, r, 1.388888888888889e-3);
  p = fma(p, r, 8.333333333333333e-3);
  p = fma(p, r, 4.1666666666666664e-2);
  p = fma(p, r, 1.6666666666666666e-1);
  p = fma(p, r, 0.5);
  p = fma(p, r, 1.0);
  p = fma(p, r, 1.0);
  const double e = __longlong_as_double(__double_as_longlong(p) + ((long long)(int)n << 52));   // * 2^n (|n| <= 87)
  const double d = 1.0 + e;
  // x / d by Newton's iteration on the reciprocal (d lies in [1, 2^88]: no overflow in single precision)
  double y = (double)__frcp_rn((float)d);
  y = fma(y, fma(-d, y, 1.0), y);
  y = fma(y, fma(-d, y, 1.0), y);
  const double q = x * y;
  return fma(fma(-d, q, x), y, q);
}
__device__ __forceinline__ __half silu_fp16(__half g) {
  const float x = __half2float(g);
  const float s = __fdiv_rn(x, 1.f + expf(-x));
  const __half lo = __float2half_rn(s * 0.999999f), hi = __float2half_rn(s * 1.000001f);
  if (__half_as_ushort(lo) == __half_as_ushort(hi)) return lo;
  return __float2half_rn((float)silu_f64((double)x));
}
// fp16 product of two fp16 values: exact in fp32 (two 11-bit significands), one rounding
__device__ __forceinline__ __half mul_fp16(__half a, __half b) {
  return __float2half_rn(__half2float(a) * __half2float(b));
}
template <int SRC>
__device__ __forceinline__ __half transform1(const QuantParams& p, const __half* xrow, int k, float rinv) {
  const __half x = xrow[k];
  if (SRC == SRC_RMSNORM) return mul_fp16(__float2half_rn(__half2float(x) * rinv), p.norm_w[k]);
  if (SRC == SRC_SILU_MUL) return mul_fp16(silu_fp16(x), xrow[p.K + k]);
  return x;
}
// the same for the 8 consecutive columns 8c .. 8c + 7 of a 16-byte aligned row
template <int SRC>
__device__ __forceinline__ uint4 transform8(const QuantParams& p, const __half* xrow, int c, float rinv) {
  uint4 v = ld_plain(reinterpret_cast<const uint4*>(xrow) + c);
  if (SRC == SRC_PLAIN) return v;
  __half* h = reinterpret_cast<__half*>(&v);
  if (SRC == SRC_RMSNORM) {
    const bool wv = (reinterpret_cast<uintptr_t>(p.norm_w) & 15) == 0;
    uint4 w4 = wv ? ld_plain(reinterpret_cast<const uint4*>(p.norm_w) + c) : make_uint4(0, 0, 0, 0);
    const __half* w = reinterpret_cast<const __half*>(&w4);
#pragma unroll
    for (int j = 0; j < 8; ++j) h[j] = mul_fp16(__float2half_rn(__half2float(h[j]) * rinv), wv ? w[j] : p.norm_w[c * 8 + j]);
  } else {
    const bool uv = ((reinterpret_cast<uintptr_t>(xrow + p.K)) & 15) == 0;
    uint4 u4 = uv ? ld_plain(reinterpret_cast<const uint4*>(xrow + p.K) + c) : make_uint4(0, 0, 0, 0);
    const __half* u = reinterpret_cast<const __half*>(&u4);
#pragma unroll
    for (int j = 0; j < 8; ++j) h[j] = mul_fp16(silu_fp16(h[j]), uv ? u[j] : xrow[p.K + c * 8 + j]);
  }
  return v;
}

// One packed word (8 codes) -> 8 bytes.  fmt 0: sign-extended s8, its four even-indexed codes, then its
// four odd-indexed ones (the order the s8 widening of the weights produces).  fmt 1: e4m3 encodings in the
// codes' natural order (the order of the weights' table look-up and of prepared weights).
// fmt 2: e4m3 encodings in the even-then-odd order of fmt 0 (read against packed weights widened on the SM).
__device__ __forceinline__ uint2 expand_word(uint32_t w, int fmt = 0) {
  if (fmt != 0) {
    uint2 r;
    nib8_to_e4m3(w, r.x, r.y);
    if (fmt == 2) r = make_uint2(prmt_b32(r.x, r.y, 0x6420u), prmt_b32(r.x, r.y, 0x7531u));
    return r;
  }
  return make_uint2(nib_lo_s8(w), nib_hi_s8(w));
}

// Expanded activation layout ("XE") read by both GEMM kernels: one byte per code,
// group-major, [K/128][t_pad][128 bytes].  The 128 bytes of one (group, token)
// hold the group's 16 packed words in order, each word turned into 8 bytes (its
// four even-indexed codes, then its four odd-indexed ones, sign-extended), and
// the eight 16-byte chunks of the line are stored at chunk ^ (token & 7).  A run
// of consecutive tokens of one group is therefore contiguous in memory and is
// already the 128-byte-swizzled K-major operand tile an int8 MMA reads, so the
// GEMM kernels fetch it with one plain bulk copy.  `c` is the index of the packed
// word in the token's row (c / 16 = group).
__device__ __forceinline__ size_t xe_offset(int t, int c, int t_pad) {
  const int g = c >> 4, w = c & 15;
  return ((size_t)g * t_pad + t) * 128 + ((((w >> 1) ^ (t & 7)) << 4) | ((w & 1) << 3));
}

// max(m, |v[0..7]|): the maximum is taken in half precision (exact), one conversion pair at the end;
// like fmaxf, __hmax2 returns the other operand when one is NaN
__device__ __forceinline__ float half_abs_max8(const uint4& v, float m) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
  const __half2 mm = __hmax2(__hmax2(__habs2(h[0]), __habs2(h[1])), __hmax2(__habs2(h[2]), __habs2(h[3])));
  const float2 f = __half22float2(mm);
  return fmaxf(m, fmaxf(f.x, f.y));
}

// The code of x for the token scale s: clamp(rint(x / s), -8, 7) with the IEEE quotient.  The divisor is
// the same for a whole token, so the division is a product with r = RN(1 / s) followed by one residual
// correction (q0 = x r; e = x - s q0, exact in an FMA; q = q0 + e r).  For every x and s that are fp16
// values - all this kernel sees - that equals div.rn(x, s) bit for bit wherever |x / s| < 16 and gives the
// same code everywhere: checked exhaustively on the GPU over all 31 743 positive fp16 scales x all finite
// fp16 values.  Three instructions instead of the ten-odd of a full division.
__device__ __forceinline__ int quant_code(float x, float s, float r) {
  const float q0 = __fmul_rn(x, r);
  const float q = fmaf(fmaf(-s, q0, x), r, q0);
  const int c = __float2int_rn(q);                          // round to nearest even, like rint
  return max(min(c, 7), -8);
}

// Quantises slice `rank` (of p.C) of token t with a CTA of NTHREADS threads.  Every
// thread of the CTA calls it; for p.C > 1 the CTAs of a cluster call it together
// with rank = their cluster rank.  `quant_smem` (16-byte aligned) holds the slice
// (2 * K / C bytes; with p.stage_row - one CTA per token - the raw row, 2 * K bytes).
// With WAIT_DEP the function itself waits for the preceding kernel in the stream
// (programmatic dependent launch) - after it has fetched the thread's first
// permutation indices, which belong to the weights and do not depend on that
// kernel: the dependent part of the load phase is then one global round trip.
template <int NTHREADS, bool WAIT_DEP, int SRC = SRC_PLAIN>
__device__ __forceinline__ void quant_token(const QuantParams& p, int t, int rank, unsigned char* quant_smem,
                                            float* warp_max, float* peer_max) {
  constexpr int QUANT_THREADS = NTHREADS;
  uint4* row = reinterpret_cast<uint4*>(quant_smem);          // this CTA's chunks of 8 halfs
  const int C = p.C;
  const int tid = threadIdx.x;
  const int nchunk_row = p.K >> 3;
  const int c_lo = rank * (nchunk_row / C), c_hi = c_lo + nchunk_row / C;   // slice, a multiple of 16 chunks
  const __half* xrow = p.X + (long long)t * p.ldx;

  // source columns of chunk c (8 consecutive permuted positions)
  const bool perm_vec = (reinterpret_cast<uintptr_t>(p.perm) & 15) == 0;
  auto load_perm = [&](int c, int4& pa, int4& pb) {
    if (perm_vec) {
      pa = ld_plain(reinterpret_cast<const int4*>(p.perm) + c * 2);
      pb = ld_plain(reinterpret_cast<const int4*>(p.perm) + c * 2 + 1);
    } else {
      pa = make_int4(p.perm[c * 8], p.perm[c * 8 + 1], p.perm[c * 8 + 2], p.perm[c * 8 + 3]);
      pb = make_int4(p.perm[c * 8 + 4], p.perm[c * 8 + 5], p.perm[c * 8 + 6], p.perm[c * 8 + 7]);
    }
  };
  int4 pa = make_int4(0, 0, 0, 0), pb = pa;
  // A CTA may write into a peer's shared memory only once that peer is known to have started: every
  // CTA of the cluster arrives here at once and the matching wait sits just before the remote stores,
  // so the row load hides the barrier's latency.
  if (C > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  if (p.perm != nullptr && c_lo + tid < c_hi) load_perm(c_lo + tid, pa, pb);
  if (WAIT_DEP) grid_dependency_wait();

  float rinv = 1.f;
  if (SRC == SRC_RMSNORM) {
    // Mean square of the WHOLE row (every CTA of a token's cluster reads it: a few KB from L2), summed in
    // double precision - the squares of fp16 values are exact there and the sum's rounding error is far
    // below the fp32 rounding that follows - then r = 1 / sqrt(fp32(mean) + eps) with IEEE operations.
    __shared__ double warp_ss[NTHREADS / 32];
    double ss = 0.0;
    if (p.vec_ok) {
      const uint4* src = reinterpret_cast<const uint4*>(xrow);
      for (int c = tid; c < nchunk_row; c += QUANT_THREADS) {
        const uint4 v = ld_plain(src + c);
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __half22float2(h[i]);
          ss += (double)(f.x * f.x) + (double)(f.y * f.y);
        }
      }
    } else {
      for (int k = tid; k < p.K; k += QUANT_THREADS) {
        const float f = __half2float(xrow[k]);
        ss += (double)(f * f);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((tid & 31) == 0) warp_ss[tid >> 5] = ss;
    __syncthreads();
    ss = 0.0;
#pragma unroll
    for (int w = 0; w < NTHREADS / 32; ++w) ss += warp_ss[w];
    const float ms = (float)(ss / (double)p.K);
    rinv = __frcp_rn(__fsqrt_rn(__fadd_rn(ms, p.eps)));
  }

  float m = 0.f;
  if (p.perm == nullptr && p.vec_ok) {
    for (int c = c_lo + tid; c < c_hi; c += QUANT_THREADS) {
      uint4 v = transform8<SRC>(p, xrow, c, rinv);
      row[c - c_lo] = v;
      m = half_abs_max8(v, m);
    }
  } else if (p.stage_row) {
    // Column permutation, one CTA per token: the whole raw row is brought into shared memory with
    // coalesced 128-bit loads (one global round trip, in flight together with the first permutation
    // indices).  The maximum does not depend on the order of the columns, so it is taken from the values
    // as they arrive; the gather runs on shared memory while quantising.  (A gather from global memory
    // costs a second, dependent round trip and one L1 wavefront per element.)
    __half* raw = reinterpret_cast<__half*>(row);
    if (p.vec_ok) {
      for (int c = tid; c < nchunk_row; c += QUANT_THREADS) {
        const uint4 v = transform8<SRC>(p, xrow, c, rinv);
        row[c] = v;
        m = half_abs_max8(v, m);
      }
    } else {
      for (int k = tid; k < p.K; k += QUANT_THREADS) {
        const __half x = transform1<SRC>(p, xrow, k, rinv);
        raw[k] = x;
        m = fmaxf(m, fabsf(__half2float(x)));
      }
    }
  } else {
    for (int c = c_lo + tid; c < c_hi; c += QUANT_THREADS) {
      __align__(16) __half h[8];
      if (p.perm) {
        if (c != c_lo + tid) load_perm(c, pa, pb);
        const int idx[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = transform1<SRC>(p, xrow, idx[j], rinv);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) h[j] = transform1<SRC>(p, xrow, c * 8 + j, rinv);
      }
      uint4 v = *reinterpret_cast<uint4*>(h);
      row[c - c_lo] = v;
      m = half_abs_max8(v, m);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((tid & 31) == 0) warp_max[tid >> 5] = m;
  __syncthreads();
  m = warp_max[0];
#pragma unroll
  for (int w = 1; w < QUANT_THREADS / 32; ++w) m = fmaxf(m, warp_max[w]);
  if (C > 1) {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");   // all peers have started
    // push this CTA's maximum into slot `rank` of every CTA of the cluster
    if (tid < C) {
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(&peer_max[rank])), "r"(tid));
      asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(m) : "memory");
    }
    __syncwarp();
    // every thread of every CTA of the cluster arrives here: hardware barrier, no spin
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    for (int c = 0; c < C; ++c) m = fmaxf(m, peer_max[c]);
  }

  const __half scale16 = __float2half_rn(__fdiv_rn(m, 7.0f));
  const float s = __half2float(scale16);
  const bool zero_row = !(s > 0.f);
  const float s_safe = zero_row ? 1.0f : s;
  const float r_safe = __frcp_rn(s_safe);
  if (tid == 0 && rank == 0) p.scale_x[t] = scale16;

  uint32_t* out = p.X_s4 ? reinterpret_cast<uint32_t*>(p.X_s4 + (long long)t * (p.K >> 1)) : nullptr;
  int* sums = p.sum_X ? p.sum_X + (long long)t * (p.K >> 7) : nullptr;
  const int ng = p.K >> 7;
  float* sumsf = p.sumxf ? p.sumxf + ((long long)(t >> 4) * ng) * 16 + (t & 15) : nullptr;
  // All lanes of a warp run the same number of iterations (the slice is a multiple
  // of 16 chunks and lanes are consecutive), so the shuffles below are convergent
  // for every 16-lane half that holds a live group.
  for (int c0 = c_lo; c0 < c_hi; c0 += QUANT_THREADS) {
    const int c = c0 + tid;
    const bool live = c < c_hi;
    uint32_t word = 0;
    int sum = 0;
    if (live) {
      uint4 v;
      if (p.stage_row) {
        const __half* raw = reinterpret_cast<const __half*>(row);
        if (c0 != c_lo) load_perm(c, pa, pb);        // the first chunk's indices were fetched up front
        __align__(16) __half g[8];
        g[0] = raw[pa.x]; g[1] = raw[pa.y]; g[2] = raw[pa.z]; g[3] = raw[pa.w];
        g[4] = raw[pb.x]; g[5] = raw[pb.y]; g[6] = raw[pb.z]; g[7] = raw[pb.w];
        v = *reinterpret_cast<uint4*>(g);
      } else {
        v = row[c - c_lo];
      }
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        // a row whose scale rounds to zero holds only values far below 0.5: divided by 1 they give code 0
        const int i0 = quant_code(f.x, s_safe, r_safe), i1 = quant_code(f.y, s_safe, r_safe);
        sum += i0 + i1;
        // the low four bits of each code into their nibble (constant positions after unrolling)
        asm("bfi.b32 %0, %1, %0, %2, 4;" : "+r"(word) : "r"(i0), "r"(8 * i));
        asm("bfi.b32 %0, %1, %0, %2, 4;" : "+r"(word) : "r"(i1), "r"(8 * i + 4));
      }
      if (out) out[c] = word;
      if (p.XE) *reinterpret_cast<uint2*>(p.XE + xe_offset(t, c, p.t_pad)) = expand_word(word, p.fmt);
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (live && (tid & 15) == 0) {
      if (sums) sums[c >> 4] = sum;
      if (sumsf) sumsf[(c >> 4) * 16] = (float)sum;
    }
  }
}

// NT threads per CTA: 256 when a token is spread over a cluster or few tokens are in flight (latency), 128 when
// there are many tokens (throughput: a thread's set-up - permutation indices, address arithmetic, the
// reductions - is then shared by twice as many elements and twice as many CTAs fit an SM).
template <int NT, int SRC = SRC_PLAIN>
__global__ void __launch_bounds__(NT)
act_quant_kernel(const QuantParams p) {
  extern __shared__ __align__(16) unsigned char quant_dyn_smem[];
  __shared__ float warp_max[NT / 32];
  __shared__ float peer_max[8];
  // Let the next kernel in the stream be scheduled early; then wait until the
  // producer of X (and every earlier user of the output buffers) has finished.
  // (the wait for the producer of X and for every earlier user of the output buffers happens inside)
  grid_launch_dependents();
  const int t = blockIdx.x / p.C;
  quant_token<NT, true, SRC>(p, t, blockIdx.x - t * p.C, quant_dyn_smem, warp_max, peer_max);
}

// Builds the expanded layout and the transposed float group sums from already
// quantised activations (the operator-level entry points that receive X_s4 /
// sum_X from the caller).
struct ExpandParams {
  const int8_t* X_s4;   // (T, K/2)
  const int* sum_X;     // (T, K/128) or nullptr
  int8_t* XE;           // group-major expanded codes (see xe_offset)
  float* sumxf;         // [ceil(T/16)][K/128][16]
  int T, K, t_pad;
  int fmt;              // as QuantParams::fmt
};

__global__ void __launch_bounds__(256) expand_activations_kernel(const ExpandParams p) {
  grid_launch_dependents();
  grid_dependency_wait();
  const long long words = (long long)p.T * (p.K >> 3);
  const long long stride = (long long)gridDim.x * blockDim.x;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(p.X_s4);
  const int wpr = p.K >> 3;     // packed words per token
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += stride) {
    const int t = (int)(i / wpr), c = (int)(i - (long long)t * wpr);
    *reinterpret_cast<uint2*>(p.XE + xe_offset(t, c, p.t_pad)) = expand_word(ld_plain(src + i), p.fmt);
  }
  if (p.sum_X) {
    const int ng = p.K >> 7;
    const long long n = (long long)p.T * ng;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
      const int t = (int)(i / ng), g = (int)(i - (long long)t * ng);
      p.sumxf[((long long)(t >> 4) * ng + g) * 16 + (t & 15)] = (float)ld_plain(p.sum_X + i);
    }
  }
}

// Weights prepared for the fp8 tensor-core path: every packed word of nibbles (dense rows or residual
// blocks alike) becomes its 8 codes as e4m3 bytes in their natural order, so a row of K codes is K bytes
// and the row-major shape is kept.
__global__ void __launch_bounds__(256) prepare_weights_kernel(const uint32_t* packed, uint2* out, long long words) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += stride)
    out[i] = expand_word(ld_plain(packed + i), 1);
}

// Dense fp16 copy of the low-precision weights for the W4A16 route (many tokens, no residual blocks):
// out[n, k] = fp16( fp16( fp16(code) - zero[n, g] ) * scale[n, g] ), two roundings in half precision, exactly what the
// reference's dequantisation kernel computes (triton_kernel/dequant_w4_to_fp16.py:61-128).  One thread per packed word.
__global__ void __launch_bounds__(256) dequant_weights_kernel(const uint32_t* __restrict__ packed, const __half* __restrict__ scale,
                                                              const __half* __restrict__ zero, uint4* __restrict__ out, int N, int K) {
  const long long words = (long long)N * (K >> 3);
  const long long stride = (long long)gridDim.x * blockDim.x;
  const int wpr = K >> 3, ng = K >> 7;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += stride) {
    const int n = (int)(i / wpr), c = (int)(i - (long long)n * wpr);
    const uint32_t w = ld_plain(packed + i);
    const __half s = scale[(size_t)n * ng + (c >> 4)], z = zero[(size_t)n * ng + (c >> 4)];
    __align__(16) __half h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int code = ((int)(w << (28 - 4 * j))) >> 28;           // sign-extended nibble j
      h[j] = __hmul(__hsub(__int2half_rn(code), z), s);
    }
    out[i] = *reinterpret_cast<uint4*>(h);
  }
}

}  // namespace w4a4
