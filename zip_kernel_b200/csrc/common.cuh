// Shared device helpers for the sm_100a W4A4 kernels: mbarrier / TMA / tcgen05
// PTX wrappers, bounded waits, nibble unpacking and the device error word.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace w4a4 {

constexpr int BROW = 128;   // residual block rows  (reference: csrc/common/arch.cuh:30)
constexpr int BCOL = 128;   // quantisation group / residual block columns (arch.cuh:31)
constexpr int GROUP_BYTES = BCOL / 2;   // packed bytes of one group of one row

// Every device-side wait polls at most this many times, then records an error
// and gives up, so a logic error can never leave the GPU spinning.  (A long
// hardware suspend hint on try_wait was measured slower than plain polling:
// the wake-up adds latency to every pipeline step.)
constexpr uint32_t WAIT_POLL_LIMIT = 1u << 22;

// Device error word: 0 = ok.  Non-zero = (site id << 8) | detail of the first
// wait that gave up.  Read and cleared by w4a4_device_error().
__device__ int g_error_word = 0;

__device__ __forceinline__ void record_error(int site, int detail) {
  atomicCAS(&g_error_word, 0, (site << 8) | (detail & 0xff) | 0x40000000);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Plain (non-speculatable) global load.  The __ldg intrinsic is a non-volatile
// asm statement that the compiler may hoist above the branch that guards it, so
// a load whose address is only valid under a condition (a nullable operand, a
// ragged tail) must not use it: a hoisted __ldg on a null pointer faults.
template <typename T>
__device__ __forceinline__ T ld_plain(const T* p) { return *p; }

// Shared-memory accesses by 32-bit shared-window address.  The kernels carve their
// dynamic shared memory up with integer arithmetic, which hides the address space
// from the compiler: a plain dereference would become a generic load with 64-bit
// address arithmetic.  volatile: never moved across the barrier waits around them.
__device__ __forceinline__ uint4 lds_v4(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ float lds_f1(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t a) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ float4 lds_f4(uint32_t a) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(a));
  return v;
}
// two packed fp32 pairs (the operand form of the f32x2 instructions) with one load
__device__ __forceinline__ void lds_f32x2_pair(uint32_t a, unsigned long long& lo, unsigned long long& hi) {
  asm volatile("ld.shared.v2.u64 {%0,%1}, [%2];" : "=l"(lo), "=l"(hi) : "r"(a));
}
__device__ __forceinline__ void sts_v4(uint32_t a, const uint4& v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void sts_f2(uint32_t a, const float2& v) {
  asm volatile("st.shared.v2.f32 [%0], {%1,%2};" ::"r"(a), "f"(v.x), "f"(v.y) : "memory");
}

// Asynchronous global -> shared copies of 4 or 16 bytes that occupy no register
// while in flight (classic cp.async, tracked per thread with commit / wait groups).
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void sts_f1(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v) : "memory"); }

// ---------------------------------------------------------------- packed fp32 pairs
// The f32x2 instructions take two floats in one 64-bit register.  Values that
// live in that form (accumulators, broadcast scales) are kept as 64-bit integers
// so that no pack/unpack moves surround every instruction.
typedef unsigned long long f32x2_t;
__device__ __forceinline__ f32x2_t pack_f32x2(float lo, float hi) {
  f32x2_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ float2 unpack_f32x2(f32x2_t v) {
  float2 d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(v));
  return d;
}
__device__ __forceinline__ f32x2_t fma_f32x2(f32x2_t a, f32x2_t b, f32x2_t c) {
  f32x2_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
// two int32 -> one packed pair of floats
__device__ __forceinline__ f32x2_t cvt_s32x2_f32x2(uint32_t lo, uint32_t hi) {
  f32x2_t d;
  asm("{\n\t.reg .f32 l, h;\n\tcvt.rn.f32.s32 l, %1;\n\tcvt.rn.f32.s32 h, %2;\n\tmov.b64 %0, {l, h};\n\t}" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Arrival that cannot issue before `dep` is available (pass 0 in `zero` at run time): for handing back a buffer
// after plain shared-memory loads, whose data must have returned before the buffer's next writer is let in.
__device__ __forceinline__ void mbar_arrive_after(uint64_t* bar, uint32_t dep, uint32_t zero) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar) + (dep & zero)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
#ifdef W4A4_TEST_WAIT
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#else
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#endif
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (after recording the site) when the phase never
// completed; callers then stop using the pipeline and fall through to the exit.
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, uint32_t parity, int site, uint32_t limit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 4096) __nanosleep(64);
  }
  record_error(site, parity);
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int site) {
  for (uint32_t i = 0; i < WAIT_POLL_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i > 4096) __nanosleep(64);
  }
  record_error(site, parity);
  return false;
}

// The same for a role with slack (a producer that runs ahead of its consumer): it
// sleeps between polls from the first miss on, so that its polling does not take
// issue slots from the warps that do the arithmetic.  The bound in time is the same.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, int site) {
  for (uint32_t i = 0; i < WAIT_POLL_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    __nanosleep(i > 4096 ? 64 : 32);
  }
  record_error(site, parity);
  return false;
}

// ---------------------------------------------------------------- proxies / PDL
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Programmatic dependent launch: wait until the preceding kernel in the stream
// has completed and its writes are visible (no-op without the launch attribute).
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
// The same for a thread that goes on to read the preceding kernel's output with asynchronous copies
// (cp.async.bulk / TMA read through the async proxy; the preceding kernel wrote through the generic proxy).
// A kernel boundary orders the two proxies; a programmatic dependency is not documented to, so the
// cross-proxy fence is stated explicitly.  Once per issuing thread and launch.
__device__ __forceinline__ void grid_dependency_wait_for_async_reads() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("fence.proxy.async.global;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------- TMA (no multicast anywhere)
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, int c0, int c1,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1),
        "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, int c0, int c1, int c2,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(c0), "r"(c1), "r"(c2),
        "r"(smem_u32(bar))
      : "memory");
}

// 1-D bulk copy global -> shared; both addresses and the size are multiples of 16 bytes.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// ---------------------------------------------------------------- nibble helpers
// A packed word holds 8 signed nibbles: byte b = elements 2b (low) and 2b+1 (high).
// Even elements scaled by 16 as four s8 lanes.
__device__ __forceinline__ uint32_t nib_lo_x16(uint32_t w) { return (w << 4) & 0xF0F0F0F0u; }
// Odd elements scaled by 16 as four s8 lanes.
__device__ __forceinline__ uint32_t nib_hi_x16(uint32_t w) { return w & 0xF0F0F0F0u; }
// Sign-extend four 4-bit values sitting in the low nibble of each byte.
__device__ __forceinline__ uint32_t sext4_bytes(uint32_t x) {
  return x | ((x & 0x08080808u) * 0x1Eu);
}
__device__ __forceinline__ uint32_t nib_lo_s8(uint32_t w) { return sext4_bytes(w & 0x0F0F0F0Fu); }
__device__ __forceinline__ uint32_t nib_hi_s8(uint32_t w) { return sext4_bytes((w >> 4) & 0x0F0F0F0Fu); }
// One packed word (8 two's-complement nibbles) -> the e4m3 encodings of its 8 codes in their natural
// order: `first` = codes 0..3, `second` = codes 4..7.  prmt reads a selector's four low nibbles as
// byte indices into an 8-byte table - the packed nibbles ARE such indices: a nibble 0..7 picks the table
// byte, a nibble 8..15 (a negative code) selects "replicate the sign bit of table[nibble & 7]" and gives
// 0x00 for a table byte below 0x80.  Two look-ups per four codes: non-negative codes in the table of
// their encodings (negatives read 0x00); with bit 3 of every nibble flipped, negative codes in the table
// of their COMPLEMENTED encodings (which are below 0x80, so non-negatives read 0x00); a third prmt makes
// the 0xFF-where-negative mask that undoes the complement.  12 logic / permute operations per 8 codes.
__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ void nib8_to_e4m3(uint32_t w, uint32_t& first, uint32_t& second) {
  //            code = 0     1     2     3            4     5     6     7
  constexpr uint32_t POS_LO = 0x44403800u, POS_HI = 0x4E4C4A48u;
  //          ~e4m3 of -8    -7    -6    -5           -4    -3    -2    -1      (e4m3: D0 CE CC CA  C8 C4 C0 B8)
  constexpr uint32_t NEGC_LO = 0x3533312Fu, NEGC_HI = 0x473F3B37u;
  const uint32_t t = w ^ 0x88888888u, b = w << 4;
  // sign bits of codes 0..3 are bits 3, 7, 11, 15 of w = the top bits of b.byte0, w.byte0, b.byte1, w.byte1
  const uint32_t m0 = prmt_b32(w, b, 0x9D8Cu), m1 = prmt_b32(w, b, 0xBFAEu);
  first = prmt_b32(POS_LO, POS_HI, w) ^ prmt_b32(NEGC_LO, NEGC_HI, t) ^ m0;
  second = prmt_b32(POS_LO, POS_HI, w >> 16) ^ prmt_b32(NEGC_LO, NEGC_HI, t >> 16) ^ m1;
}

// The same two nibble sets as e4m3 bytes WITHOUT a table: an e4m3 byte 0x00..0x0F (exponent field 0 or 1) has
// the value byte * 2^-9 - the subnormals and the first binade of any binary float format are one linear
// ramp - so a nibble moved into a byte of its own IS a float proportional to the nibble.  Flipping bit 3
// turns the two's-complement nibble of a code c into c + 8 (0..15): four e4m3 lanes of value (c + 8) * 2^-9
// for one and two logic operations, the cost of the s8 widening above.  The offset 8 multiplies the
// activations' group sum and leaves with the zero-point term.
__device__ __forceinline__ uint32_t nib_lo_off8(uint32_t w) { return (w & 0x0F0F0F0Fu) ^ 0x08080808u; }
__device__ __forceinline__ uint32_t nib_hi_off8(uint32_t w) { return ((w >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u; }
constexpr float OFF8_UNIT = 1.f / 512.f;          // value of the e4m3 byte 0x01

// ---------------------------------------------------------------- legacy int8 MMA (decode path)
// D(16x8,s32) += A(16x32,s8,row) * B(32x8,s8,col)
__device__ __forceinline__ void mma_m16n8k32_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

}  // namespace w4a4
