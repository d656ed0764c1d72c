// Output exchange of the column-parallel linear without a collective library: every rank stores its
// shard of the output straight into every rank's copy of the full output (plain 16-byte stores to
// peer-mapped memory over NVLink - no TMA, no multicast, no bulk copy from or to peer memory), then
// raises one flag per peer; the same kernel then waits, with a bound, until the flags of all ranks
// have reached the current epoch.  The reference is single-GPU and has no counterpart.
//
// Memory model: data stores -> __threadfence_system() -> per-destination block counter -> the last
// block of a destination stores the flag with release semantics at system scope; the waiting side loads
// the flags with acquire semantics at system scope.  A flag that never arrives makes the wait give up
// after its poll limit: the kernel records the device error word and returns, the context stays usable.
#pragma once

#include "common.cuh"

namespace w4a4 {

constexpr int PEER_MAX_WORLD = 16;
constexpr int SITE_PEER_WAIT = 0x60;

struct PushParams {
  const unsigned char* src;        // this rank's shard: `rows` rows of `row_bytes` bytes, `src_pitch` bytes apart
  long long src_pitch;
  unsigned char* dst[PEER_MAX_WORLD];      // every rank's full-output buffer (own buffer included), peer-mapped
  unsigned int* flags[PEER_MAX_WORLD];     // every rank's flag array [world]; this rank writes entry `rank`
  long long dst_pitch;             // row pitch of the full output in bytes
  long long dst_offset;            // byte offset of this rank's shard inside the full output (first row, first column)
  int rows, row_bytes;
  int world, rank;
  unsigned int* state;             // local device words: [0] calls completed by this rank (what the wait expects next, minus 1),
                                   // [1 .. world] shards sent to each destination so far, [1 + world .. 2 world] blocks finished
                                   // per destination in the running call (zero between calls)
  unsigned int poll_limit;
  int blocks_per_dst;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256) peer_push_wait_kernel(const PushParams p) {
  grid_launch_dependents();
  grid_dependency_wait();                   // the shard is written by the preceding kernel in the stream
  const int dst_i = blockIdx.x / p.blocks_per_dst, blk = blockIdx.x - dst_i * p.blocks_per_dst;
  unsigned char* dst = p.dst[dst_i] + p.dst_offset;
  const bool vec = ((reinterpret_cast<uintptr_t>(p.src) | reinterpret_cast<uintptr_t>(dst) | (uintptr_t)p.src_pitch |
                     (uintptr_t)p.dst_pitch | (uintptr_t)p.row_bytes) & 15) == 0;
  if (vec) {
    const int vpr = p.row_bytes >> 4;                   // 16-byte vectors per row
    const long long total = (long long)p.rows * vpr;
    for (long long i = (long long)blk * blockDim.x + threadIdx.x; i < total; i += (long long)p.blocks_per_dst * blockDim.x) {
      const long long r = i / vpr, c = i - r * vpr;
      const uint4 v = *reinterpret_cast<const uint4*>(p.src + r * p.src_pitch + c * 16);
      *reinterpret_cast<uint4*>(dst + r * p.dst_pitch + c * 16) = v;
    }
  } else {
    const long long total = (long long)p.rows * (p.row_bytes >> 1);   // fp16 elements
    const int epr = p.row_bytes >> 1;
    for (long long i = (long long)blk * blockDim.x + threadIdx.x; i < total; i += (long long)p.blocks_per_dst * blockDim.x) {
      const long long r = i / epr, c = i - r * epr;
      *reinterpret_cast<unsigned short*>(dst + r * p.dst_pitch + c * 2) = *reinterpret_cast<const unsigned short*>(p.src + r * p.src_pitch + c * 2);
    }
  }
  __threadfence_system();                                    // this thread's stores are performed at the destination
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned int* finished = p.state + 1 + p.world + dst_i;
    // with one block per destination (a decode-sized shard) there is nothing to count
    const bool last = p.blocks_per_dst == 1 || atomicAdd(finished, 1u) + 1 == (unsigned int)p.blocks_per_dst;
    if (last) {
      if (p.blocks_per_dst > 1) *finished = 0;               // ready for the next call (stream-ordered after this kernel)
      // only this one thread touches the destination's send count in a call: flag = number of shards sent so far
      const unsigned int sent = ++p.state[1 + dst_i];
      st_release_sys(p.flags[dst_i] + p.rank, sent);         // "my shard number `sent` is in your buffer"
    }
  }
  // block 0 waits for every rank's shard of this call (its own included); only block 0 reads and advances
  // the call count, so no other block can observe it half-way
  if (blockIdx.x == 0) {
    const unsigned int epoch = p.state[0] + 1;
    __shared__ int failed;
    if (threadIdx.x == 0) failed = 0;
    __syncthreads();
    if (threadIdx.x < p.world) {
      const unsigned int* f = p.flags[p.rank] + threadIdx.x;
      bool ok = false;
      for (unsigned int i = 0; i < p.poll_limit; ++i) {
        if ((int)(ld_acquire_sys(f) - epoch) >= 0) { ok = true; break; }
        if (i > 4096) __nanosleep(100);
      }
      if (!ok) {
        record_error(SITE_PEER_WAIT, threadIdx.x);
        failed = 1;
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) p.state[0] = epoch;                // also after a timeout: the next call expects the next shard
    (void)failed;
  }
}

}  // namespace w4a4
