// extern "C" entry points of libw4a4_b200.so: argument validation, tensor-map
// construction, kernel selection and launch.  The contract of every function
// is documented in include/w4a4_b200.h.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_map>

#include "../../include/w4a4_b200.h"
#include "act_quant.cuh"
#include "common.cuh"
#include "decode_gemm.cuh"
#include "prefill_gemm.cuh"
#include "prefill_pair_gemm.cuh"
#include "peer_gather.cuh"

namespace {

thread_local std::string t_last_error;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  t_last_error = buf;
  return code;
}

// Every entry point starts with a clean per-thread message, so w4a4_last_error()
// never reports the failure of an earlier call after a successful one.
inline void begin_call() { t_last_error.clear(); }

#define CHECK_ARG(cond, ...) \
  do {                       \
    if (!(cond)) return fail(W4A4_ERR_BAD_ARG, __VA_ARGS__); \
  } while (0)

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// ------------------------------------------------------------------ device info
struct DeviceInfo {
  int sm_count = 0;
  bool attrs_set = false;
};
std::mutex g_mutex;
DeviceInfo g_dev[64];

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

// The kernels' dynamic shared-memory limits are function attributes of the device's
// context: they are set once per device, on the first call that reaches it.
cudaError_t set_kernel_attributes() {
  using namespace w4a4;
  cudaError_t e = cudaSuccess;
  // W4A4_CARVEOUT=0 leaves the shared-memory carve-out to the driver's heuristic (A/B experiments).  By default
  // the kernels ask for the largest carve-out: a launch that keeps ONE ~100 KB CTA per SM would otherwise be
  // given a carve-out that has no room for the next kernel's CTA, and the two could never overlap.
  const bool carve = !(getenv("W4A4_CARVEOUT") && atoi(getenv("W4A4_CARVEOUT")) == 0);
  auto set = [&](auto kern, size_t smem) {
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess && carve)
      e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  };
  set(dec::decode_gemm_kernel<1, false>, dec::smem_bytes(1));
  set(dec::decode_gemm_kernel<2, false>, dec::smem_bytes(2));
  set(dec::decode_gemm_kernel<4, false>, dec::smem_bytes(4));
  set(dec::decode_gemm_kernel<1, true>, dec::smem_bytes(1));
  set(dec::decode_gemm_kernel<2, true>, dec::smem_bytes(2));
  set(dec::decode_gemm_kernel<4, true>, dec::smem_bytes(4));
  set(pre::prefill_gemm_kernel<false, false, false>, pre::smem_bytes(false, false));
  set(pre::prefill_gemm_kernel<true, false, false>, pre::smem_bytes(false, false));
  set(pre::prefill_gemm_kernel<false, true, true>, pre::smem_bytes(true, true));
  set(pre::prefill_gemm_kernel<true, true, true>, pre::smem_bytes(true, true));
  set(pre::prefill_gemm_kernel<false, true, false>, pre::smem_bytes(true, false));
  set(pre::prefill_gemm_kernel<true, true, false>, pre::smem_bytes(true, false));
  set(pp::prefill_pair_gemm_kernel<false, false, false>, pp::smem_bytes(false));
  set(pp::prefill_pair_gemm_kernel<true, false, false>, pp::smem_bytes(false));
  set(pp::prefill_pair_gemm_kernel<false, true, true>, pp::smem_bytes(true));
  set(pp::prefill_pair_gemm_kernel<true, true, true>, pp::smem_bytes(true));
  set(act_quant_kernel<128>, QUANT_MAX_SMEM);
  set(act_quant_kernel<QUANT_THREADS>, QUANT_MAX_SMEM);
  set(act_quant_kernel<128, SRC_RMSNORM>, QUANT_MAX_SMEM);
  set(act_quant_kernel<QUANT_THREADS, SRC_RMSNORM>, QUANT_MAX_SMEM);
  set(act_quant_kernel<128, SRC_SILU_MUL>, QUANT_MAX_SMEM);
  set(act_quant_kernel<QUANT_THREADS, SRC_SILU_MUL>, QUANT_MAX_SMEM);
  return e;
}

int current_device(DeviceInfo** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(W4A4_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceInfo& d = g_dev[dev];
  if (d.sm_count == 0) {
    e = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));
  }
  if (!d.attrs_set) {
    e = set_kernel_attributes();
    if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    d.attrs_set = true;
  }
  if (!g_encode) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
      return fail(W4A4_ERR_LAUNCH, "cuTensorMapEncodeTiled entry point unavailable");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  *out = &d;
  return W4A4_OK;
}

// 2-D byte tensor map: `rows` rows of `row_bytes` bytes (pitch = row_bytes), box
// box_bytes x box_rows.  Out-of-range rows read as zero.  A map depends only on the
// address and the geometry, so encoded maps are kept (weights are called with the
// same pointers over and over) and a repeated call costs a table look-up instead
// of a driver call.
struct MapKey {
  const void* ptr;
  uint64_t row_bytes, rows;
  uint32_t box_bytes, box_rows;
  int swz;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && row_bytes == o.row_bytes && rows == o.rows && box_bytes == o.box_bytes &&
           box_rows == o.box_rows && swz == o.swz;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
    h ^= (k.row_bytes + 0x9E3779B9u + (h << 6) + (h >> 2));
    h ^= (k.rows + 0x9E3779B9u + (h << 6) + (h >> 2));
    h ^= (((uint64_t)k.box_bytes << 32 | k.box_rows) + (uint64_t)k.swz + (h << 6) + (h >> 2));
    return h;
  }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
constexpr size_t MAP_CACHE_LIMIT = 4096;

int make_map(CUtensorMap* m, const void* ptr, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes,
             uint32_t box_rows, CUtensorMapSwizzle swz) {
  const MapKey key{ptr, row_bytes, rows, box_bytes, box_rows, (int)swz};
  {
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) {
      *m = it->second;
      return W4A4_OK;
    }
  }
  cuuint64_t dims[2] = {row_bytes, rows ? rows : 1};
  cuuint64_t strides[1] = {row_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(W4A4_ERR_LAUNCH, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_maps.size() >= MAP_CACHE_LIMIT) g_maps.clear();
  g_maps.emplace(key, *m);
  return W4A4_OK;
}

// Expanded activations: [K/128][t_pad][128] bytes with t_pad = T rounded up to 16,
// plus slack so that a full 128-token tile copy of the last group stays inside.
inline int xe_t_pad(int T) { return (T + 15) / 16 * 16; }
inline size_t xe_bytes(int T, int K) { return (size_t)xe_t_pad(T) * K + 128 * 128; }

// ------------------------------------------------------------------ workspace layout
// Scratch for activations in the layout the GEMM kernels read: per-token scales
// (only when the library quantises), expanded codes and transposed group sums.
struct WsLayout {
  size_t scale_x, xe, sumxf, total;
};
WsLayout ws_layout(int T, int K) {
  WsLayout w;
  const size_t ng = K / 128, tok_tiles = (T + 15) / 16;
  size_t off = 0;
  w.scale_x = off;  off += round_up((size_t)T * 2, 256);
  w.xe = off;       off += round_up(xe_bytes(T, K), 1024);
  w.sumxf = off;    off += round_up(tok_tiles * ng * 16 * 4, 256);
  w.total = off;
  return w;
}

// ------------------------------------------------------------------ plans
struct DecodePlan {
  int row_tiles, tok_tiles, split;   // split = CTAs (cluster size) per block-row
};
DecodePlan plan_decode(int T, int N, int dense_steps, int sm_count, int tokens_per_pass) {
  using namespace w4a4;
  DecodePlan p;
  p.row_tiles = (N + dec::ROWS - 1) / dec::ROWS;
  p.tok_tiles = (T + tokens_per_pass - 1) / tokens_per_pass;
  // Largest power-of-two cluster that keeps the grid within the two CTAs per SM that fit at once (a grid
  // that needs a second wave costs far more than it gains; measured on the Llama-3-8B decode shapes with
  // dependent launches enabled).  Measured and not adopted: at most ONE CTA per SM (any cluster size up to
  // 8, persistent CTAs walking several block-rows when there are more block-rows than SMs) so that the
  // next kernel's CTAs become resident early - a pure-copy kernel of this footprint gains 3 us per launch
  // that way (8.4 MB: 6.7 -> 3.1 us), this kernel loses 1-8 us: its time after the dependency resolves
  // (activation fetch, the MMAs of the prefetched tiles, cluster reduction) is serial and halving the
  // warps per SM doubles it, 128-byte wide TMA boxes feed one SM at only ~34 GB/s, so a CTA with two
  // block-rows is bound by its copy engine, and the loop over block-rows itself cost 5 % on every shape.
  const long long base = (long long)p.row_tiles * p.tok_tiles;
  long long s = 1;
  while (s * 2 <= dec::MAX_CLUSTER && base * s * 2 * 10 <= 18LL * sm_count) s *= 2;
  // tuning override for A/B experiments and for the split-parity test; read on every call so that one
  // process can compare cluster sizes on one shape
  const char* env_split_s = getenv("W4A4_DECODE_SPLIT");
  const int env_split = env_split_s ? atoi(env_split_s) : 0;
  if (env_split > 0) s = env_split;
  if (s > dec::MAX_CLUSTER) s = dec::MAX_CLUSTER;
  while (s > dense_steps && s > 1) s /= 2;
  p.split = (int)s;
  return p;
}

struct GemmArgs {
  const void* W_low;
  const void* W_high;
  const void* W_low_prep;  // weights prepared as e4m3 bytes (w4a4_prepare_weights), or NULL: the tensor-core path
  const void* W_high_prep; // then runs its fp8 instantiation; the streaming path always reads the packed arrays
  const int32_t* hp_row_offsets;
  const int32_t* hp_col_indices;
  const void* X_s4;        // packed activation codes, or NULL when XE is given
  const void* XE;          // expanded activation codes (T, K), or NULL
  const float* sumxf;      // transposed float group sums that go with XE
  const void* scale_u4;
  const void* zero_u4;
  const int32_t* sum_X;
  const void* scale_x;
  void* Y;
  int32_t* acc_dump;
  int32_t* acc_hi_dump;
  int T, K, N, nnz, flags;
  bool do_dense;
  float sparse_weight;
  int xe_fmt;              // bytes of the expanded codes: W4A4_CODES_S8 / _E4M3 (prepared weights) / _E4M3_PACKED
  void* ws;
  size_t ws_bytes;
  cudaStream_t stream;
};

// Launch with the programmatic-dependent-launch attribute (the kernels call
// griddepcontrol.wait before they touch memory another kernel may still use) and,
// for cluster > 1, a 1-D thread-block cluster.
template <typename... KArgs, typename... Args>
cudaError_t launch_ex(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, int cluster,
                      Args... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  // W4A4_NO_PDL=1 switches programmatic dependent launch off (A/B experiments)
  static const bool no_pdl = getenv("W4A4_NO_PDL") && atoi(getenv("W4A4_NO_PDL")) != 0;
  if (!no_pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

int launch_expand(const GemmArgs& a, void* XE, float* sumxf, DeviceInfo* dev) {
  using namespace w4a4;
  ExpandParams e;
  e.X_s4 = static_cast<const int8_t*>(a.X_s4);
  e.sum_X = a.sum_X;
  e.XE = static_cast<int8_t*>(XE);
  e.sumxf = sumxf;
  e.T = a.T;
  e.K = a.K;
  e.t_pad = xe_t_pad(a.T);
  e.fmt = a.xe_fmt;
  const long long words = (long long)a.T * (a.K / 8);
  long long blocks = (words + 255) / 256;
  if (blocks > 4LL * dev->sm_count) blocks = 4LL * dev->sm_count;
  cudaError_t err = launch_ex(expand_activations_kernel, dim3((unsigned)blocks), dim3(256), 0, a.stream, 1, e);
  if (err != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "expand kernel launch: %s", cudaGetErrorString(err));
  return W4A4_OK;
}

int launch_decode(const GemmArgs& a, DeviceInfo* dev) {
  using namespace w4a4;
  const bool dump = a.acc_dump || a.acc_hi_dump;
  const bool has_sparse = a.nnz > 0 && a.sparse_weight != 0.f;
  if (!a.do_dense && !has_sparse) return fail(W4A4_ERR_BAD_ARG, "neither a dense nor a residual operand was given");
  const int ng = a.K / BCOL;
  const int row_tiles = (a.N + dec::ROWS - 1) / dec::ROWS;
  const int dense_steps = a.do_dense ? (ng + 1) / 2 : 0;      // two groups per dense step
  // MMA tiles of 8 tokens per CTA pass: 1 or 2 up to 16 tokens.  Beyond, passes of 16 tokens re-read the
  // weights from L2, which is cheap; one pass of 32 tokens (4 tiles) halves the number of steps but each
  // step is bound by instruction issue, so it only pays for 17..32 tokens on the large shapes (measured:
  // gate_up 36.2 -> 31.6 us, down 20.3 -> 18.6 us at 32 tokens; qkv and 48 tokens lose).
  static const int env_nt = getenv("W4A4_DECODE_NT") ? atoi(getenv("W4A4_DECODE_NT")) : 0;
  int nt = a.T > 8 ? 2 : 1;
  if (a.T > 16 && a.T <= 32 && (a.K >= 8192 || row_tiles >= dev->sm_count)) nt = 4;
  if (env_nt == 1 || env_nt == 2 || env_nt == 4) nt = env_nt;
  if (nt == 1 && a.T > 8) nt = 2;
  DecodePlan plan = plan_decode(a.T, a.N, dense_steps > 0 ? dense_steps : 1, dev->sm_count, dec::tokens_per_pass(nt));
  if ((long long)plan.row_tiles * plan.split > 2147483647LL)
    return fail(W4A4_ERR_UNSUPPORTED, "d_out=%d is too large", a.N);
  // expanded activations: given by the caller, or built here from the packed codes
  const void* XE = a.XE;
  const float* sumxf = a.sumxf;
  if (XE == nullptr) {
    const WsLayout wl = ws_layout(a.T, a.K);
    if (a.ws == nullptr || a.ws_bytes < wl.total)
      return fail(W4A4_ERR_WORKSPACE, "workspace of %zu bytes required, got %zu", wl.total, a.ws_bytes);
    char* ws = static_cast<char*>(a.ws);
    int rc = launch_expand(a, ws + wl.xe, reinterpret_cast<float*>(ws + wl.sumxf), dev);
    if (rc) return rc;
    XE = ws + wl.xe;
    sumxf = a.sum_X ? reinterpret_cast<float*>(ws + wl.sumxf) : nullptr;
  }
  if (!aligned(XE, 16)) return fail(W4A4_ERR_ALIGNMENT, "expanded activations must be 16-byte aligned");

  CUtensorMap tm_low;
  // dense weights: 128 rows x two groups (128 bytes) per copy, 16-byte chunks of a row stored at chunk ^ (row & 7);
  // unused (but valid) when the dense part is off
  int rc = make_map(&tm_low, a.do_dense ? a.W_low : a.W_high, a.do_dense ? (uint64_t)a.K / 2 : 64,
                    a.do_dense ? (uint64_t)a.N : (uint64_t)a.nnz * BROW, a.do_dense ? 2 * GROUP_BYTES : GROUP_BYTES,
                    dec::ROWS, a.do_dense ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc) return rc;

  dec::Params p;
  p.hp_row_offsets = a.hp_row_offsets;
  p.hp_col_indices = a.hp_col_indices;
  p.W_high = static_cast<const int8_t*>(a.W_high);
  p.XE = static_cast<const int8_t*>(XE);
  p.t_pad = xe_t_pad(a.T);
  p.scale_u4 = static_cast<const __half*>(a.scale_u4);
  p.zero_u4 = static_cast<const __half*>(a.zero_u4);
  p.sumxf = a.do_dense ? sumxf : nullptr;
  p.scale_x = static_cast<const __half*>(a.scale_x);
  p.Y = static_cast<__half*>(a.Y);
  if (a.flags & W4A4_FLAG_OUT_TOKEN_MAJOR) {
    p.y_stride_n = 1;
    p.y_stride_t = a.N;
  } else {
    p.y_stride_n = a.T;
    p.y_stride_t = 1;
  }
  p.acc_dump = a.acc_dump;
  p.acc_hi_dump = a.acc_hi_dump;
  p.T = a.T; p.K = a.K; p.N = a.N; p.ng = ng; p.nnz = has_sparse ? a.nnz : 0;
  p.row_tiles = row_tiles;
  p.nd = dense_steps;
  p.sparse_on = has_sparse ? 1 : 0;
  p.sz_vec = (ng % 8 == 0 && aligned(a.scale_u4, 16) && aligned(a.zero_u4, 16)) ? 1 : 0;
  p.split = plan.split;
  p.sparse_weight = has_sparse ? a.sparse_weight : 0.f;

  const size_t smem = dec::smem_bytes(nt);
  void (*kern)(const CUtensorMap, const dec::Params) =
      dump ? (nt == 4 ? dec::decode_gemm_kernel<4, true> : nt == 2 ? dec::decode_gemm_kernel<2, true> : dec::decode_gemm_kernel<1, true>)
           : (nt == 4 ? dec::decode_gemm_kernel<4, false> : nt == 2 ? dec::decode_gemm_kernel<2, false> : dec::decode_gemm_kernel<1, false>);
  cudaError_t e = launch_ex(kern, dim3(plan.row_tiles * plan.split, plan.tok_tiles, 1), dim3(dec::THREADS), smem, a.stream,
                plan.split, tm_low, p);
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "decode kernel launch: %s", cudaGetErrorString(e));
  return W4A4_OK;
}

// Packed weights read as e4m3 numbers by fp8 MMAs when the library expands the activation codes itself and
// the call carries their group sums: W4A4_PREFILL_F8=1.  Off by default: measured slower than the integer
// MMAs on s8 codes (gate_up, 4096 tokens: 1397 against 1175 us) - both are bound by the unpack warps'
// hand-over, and this form adds 16 KB of shared-memory stores per step.  Read on every call: tests compare
// the two in one process.
bool f8_on_packed() {
  const char* e = getenv("W4A4_PREFILL_F8");
  return e ? atoi(e) != 0 : false;
}

// True when the call carries prepared weights for every operand it uses.
bool has_prepared(const GemmArgs& a) {
  const bool has_sparse = a.nnz > 0 && a.sparse_weight != 0.f;
  return (!a.do_dense || a.W_low_prep != nullptr) && (!has_sparse || a.W_high_prep != nullptr) &&
         (a.W_low_prep != nullptr || a.W_high_prep != nullptr);
}

#ifdef W4A4_TRACE
static long long* g_trace_ptr = nullptr;
#endif
int launch_prefill(const GemmArgs& a_in, DeviceInfo* dev) {
  using namespace w4a4;
  GemmArgs a = a_in;
  const bool prep = has_prepared(a);
  // The expanded codes say which instantiation runs: e4m3 in natural order goes with prepared weights (fp8
  // MMAs on bytes as they land), e4m3 in even/odd order with packed weights read as e4m3 numbers (fp8
  // MMAs, see nib_lo_off8), s8 with packed weights widened to s8 (integer MMAs).  When the library expands
  // the codes itself it picks the e4m3 form that matches the weights; the integer instantiation remains for
  // callers' s8 codes and for calls that carry no activation group sums (the e4m3 form of packed weights
  // has an offset that only the sums can take out).
  const bool dump = a.acc_dump || a.acc_hi_dump;
  const bool has_sparse = a.nnz > 0 && a.sparse_weight != 0.f;
  if (a.XE == nullptr)
    a.xe_fmt = prep ? W4A4_CODES_E4M3
                    : ((dump ? (a.flags & W4A4_FLAG_CODES_E4M3_PACKED) != 0 : (a.sum_X != nullptr && f8_on_packed()))
                           ? W4A4_CODES_E4M3_PACKED : W4A4_CODES_S8);
  if (prep && a.xe_fmt != W4A4_CODES_E4M3)
    return fail(W4A4_ERR_BAD_ARG, "prepared weights need activation codes expanded as W4A4_CODES_E4M3 (W4A4_FLAG_CODES_E4M3)");
  if (!prep && a.xe_fmt == W4A4_CODES_E4M3)
    return fail(W4A4_ERR_BAD_ARG, "W4A4_CODES_E4M3 activation codes need prepared weights (w4a4_prepare_weights) for every "
                                  "operand in use; packed weights read W4A4_CODES_E4M3_PACKED or W4A4_CODES_S8");
  const bool f8 = a.xe_fmt != W4A4_CODES_S8;
  if (f8 && !prep && !dump && a.XE != nullptr && a.sumxf == nullptr)
    return fail(W4A4_ERR_BAD_ARG, "W4A4_CODES_E4M3_PACKED activation codes need the group sums (sumxf)");
  if (!a.do_dense && !has_sparse) return fail(W4A4_ERR_BAD_ARG, "neither a dense nor a residual operand was given");
  const int ng = a.K / BCOL;
  const int row_tiles = (a.N + pre::ROWS - 1) / pre::ROWS;
  const int tok_tiles = (a.T + pre::TN - 1) / pre::TN;
  if (tok_tiles > 65535) return fail(W4A4_ERR_UNSUPPORTED, "T=%d exceeds the grid limit of the tensor-core path", a.T);
  // expanded activations: given by the caller, or built here from the packed codes
  const void* XE = a.XE;
  const float* sumxf = a.sumxf;
  if (XE == nullptr) {
    const WsLayout wl = ws_layout(a.T, a.K);
    if (a.ws == nullptr || a.ws_bytes < wl.total)
      return fail(W4A4_ERR_WORKSPACE, "workspace of %zu bytes required, got %zu", wl.total, a.ws_bytes);
    char* ws = static_cast<char*>(a.ws);
    int rc = launch_expand(a, ws + wl.xe, reinterpret_cast<float*>(ws + wl.sumxf), dev);
    if (rc) return rc;
    XE = ws + wl.xe;
    sumxf = a.sum_X ? reinterpret_cast<float*>(ws + wl.sumxf) : nullptr;
  }
  if (!aligned(XE, 16)) return fail(W4A4_ERR_ALIGNMENT, "expanded activations must be 16-byte aligned");

  CUtensorMap tm_w, tm_wh;
  // the operand that is switched off borrows the other one's map and is never read.  Packed rows hold
  // two codes per byte and land under the 64-byte swizzle the unpack warps read; prepared rows hold one
  // code per byte and land under the 128-byte swizzle of an MMA operand tile.
  const void* w_lo = prep ? a.W_low_prep : a.W_low;
  const void* w_hi = prep ? a.W_high_prep : a.W_high;
  const uint64_t lo_row = prep ? (uint64_t)a.K : (uint64_t)a.K / 2, hi_row = prep ? BCOL : GROUP_BYTES;
  const uint32_t box = prep ? BCOL : GROUP_BYTES;
  const CUtensorMapSwizzle swz = prep ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  int rc = make_map(&tm_w, a.do_dense ? w_lo : w_hi, a.do_dense ? lo_row : hi_row,
                    a.do_dense ? (uint64_t)a.N : (uint64_t)a.nnz * BROW, box, pre::ROWS, swz);
  if (rc) return rc;
  rc = make_map(&tm_wh, has_sparse ? w_hi : w_lo, has_sparse ? hi_row : lo_row,
                has_sparse ? (uint64_t)a.nnz * BROW : (uint64_t)a.N, box, pre::ROWS, swz);
  if (rc) return rc;

  pre::Params p;
  p.hp_row_offsets = a.hp_row_offsets;
  p.hp_col_indices = a.hp_col_indices;
  p.XE = static_cast<const int8_t*>(XE);
  p.t_pad = xe_t_pad(a.T);
  p.scale_u4 = static_cast<const __half*>(a.scale_u4);
  p.zero_u4 = static_cast<const __half*>(a.zero_u4);
  p.sumxf = (a.do_dense || (f8 && !prep)) ? sumxf : nullptr;
  p.scale_x = static_cast<const __half*>(a.scale_x);
  p.Y = static_cast<__half*>(a.Y);
  if (a.flags & W4A4_FLAG_OUT_TOKEN_MAJOR) {
    p.y_stride_n = 1;
    p.y_stride_t = a.N;
  } else {
    p.y_stride_n = a.T;
    p.y_stride_t = 1;
  }
  p.acc_dump = a.acc_dump;
  p.acc_hi_dump = a.acc_hi_dump;
  p.T = a.T; p.K = a.K; p.N = a.N; p.ng = ng; p.nnz = has_sparse ? a.nnz : 0;
  p.nd = a.do_dense ? ng : 0;
  p.sparse_on = has_sparse ? 1 : 0;
  p.sz_vec = (ng % 8 == 0 && aligned(a.scale_u4, 16) && aligned(a.zero_u4, 16)) ? 1 : 0;
  p.sparse_weight = has_sparse ? a.sparse_weight : 0.f;
#ifdef W4A4_TRACE
  {
    static long long* g_trace = nullptr;
    if (!g_trace) { cudaMalloc(&g_trace, 16 * 64 * 8); }
    cudaMemsetAsync(g_trace, 0, 16 * 64 * 8, a.stream);
    p.trace = g_trace;
    p.trace_cta = getenv("W4A4_TRACE_CTA") ? atoi(getenv("W4A4_TRACE_CTA")) : 1000;
    g_trace_ptr = g_trace;
  }
#endif
  // W4A4_PREFILL_BAND overrides the band height of the CTA order (A/B runs)
  static const int env_band = getenv("W4A4_PREFILL_BAND") ? atoi(getenv("W4A4_PREFILL_BAND")) : 0;
  p.band = env_band > 0 ? env_band : 16;

  // CTA pairs (tcgen05 cta_group::2: two block-rows share one token tile, see prefill_pair_gemm.cuh) with
  // W4A4_PREFILL_PAIR=1.  Bit-identical outputs, 30 % less L2 -> SM traffic, but measured SLOWER than one CTA
  // per tile (Llama-3-8B shapes, 2048 / 8192 tokens: packed 0.20 against 0.225 of the 8-bit tensor peak,
  // prepared 0.23 against 0.29): the step time is set by the fold warps' accumulator round trip, which the
  // pair leaves unchanged, and every hand-over now crosses two SMs.  Kept selectable for A/B runs.
  const char* env_pair = getenv("W4A4_PREFILL_PAIR");
  const bool pair = env_pair && atoi(env_pair) != 0 && pp::supported(a.T, a.K, a.N) && (!f8 || prep);
  cudaError_t e;
  if (pair) {
    const size_t smem = pp::smem_bytes(prep);
    void (*kern)(const CUtensorMap, const CUtensorMap, const pre::Params) =
        prep ? (dump ? pp::prefill_pair_gemm_kernel<true, true, true> : pp::prefill_pair_gemm_kernel<false, true, true>)
             : (dump ? pp::prefill_pair_gemm_kernel<true, false, false> : pp::prefill_pair_gemm_kernel<false, false, false>);
    e = launch_ex(kern, dim3(2 * ((row_tiles + 1) / 2), tok_tiles, 1), dim3(pp::THREADS), smem, a.stream, 2, tm_w, tm_wh, p);
  } else {
    const size_t smem = pre::smem_bytes(f8, prep);
    void (*kern)(const CUtensorMap, const CUtensorMap, const pre::Params) =
        prep ? (dump ? pre::prefill_gemm_kernel<true, true, true> : pre::prefill_gemm_kernel<false, true, true>)
        : f8 ? (dump ? pre::prefill_gemm_kernel<true, true, false> : pre::prefill_gemm_kernel<false, true, false>)
             : (dump ? pre::prefill_gemm_kernel<true, false, false> : pre::prefill_gemm_kernel<false, false, false>);
    e = launch_ex(kern, dim3(row_tiles, tok_tiles, 1), dim3(pre::THREADS), smem, a.stream, 1, tm_w, tm_wh, p);
  }
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "prefill kernel launch: %s", cudaGetErrorString(e));
  return W4A4_OK;
}

int launch_quant(const void* X, long long ldx, const int32_t* perm, void* X_s4, void* scale_x, int32_t* sum_X,
                 void* XE, float* sumxf, int T, int K, cudaStream_t stream, int sm_count, int xe_fmt = 0,
                 int src = w4a4::SRC_PLAIN, const void* norm_w = nullptr, float eps = 0.f) {
  using namespace w4a4;
  QuantParams q;
  q.fmt = xe_fmt;
  q.norm_w = static_cast<const __half*>(norm_w);
  q.eps = eps;
  q.X = static_cast<const __half*>(X);
  q.ldx = ldx;
  q.perm = perm;
  q.X_s4 = static_cast<int8_t*>(X_s4);
  q.scale_x = static_cast<__half*>(scale_x);
  q.sum_X = sum_X;
  q.XE = static_cast<int8_t*>(XE);
  q.sumxf = sumxf;
  q.T = T;
  q.K = K;
  q.t_pad = xe_t_pad(T);
  q.vec_ok = (aligned(X, 16) && (ldx % 8 == 0)) ? 1 : 0;
  // few tokens: spread each token over a cluster so the row is read by many SMs at once
  int C = 1;
  const int ng = K / 128;
  for (int c = 8; c > 1; c >>= 1)
    if (ng % c == 0 && (long long)T * c <= 2LL * sm_count) { C = c; break; }
  q.C = C;
  size_t smem = (size_t)K * 2 / C;
  if (smem > QUANT_MAX_SMEM) return fail(W4A4_ERR_UNSUPPORTED, "K=%d exceeds the quantisation kernel's row buffer", K);
  // with a column permutation and one CTA per token the row is staged as it is and gathered while quantising
  q.stage_row = (perm != nullptr && C == 1) ? 1 : 0;
  // many tokens: smaller CTAs (see act_quant_kernel); W4A4_QUANT_THREADS=128|256 overrides (A/B runs)
  static const int env_nt = getenv("W4A4_QUANT_THREADS") ? atoi(getenv("W4A4_QUANT_THREADS")) : 0;
  // (measured, 8192 tokens: K = 4096 54 -> 44 us; K = 14336, where shared memory limits an SM to three CTAs, 194 -> 235 us)
  const bool small_cta = env_nt ? env_nt == 128 : (C == 1 && T >= 4 * sm_count && smem <= 32 * 1024);
  void (*kern)(const QuantParams) =
      src == SRC_RMSNORM    ? (small_cta ? act_quant_kernel<128, SRC_RMSNORM> : act_quant_kernel<QUANT_THREADS, SRC_RMSNORM>)
      : src == SRC_SILU_MUL ? (small_cta ? act_quant_kernel<128, SRC_SILU_MUL> : act_quant_kernel<QUANT_THREADS, SRC_SILU_MUL>)
                            : (small_cta ? act_quant_kernel<128> : act_quant_kernel<QUANT_THREADS>);
  cudaError_t e = launch_ex(kern, dim3((unsigned)((long long)T * C)), dim3(small_cta ? 128 : QUANT_THREADS), smem, stream, C, q);
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "quant kernel launch: %s", cudaGetErrorString(e));
  return W4A4_OK;
}

int check_common(int T, int K, int N, int nnz) {
  CHECK_ARG(T >= 1, "T must be >= 1, got %d", T);
  CHECK_ARG(K >= 128 && K % 128 == 0, "d_in (%d) must be a positive multiple of 128", K);
  CHECK_ARG(N >= 1, "d_out must be >= 1, got %d", N);
  CHECK_ARG(nnz >= 0, "nnz must be >= 0, got %d", nnz);
  CHECK_ARG((long long)T <= 16LL * 65535, "T=%d exceeds the grid limit", T);
  return W4A4_OK;
}

// Many tokens take the tcgen05 kernel, few the weight-streaming one.
bool wants_tensor_path(int T, int K, int N, int flags, int sm_count, bool prepared) {
  // W4A4_TENSOR_MIN_T moves the switch-over (A/B runs)
  static const int min_t = getenv("W4A4_TENSOR_MIN_T") ? atoi(getenv("W4A4_TENSOR_MIN_T")) : 0;
  bool tensor_path;
  if (min_t > 0) {
    tensor_path = T >= min_t;
  } else {
    // Cross-over between 64 and 255 tokens from a cost model fitted on B200 (quantisation included, us):
    // the streaming kernel re-reads the weights from L2 once per 32 tokens at ~2.4 TB/s; the tensor-core
    // kernel takes ~0.6 us (0.53 on prepared weights) per K-step of a 128 x 128 tile and wave of tiles.
    // It reproduces the measured winner on the Llama-3-8B shapes at 64, 96, 128 and 192 tokens.
    const long long tiles = (long long)((N + 127) / 128) * ((T + w4a4::pre::TN - 1) / w4a4::pre::TN);
    const double waves = (double)((tiles + sm_count - 1) / sm_count);
    const double stream_us = 10.0 + (double)((T + 31) / 32) * ((double)K * N / 2) / 2.4e6;
    const double tensor_us = 9.0 + waves * (K / 128) * (prepared ? 0.53 : 0.6);
    tensor_path = T >= 256 || (T >= 64 && tensor_us < stream_us);
  }
  tensor_path = tensor_path && w4a4::pre::supported(T, K, N);
  if (flags & W4A4_FLAG_FORCE_STREAM) tensor_path = false;
  if ((flags & W4A4_FLAG_FORCE_TENSOR) && w4a4::pre::supported(T, K, N)) tensor_path = true;
  return tensor_path;
}

int run_gemm(GemmArgs& a) {
  int rc = check_common(a.T, a.K, a.N, a.nnz);
  if (rc) return rc;
  CHECK_ARG(a.X_s4 != nullptr || a.XE != nullptr, "X_s4 is NULL");
  CHECK_ARG(a.scale_u4 != nullptr || (a.acc_dump || a.acc_hi_dump), "scale_u4 is NULL");
  CHECK_ARG(!a.do_dense || a.W_low != nullptr, "W_low is NULL");
  CHECK_ARG(a.nnz == 0 || (a.W_high && a.hp_row_offsets && a.hp_col_indices), "residual arrays are NULL with nnz=%d", a.nnz);
  if (!aligned(a.W_low, 16) || !aligned(a.W_high, 16))
    return fail(W4A4_ERR_ALIGNMENT, "weight pointers must be 16-byte aligned");
  if (!aligned(a.X_s4, 4)) return fail(W4A4_ERR_ALIGNMENT, "X_s4 must be 4-byte aligned");
  if ((long long)a.T > 16LL * 65535) return fail(W4A4_ERR_UNSUPPORTED, "T=%d exceeds the grid limit", a.T);
  DeviceInfo* dev = nullptr;
  rc = current_device(&dev);
  if (rc) return rc;
  if ((a.flags & W4A4_FLAG_FORCE_TENSOR) && !w4a4::pre::supported(a.T, a.K, a.N))
    return fail(W4A4_ERR_UNSUPPORTED, "tensor-core path does not support T=%d K=%d N=%d", a.T, a.K, a.N);
  if (!aligned(a.W_low_prep, 16) || !aligned(a.W_high_prep, 16))
    return fail(W4A4_ERR_ALIGNMENT, "weight pointers must be 16-byte aligned");
  // e4m3 codes exist only for the tensor-core kernel: such a call goes there whatever the token count
  if ((a.XE != nullptr && a.xe_fmt != 0) || ((a.acc_dump || a.acc_hi_dump) && (a.flags & W4A4_FLAG_CODES_E4M3_PACKED))) {
    if (a.flags & W4A4_FLAG_FORCE_STREAM) return fail(W4A4_ERR_BAD_ARG, "the streaming path reads s8 expanded codes");
    return launch_prefill(a, dev);
  }
  if (wants_tensor_path(a.T, a.K, a.N, a.flags, dev->sm_count, has_prepared(a))) return launch_prefill(a, dev);
  return launch_decode(a, dev);
}

// ------------------------------------------------------------------ built-in scratch
// Scratch for w4a4_fused_dense_sparse_noalloc: expanded activation codes of up to
// NOALLOC_MAX_T tokens of up to NOALLOC_MAX_K features, followed by their
// transposed group sums.  It lives in the library image, so every GPU that loads
// the library holds these 544 KiB (557 056 bytes) until the process exits.
constexpr int NOALLOC_MAX_T = W4A4_NOALLOC_MAX_T;
constexpr int NOALLOC_MAX_K = W4A4_NOALLOC_MAX_K;
constexpr size_t NOALLOC_XE_BYTES = (size_t)NOALLOC_MAX_T * NOALLOC_MAX_K + 128 * 128;
constexpr size_t NOALLOC_SUMS_BYTES = (size_t)(NOALLOC_MAX_K / 128) * 16 * sizeof(float);
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_XE_BYTES + NOALLOC_SUMS_BYTES];

// In host code `g_noalloc_scratch` is only a handle for the symbol, not an address
// a kernel can use.  The device address is looked up once per device, with that
// device current, and remembered.
void* g_noalloc_addr[64] = {};

int noalloc_scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return fail(W4A4_ERR_UNSUPPORTED, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_noalloc_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(W4A4_ERR_LAUNCH, "cudaGetSymbolAddress(built-in scratch): %s", cudaGetErrorString(e));
    g_noalloc_addr[dev] = p;
  }
  *out = g_noalloc_addr[dev];
  return W4A4_OK;
}

// Self-test of the bounded wait: one thread polls a barrier nobody ever arrives on (no copy
// in flight, nothing else running in the CTA), gives up after `polls` polls, records the
// error word like any production wait and returns.
constexpr int SITE_SELFTEST = 0x7e;
__global__ void selftest_wait_kernel(uint32_t polls) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    w4a4::mbar_init(&bar, 1);
    w4a4::mbar_fence_init();
    w4a4::mbar_wait_limit(&bar, 0, SITE_SELFTEST, polls);
  }
}

#ifdef W4A4_TRACE
long long* trace_ptr() { return g_trace_ptr; }
#endif
}  // namespace

#ifdef W4A4_TRACE
extern "C" int w4a4_debug_trace(long long* dst) {
  if (!trace_ptr()) return 1;
  return (int)cudaMemcpy(dst, trace_ptr(), 16 * 64 * 8, cudaMemcpyDeviceToHost);
}
#endif

// ===================================================================== C ABI
extern "C" {

int w4a4_abi_version(void) { return W4A4_ABI_VERSION; }

const char* w4a4_status_string(int status) {
  switch (status) {
    case W4A4_OK: return "ok";
    case W4A4_ERR_BAD_ARG: return "bad argument";
    case W4A4_ERR_ALIGNMENT: return "misaligned pointer or stride";
    case W4A4_ERR_WORKSPACE: return "workspace missing or too small";
    case W4A4_ERR_LAUNCH: return "CUDA launch error";
    case W4A4_ERR_DEVICE: return "device-side wait gave up";
    case W4A4_ERR_UNSUPPORTED: return "unsupported shape";
    default: return "unknown status";
  }
}

const char* w4a4_last_error(void) { return t_last_error.c_str(); }

int w4a4_device_error(int* word, void* stream) {
  begin_call();
  CHECK_ARG(word != nullptr, "word is NULL");
  int zero = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyFromSymbolAsync(word, w4a4::g_error_word, sizeof(int), 0, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaMemcpyToSymbolAsync(w4a4::g_error_word, &zero, sizeof(int), 0, cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "w4a4_device_error: %s", cudaGetErrorString(e));
  return *word ? W4A4_ERR_DEVICE : W4A4_OK;
}

int w4a4_selftest_bounded_wait(int polls, void* stream) {
  begin_call();
  CHECK_ARG(polls >= 1 && polls <= (1 << 20), "polls must be in 1..2^20, got %d", polls);
  selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>((uint32_t)polls);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "self-test kernel launch: %s", cudaGetErrorString(e));
  return W4A4_OK;
}

int w4a4_activation_quant(const void* X, long long ldx, const int32_t* perm, void* X_s4, void* scale_x,
                          int32_t* sum_X, int T, int K, void* stream) {
  begin_call();
  int rc = check_common(T, K, 1, 0);
  if (rc) return rc;
  CHECK_ARG(X && X_s4 && scale_x && sum_X, "NULL tensor pointer");
  CHECK_ARG(ldx >= K, "ldx (%lld) must be >= K (%d)", ldx, K);
  if (!aligned(X, 2) || !aligned(X_s4, 4) || !aligned(sum_X, 4) || !aligned(scale_x, 2))
    return fail(W4A4_ERR_ALIGNMENT, "activation_quant pointer alignment");
  DeviceInfo* dev = nullptr;
  rc = current_device(&dev);
  if (rc) return rc;
  return launch_quant(X, ldx, perm, X_s4, scale_x, sum_X, nullptr, nullptr, T, K, static_cast<cudaStream_t>(stream),
                      dev->sm_count);
}

namespace {
int fused_prologue_quant(int src, const void* X, long long ldx, long long min_ld, const void* norm_w, float eps,
                         const int32_t* perm, void* X_s4, void* scale_x, int32_t* sum_X, void* XE, float* sumxf,
                         int code_format, int T, int K, void* stream) {
  int rc = check_common(T, K, 1, 0);
  if (rc) return rc;
  CHECK_ARG(code_format == W4A4_CODES_S8 || code_format == W4A4_CODES_E4M3 || code_format == W4A4_CODES_E4M3_PACKED,
            "unknown code format %d", code_format);
  CHECK_ARG(X && scale_x, "NULL tensor pointer");
  CHECK_ARG((X_s4 != nullptr) == (sum_X != nullptr), "X_s4 and sum_X go together");
  CHECK_ARG((XE != nullptr) == (sumxf != nullptr), "XE and sumxf go together");
  CHECK_ARG(X_s4 || XE, "no output requested: pass X_s4 + sum_X, XE + sumxf, or both");
  CHECK_ARG(ldx >= min_ld, "row stride (%lld) must be >= %lld", ldx, min_ld);
  if (!aligned(X, 2) || !aligned(X_s4, 4) || !aligned(sum_X, 4) || !aligned(scale_x, 2) || !aligned(XE, 16) ||
      !aligned(sumxf, 16) || !aligned(norm_w, 2))
    return fail(W4A4_ERR_ALIGNMENT, "pointer alignment");
  DeviceInfo* dev = nullptr;
  rc = current_device(&dev);
  if (rc) return rc;
  return launch_quant(X, ldx, perm, X_s4, scale_x, sum_X, XE, sumxf, T, K, static_cast<cudaStream_t>(stream),
                      dev->sm_count, code_format, src, norm_w, eps);
}
}  // namespace

int w4a4_rmsnorm_quant(const void* X, long long ldx, const void* norm_weight, float eps, const int32_t* perm,
                       void* X_s4, void* scale_x, int32_t* sum_X, void* XE, float* sumxf, int code_format, int T,
                       int K, void* stream) {
  begin_call();
  CHECK_ARG(norm_weight != nullptr, "norm_weight is NULL");
  CHECK_ARG(eps >= 0.f, "eps must be >= 0");
  return fused_prologue_quant(w4a4::SRC_RMSNORM, X, ldx, K, norm_weight, eps, perm, X_s4, scale_x, sum_X, XE, sumxf,
                              code_format, T, K, stream);
}

int w4a4_silu_mul_quant(const void* GU, long long ldgu, const int32_t* perm, void* X_s4, void* scale_x,
                        int32_t* sum_X, void* XE, float* sumxf, int code_format, int T, int K, void* stream) {
  begin_call();
  return fused_prologue_quant(w4a4::SRC_SILU_MUL, GU, ldgu, 2LL * K, nullptr, 0.f, perm, X_s4, scale_x, sum_X, XE,
                              sumxf, code_format, T, K, stream);
}

// ------------------------------------------------------------------ output exchange over peer memory
int w4a4_peer_alloc(size_t bytes, void** ptr) {
  begin_call();
  CHECK_ARG(ptr != nullptr && bytes > 0, "bad arguments");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "w4a4_peer_alloc(%zu): %s", bytes, cudaGetErrorString(e));
  *ptr = p;
  return W4A4_OK;
}

int w4a4_peer_free(void* ptr) {
  begin_call();
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "w4a4_peer_free: %s", cudaGetErrorString(e));
  return W4A4_OK;
}

int w4a4_peer_export(const void* ptr, void* handle) {
  begin_call();
  CHECK_ARG(ptr && handle, "NULL pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle travels as 64 bytes");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(ptr));
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  memcpy(handle, &h, 64);
  return W4A4_OK;
}

int w4a4_peer_open(const void* handle, void** ptr) {
  begin_call();
  CHECK_ARG(ptr && handle, "NULL pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  *ptr = p;
  return W4A4_OK;
}

int w4a4_peer_close(void* ptr) {
  begin_call();
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
  return W4A4_OK;
}

int w4a4_peer_push_wait(const void* src, long long src_pitch, void* const* dst, void* const* flags, long long dst_pitch,
                        long long dst_offset, int rows, int row_bytes, int world, int rank, void* state, int poll_limit,
                        void* stream) {
  begin_call();
  CHECK_ARG(src && dst && flags && state, "NULL pointer");
  CHECK_ARG(world >= 1 && world <= w4a4::PEER_MAX_WORLD && rank >= 0 && rank < world, "world=%d rank=%d out of range", world, rank);
  CHECK_ARG(rows >= 1 && row_bytes >= 2 && row_bytes % 2 == 0, "rows=%d row_bytes=%d", rows, row_bytes);
  CHECK_ARG(src_pitch >= row_bytes && dst_pitch >= row_bytes && dst_offset >= 0, "pitches must cover a row");
  CHECK_ARG(poll_limit >= 1, "poll_limit must be >= 1");
  w4a4::PushParams p;
  memset(&p, 0, sizeof p);
  p.src = static_cast<const unsigned char*>(src);
  p.src_pitch = src_pitch;
  for (int i = 0; i < world; ++i) {
    CHECK_ARG(dst[i] && flags[i], "NULL peer pointer for rank %d", i);
    p.dst[i] = static_cast<unsigned char*>(dst[i]);
    p.flags[i] = static_cast<unsigned int*>(flags[i]);
  }
  p.dst_pitch = dst_pitch; p.dst_offset = dst_offset; p.rows = rows; p.row_bytes = row_bytes;
  p.world = world; p.rank = rank; p.state = static_cast<unsigned int*>(state); p.poll_limit = (unsigned int)poll_limit;
  // enough blocks per destination to keep the links busy on large shards, one for a decode-sized shard
  const long long bytes = (long long)rows * row_bytes;
  int bpd = (int)((bytes + (64 << 10) - 1) / (64 << 10));
  DeviceInfo* dev = nullptr;
  int rc = current_device(&dev);
  if (rc) return rc;
  const int cap = (2 * dev->sm_count) / world > 0 ? (2 * dev->sm_count) / world : 1;
  if (bpd > cap) bpd = cap;
  if (bpd < 1) bpd = 1;
  p.blocks_per_dst = bpd;
  cudaError_t e = launch_ex(w4a4::peer_push_wait_kernel, dim3((unsigned)(bpd * world)), dim3(256), 0,
                            static_cast<cudaStream_t>(stream), 1, p);
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "peer push kernel launch: %s", cudaGetErrorString(e));
  return W4A4_OK;
}

size_t w4a4_workspace_bytes(int T, int K, int N, int nnz) {
  (void)N;
  (void)nnz;
  if (T < 1 || K < 128) return 0;
  return ws_layout(T, K).total;
}

int w4a4_fused_dense_sparse(const void* W_low, const void* W_high, const int32_t* hp_row_offsets,
                            const int32_t* hp_col_indices, const void* X_s4, const void* scale_u4,
                            const void* zero_u4, const int32_t* sum_X, const void* scale_x, void* Y, int T, int K,
                            int N, int nnz, int flags, void* workspace, size_t workspace_bytes, void* stream) {
  return w4a4_fused_dense_sparse_prepared(W_low, W_high, nullptr, nullptr, hp_row_offsets, hp_col_indices, X_s4, scale_u4,
                                          zero_u4, sum_X, scale_x, Y, T, K, N, nnz, flags, workspace, workspace_bytes,
                                          stream);
}

int w4a4_dequant_weights_fp16(const void* W_low, const void* scale_u4, const void* zero_u4, void* out_fp16, int N, int K,
                              void* stream) {
  begin_call();
  int rc = check_common(1, K, N, 0);
  if (rc) return rc;
  CHECK_ARG(W_low && scale_u4 && zero_u4 && out_fp16, "NULL tensor pointer");
  if (!aligned(W_low, 4) || !aligned(out_fp16, 16) || !aligned(scale_u4, 2) || !aligned(zero_u4, 2))
    return fail(W4A4_ERR_ALIGNMENT, "dequant_weights pointer alignment");
  DeviceInfo* dev = nullptr;
  rc = current_device(&dev);
  if (rc) return rc;
  const long long words = (long long)N * (K / 8);
  long long blocks = (words + 255) / 256;
  if (blocks > 16LL * dev->sm_count) blocks = 16LL * dev->sm_count;
  w4a4::dequant_weights_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(W_low), static_cast<const __half*>(scale_u4), static_cast<const __half*>(zero_u4),
      static_cast<uint4*>(out_fp16), N, K);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "dequant_weights kernel launch: %s", cudaGetErrorString(e));
  return W4A4_OK;
}

size_t w4a4_prepared_weights_bytes(size_t packed_bytes) { return 2 * packed_bytes; }

int w4a4_prepare_weights(const void* packed, void* prepared, size_t packed_bytes, void* stream) {
  begin_call();
  CHECK_ARG(packed && prepared, "NULL tensor pointer");
  CHECK_ARG(packed_bytes % 4 == 0, "packed_bytes (%zu) must be a multiple of 4", packed_bytes);
  if (!aligned(packed, 4) || !aligned(prepared, 16)) return fail(W4A4_ERR_ALIGNMENT, "prepare_weights pointer alignment");
  if (packed_bytes == 0) return W4A4_OK;
  DeviceInfo* dev = nullptr;
  int rc = current_device(&dev);
  if (rc) return rc;
  const long long words = (long long)(packed_bytes / 4);
  long long blocks = (words + 255) / 256;
  if (blocks > 16LL * dev->sm_count) blocks = 16LL * dev->sm_count;
  w4a4::prepare_weights_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(packed), static_cast<uint2*>(prepared), words);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "prepare_weights kernel launch: %s", cudaGetErrorString(e));
  return W4A4_OK;
}

int w4a4_fused_dense_sparse_prepared(const void* W_low, const void* W_high, const void* W_low_prepared,
                                     const void* W_high_prepared, const int32_t* hp_row_offsets,
                                     const int32_t* hp_col_indices, const void* X_s4, const void* scale_u4,
                                     const void* zero_u4, const int32_t* sum_X, const void* scale_x, void* Y, int T,
                                     int K, int N, int nnz, int flags, void* workspace, size_t workspace_bytes,
                                     void* stream) {
  begin_call();
  CHECK_ARG(Y && zero_u4 && sum_X && scale_x, "NULL tensor pointer");
  GemmArgs a{};
  a.W_low_prep = W_low_prepared; a.W_high_prep = W_high_prepared;
  a.W_low = W_low; a.W_high = W_high; a.hp_row_offsets = hp_row_offsets; a.hp_col_indices = hp_col_indices;
  a.X_s4 = X_s4; a.scale_u4 = scale_u4; a.zero_u4 = zero_u4; a.sum_X = sum_X; a.scale_x = scale_x; a.Y = Y;
  a.T = T; a.K = K; a.N = N; a.nnz = nnz; a.flags = flags;
  a.do_dense = true; a.sparse_weight = 16.f;
  a.ws = workspace; a.ws_bytes = workspace_bytes; a.stream = static_cast<cudaStream_t>(stream);
  return run_gemm(a);
}

size_t w4a4_expanded_codes_bytes(int T, int K) { return (T < 1 || K < 128) ? 0 : xe_bytes(T, K); }
size_t w4a4_expanded_sums_bytes(int T, int K) {
  return (T < 1 || K < 128) ? 0 : (size_t)((T + 15) / 16) * (K / 128) * 16 * 4;
}

int w4a4_expand_activations(const void* X_s4, const int32_t* sum_X, void* XE, float* sumxf, int T, int K,
                            void* stream) {
  return w4a4_expand_activations_fmt(X_s4, sum_X, XE, sumxf, T, K, W4A4_CODES_S8, stream);
}

int w4a4_expand_activations_fmt(const void* X_s4, const int32_t* sum_X, void* XE, float* sumxf, int T, int K,
                                int code_format, void* stream) {
  begin_call();
  CHECK_ARG(code_format == W4A4_CODES_S8 || code_format == W4A4_CODES_E4M3 || code_format == W4A4_CODES_E4M3_PACKED,
            "unknown code format %d", code_format);
  int rc = check_common(T, K, 1, 0);
  if (rc) return rc;
  CHECK_ARG(X_s4 && XE && (sum_X == nullptr || sumxf != nullptr), "NULL tensor pointer");
  if (!aligned(X_s4, 4) || !aligned(XE, 16) || !aligned(sumxf, 16))
    return fail(W4A4_ERR_ALIGNMENT, "expand_activations pointer alignment");
  DeviceInfo* dev = nullptr;
  rc = current_device(&dev);
  if (rc) return rc;
  GemmArgs a{};
  a.X_s4 = X_s4; a.sum_X = sum_X; a.T = T; a.K = K; a.stream = static_cast<cudaStream_t>(stream);
  a.xe_fmt = code_format;
  return launch_expand(a, XE, sumxf, dev);
}

int w4a4_fused_dense_sparse_expanded(const void* W_low, const void* W_high, const int32_t* hp_row_offsets,
                                     const int32_t* hp_col_indices, const void* XE, const float* sumxf,
                                     const void* scale_u4, const void* zero_u4, const void* scale_x, void* Y, int T,
                                     int K, int N, int nnz, int flags, void* workspace, size_t workspace_bytes,
                                     void* stream) {
  return w4a4_fused_dense_sparse_expanded_prepared(W_low, W_high, nullptr, nullptr, hp_row_offsets, hp_col_indices, XE,
                                                   sumxf, scale_u4, zero_u4, scale_x, Y, T, K, N, nnz, flags, workspace,
                                                   workspace_bytes, stream);
}

int w4a4_fused_dense_sparse_expanded_prepared(const void* W_low, const void* W_high, const void* W_low_prepared,
                                              const void* W_high_prepared, const int32_t* hp_row_offsets,
                                              const int32_t* hp_col_indices, const void* XE, const float* sumxf,
                                              const void* scale_u4, const void* zero_u4, const void* scale_x,
                                              void* Y, int T, int K, int N, int nnz, int flags, void* workspace,
                                              size_t workspace_bytes, void* stream) {
  begin_call();
  CHECK_ARG(Y && zero_u4 && XE && sumxf && scale_x, "NULL tensor pointer");
  GemmArgs a{};
  a.W_low_prep = W_low_prepared; a.W_high_prep = W_high_prepared;
  a.do_dense = true; a.nnz = nnz; a.sparse_weight = 16.f;
  // The caller says which bytes XE holds.  Natural-order e4m3 codes are read only against prepared weights,
  // even/odd-order e4m3 codes and s8 codes only against the packed arrays; a mismatch is an error rather than
  // a silent reinterpretation of the bytes.
  CHECK_ARG((flags & W4A4_FLAG_CODES_E4M3) == 0 || (flags & W4A4_FLAG_CODES_E4M3_PACKED) == 0,
            "W4A4_FLAG_CODES_E4M3 and W4A4_FLAG_CODES_E4M3_PACKED exclude each other");
  a.xe_fmt = (flags & W4A4_FLAG_CODES_E4M3) ? W4A4_CODES_E4M3
             : (flags & W4A4_FLAG_CODES_E4M3_PACKED) ? W4A4_CODES_E4M3_PACKED : W4A4_CODES_S8;
  if (!has_prepared(a)) a.W_low_prep = a.W_high_prep = nullptr;
  if (has_prepared(a) && a.xe_fmt != W4A4_CODES_E4M3)
    return fail(W4A4_ERR_BAD_ARG, "prepared weights were passed with activation codes for packed weights: expand with "
                                  "W4A4_CODES_E4M3 and set W4A4_FLAG_CODES_E4M3, or pass NULL prepared pointers");
  a.W_low = W_low; a.W_high = W_high; a.hp_row_offsets = hp_row_offsets; a.hp_col_indices = hp_col_indices;
  a.XE = XE; a.sumxf = sumxf; a.scale_u4 = scale_u4; a.zero_u4 = zero_u4; a.scale_x = scale_x; a.Y = Y;
  a.T = T; a.K = K; a.N = N; a.nnz = nnz; a.flags = flags;
  a.do_dense = true; a.sparse_weight = 16.f;
  a.ws = workspace; a.ws_bytes = workspace_bytes; a.stream = static_cast<cudaStream_t>(stream);
  return run_gemm(a);
}

int w4a4_dense_gemm(const void* W_low, const void* X_s4, const void* scale_u4, const void* zero_u4,
                    const int32_t* sum_X, const void* scale_x, void* Y_low, int T, int K, int N, int flags,
                    void* workspace, size_t workspace_bytes, void* stream) {
  begin_call();
  CHECK_ARG(Y_low && zero_u4 && sum_X && scale_x, "NULL tensor pointer");
  GemmArgs a{};
  a.W_low = W_low; a.X_s4 = X_s4; a.scale_u4 = scale_u4; a.zero_u4 = zero_u4; a.sum_X = sum_X;
  a.scale_x = scale_x; a.Y = Y_low;
  a.T = T; a.K = K; a.N = N; a.nnz = 0; a.flags = flags;
  a.do_dense = true; a.sparse_weight = 0.f;
  a.ws = workspace; a.ws_bytes = workspace_bytes; a.stream = static_cast<cudaStream_t>(stream);
  return run_gemm(a);
}

int w4a4_sparse_gemm(const void* W_high, const int32_t* hp_row_offsets, const int32_t* hp_col_indices,
                     const void* X_s4, const void* scale_u4, const void* scale_x, void* Y_high, int T, int K, int N,
                     int nnz, int flags, void* workspace, size_t workspace_bytes, void* stream) {
  begin_call();
  CHECK_ARG(Y_high && scale_x, "NULL tensor pointer");
  {
    // block-rows without blocks are never visited by the kernel: they are zero
    // (an empty block-CSR gives an all-zero product, cuda_kernel/ops.py:367-369)
    int rc0 = check_common(T, K, N, nnz);
    if (rc0) return rc0;
    cudaError_t e = cudaMemsetAsync(Y_high, 0, (size_t)N * T * 2, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "cudaMemsetAsync: %s", cudaGetErrorString(e));
    if (nnz == 0) return W4A4_OK;
  }
  GemmArgs a{};
  a.W_high = W_high; a.hp_row_offsets = hp_row_offsets; a.hp_col_indices = hp_col_indices;
  a.X_s4 = X_s4; a.scale_u4 = scale_u4; a.scale_x = scale_x; a.Y = Y_high;
  a.T = T; a.K = K; a.N = N; a.nnz = nnz; a.flags = flags;
  a.do_dense = false; a.sparse_weight = 1.f;
  a.ws = workspace; a.ws_bytes = workspace_bytes; a.stream = static_cast<cudaStream_t>(stream);
  return run_gemm(a);
}

int w4a4_fused_quant_dense_sparse(const void* X, long long ldx, const int32_t* perm, const void* W_low,
                                  const void* W_high, const int32_t* hp_row_offsets, const int32_t* hp_col_indices,
                                  const void* scale_u4, const void* zero_u4, void* Y, int T, int K, int N, int nnz,
                                  int flags, void* workspace, size_t workspace_bytes, void* stream) {
  return w4a4_fused_quant_dense_sparse_prepared(X, ldx, perm, W_low, W_high, nullptr, nullptr, hp_row_offsets,
                                                hp_col_indices, scale_u4, zero_u4, Y, T, K, N, nnz, flags, workspace,
                                                workspace_bytes, stream);
}

int w4a4_fused_quant_dense_sparse_prepared(const void* X, long long ldx, const int32_t* perm, const void* W_low,
                                           const void* W_high, const void* W_low_prepared,
                                           const void* W_high_prepared, const int32_t* hp_row_offsets,
                                           const int32_t* hp_col_indices, const void* scale_u4, const void* zero_u4,
                                           void* Y, int T, int K, int N, int nnz, int flags, void* workspace,
                                           size_t workspace_bytes, void* stream) {
  begin_call();
  int rc = check_common(T, K, N, nnz);
  if (rc) return rc;
  CHECK_ARG(X && Y && zero_u4, "NULL tensor pointer");
  CHECK_ARG(ldx >= K, "ldx (%lld) must be >= K (%d)", ldx, K);
  const WsLayout wl = ws_layout(T, K);
  if (workspace == nullptr || workspace_bytes < wl.total)
    return fail(W4A4_ERR_WORKSPACE, "workspace of %zu bytes required, got %zu", wl.total, workspace_bytes);
  char* ws = static_cast<char*>(workspace);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  DeviceInfo* dev = nullptr;
  rc = current_device(&dev);
  if (rc) return rc;
  GemmArgs a{};
  a.W_low = W_low; a.W_high = W_high; a.hp_row_offsets = hp_row_offsets; a.hp_col_indices = hp_col_indices;
  a.nnz = nnz; a.do_dense = true; a.sparse_weight = 16.f;
  // the quantiser writes the codes in the format the GEMM kernel of this call will read
  a.W_low_prep = W_low_prepared; a.W_high_prep = W_high_prepared;
  const bool tensor = wants_tensor_path(T, K, N, flags, dev->sm_count, has_prepared(a));
  if (!tensor || !has_prepared(a)) a.W_low_prep = a.W_high_prep = nullptr;
  // the tensor-core kernel runs fp8 MMAs on e4m3 codes (natural order against prepared weights, even/odd
  // order against packed ones); the streaming kernel reads s8 codes
  a.xe_fmt = !tensor ? W4A4_CODES_S8
             : has_prepared(a) ? W4A4_CODES_E4M3 : (f8_on_packed() ? W4A4_CODES_E4M3_PACKED : W4A4_CODES_S8);
  rc = launch_quant(X, ldx, perm, nullptr, ws + wl.scale_x, nullptr, ws + wl.xe, reinterpret_cast<float*>(ws + wl.sumxf),
                    T, K, s, dev->sm_count, a.xe_fmt);
  if (rc) return rc;
  a.XE = ws + wl.xe; a.sumxf = reinterpret_cast<float*>(ws + wl.sumxf); a.scale_u4 = scale_u4; a.zero_u4 = zero_u4;
  a.scale_x = ws + wl.scale_x; a.Y = Y;
  a.T = T; a.K = K; a.N = N; a.nnz = nnz; a.flags = flags;
  a.do_dense = true; a.sparse_weight = 16.f;
  a.ws = workspace; a.ws_bytes = workspace_bytes; a.stream = s;
  return run_gemm(a);
}

int w4a4_dump_accumulators(const void* W_low, const void* W_high, const int32_t* hp_row_offsets,
                           const int32_t* hp_col_indices, const void* X_s4, int32_t* acc, int32_t* acc_hi, int T,
                           int K, int N, int nnz, int flags, void* workspace, size_t workspace_bytes, void* stream) {
  return w4a4_dump_accumulators_prepared(W_low, W_high, nullptr, nullptr, hp_row_offsets, hp_col_indices, X_s4, acc,
                                         acc_hi, T, K, N, nnz, flags, workspace, workspace_bytes, stream);
}

int w4a4_dump_accumulators_prepared(const void* W_low, const void* W_high, const void* W_low_prepared,
                                    const void* W_high_prepared, const int32_t* hp_row_offsets,
                                    const int32_t* hp_col_indices, const void* X_s4, int32_t* acc, int32_t* acc_hi,
                                    int T, int K, int N, int nnz, int flags, void* workspace, size_t workspace_bytes,
                                    void* stream) {
  begin_call();
  CHECK_ARG(acc || acc_hi, "both outputs are NULL");
  GemmArgs a{};
  a.W_low_prep = acc ? W_low_prepared : nullptr; a.W_high_prep = (acc_hi && nnz > 0) ? W_high_prepared : nullptr;
  a.W_low = W_low; a.W_high = W_high; a.hp_row_offsets = hp_row_offsets; a.hp_col_indices = hp_col_indices;
  a.X_s4 = X_s4; a.acc_dump = acc; a.acc_hi_dump = acc_hi;
  a.T = T; a.K = K; a.N = N; a.nnz = acc_hi ? nnz : 0; a.flags = flags;
  a.do_dense = acc != nullptr; a.sparse_weight = 16.f;
  a.ws = workspace; a.ws_bytes = workspace_bytes; a.stream = static_cast<cudaStream_t>(stream);
  return run_gemm(a);
}

int w4a4_fused_dense_sparse_noalloc(const void* W_low, const void* W_high, const int32_t* hp_row_offsets,
                                    const int32_t* hp_col_indices, const void* X_s4, const void* scale_u4,
                                    const void* zero_u4, const int32_t* sum_X, const void* scale_x, void* Y, int T,
                                    int K, int N, int nnz, int flags, void* stream) {
  begin_call();
  int rc = check_common(T, K, N, nnz);
  if (rc) return rc;
  CHECK_ARG(Y && X_s4 && zero_u4 && sum_X && scale_x, "NULL tensor pointer");
  if (T > NOALLOC_MAX_T || K > NOALLOC_MAX_K)
    return fail(W4A4_ERR_UNSUPPORTED,
                "T=%d, K=%d exceed the built-in scratch of w4a4_fused_dense_sparse_noalloc (T <= %d, K <= %d); "
                "use w4a4_fused_dense_sparse with a caller-provided workspace",
                T, K, NOALLOC_MAX_T, NOALLOC_MAX_K);
  if (!aligned(X_s4, 4)) return fail(W4A4_ERR_ALIGNMENT, "X_s4 must be 4-byte aligned");
  // this entry point always runs the weight-streaming kernel on s8 codes it expands itself
  CHECK_ARG((flags & (W4A4_FLAG_FORCE_TENSOR | W4A4_FLAG_CODES_E4M3 | W4A4_FLAG_CODES_E4M3_PACKED)) == 0,
            "w4a4_fused_dense_sparse_noalloc accepts neither W4A4_FLAG_FORCE_TENSOR nor W4A4_FLAG_CODES_E4M3[_PACKED]");
  void* scratch = nullptr;
  rc = noalloc_scratch_address(&scratch);      // first call on a device resolves the address
  if (rc) return rc;
  DeviceInfo* dev = nullptr;
  rc = current_device(&dev);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* xe = static_cast<char*>(scratch);
  float* sums = reinterpret_cast<float*>(xe + NOALLOC_XE_BYTES);
  // The array keeps whatever the previous call left.  The codes of the T live
  // tokens are overwritten below and rows past T are never read; the group sums of
  // the token tile are cleared so that no stale lane of an earlier call is read.
  cudaError_t e = cudaMemsetAsync(sums, 0, (size_t)(K / 128) * 16 * sizeof(float), s);
  if (e != cudaSuccess) return fail(W4A4_ERR_LAUNCH, "cudaMemsetAsync(built-in scratch): %s", cudaGetErrorString(e));
  GemmArgs x{};
  x.X_s4 = X_s4; x.sum_X = sum_X; x.T = T; x.K = K; x.stream = s;
  rc = launch_expand(x, xe, sums, dev);
  if (rc) return rc;
  GemmArgs a{};
  a.W_low = W_low; a.W_high = W_high; a.hp_row_offsets = hp_row_offsets; a.hp_col_indices = hp_col_indices;
  a.XE = xe; a.sumxf = sums; a.scale_u4 = scale_u4; a.zero_u4 = zero_u4; a.scale_x = scale_x; a.Y = Y;
  a.T = T; a.K = K; a.N = N; a.nnz = nnz; a.flags = flags | W4A4_FLAG_FORCE_STREAM;
  a.do_dense = true; a.sparse_weight = 16.f;
  a.ws = nullptr; a.ws_bytes = 0; a.stream = s;
  return run_gemm(a);
}

}  // extern "C"
