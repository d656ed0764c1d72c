/*
 * C ABI of the B200 (sm_100a) W4A4 fused-linear library  (libw4a4_b200.so).
 *
 * These entry points are what the reference project's operator layer would bind
 * in place of its pybind11 module `hkust_v9_cuda`
 * (cuda_kernel/csrc/bindings.cc:110-252, called from cuda_kernel/ops.py).
 * Plain pointers and sizes only; all pointers are DEVICE pointers unless a
 * comment says host.  Every call is stream-ordered on `stream` (a cudaStream_t
 * passed as void*), never synchronises, and never allocates: scratch memory is
 * passed in by the caller (query its size with w4a4_workspace_bytes).  Inputs
 * are borrowed until the stream work completes.
 *
 * Shapes: T tokens, K = d_in (multiple of 128), N = d_out (any), ng = K/128,
 * nnz residual blocks.  Tensors are dense row-major:
 *   X        (T, K)  fp16, row stride ldx elements
 *   perm     (K)     int32 or NULL for identity
 *   X_s4     (T, K/2) int8   two codes per byte, even element in the low nibble
 *   scale_x  (T)     fp16
 *   sum_X    (T, ng) int32
 *   W_low    (N, K/2) int8   nibbles = u4 - 8
 *   W_high   (nnz, 128, 64) int8
 *   scale_u4, zero_u4 (N, ng) fp16   (zero already shifted by -8)
 *   hp_row_offsets (ceil(N/128)+1) int32, hp_col_indices (nnz) int32
 *   Y        (N, T) fp16, or (T, N) with W4A4_FLAG_OUT_TOKEN_MAJOR
 *
 * Return value: 0 on success, otherwise one of the W4A4_ERR_* codes;
 * w4a4_last_error() gives a host-side message for the calling thread.
 */
#ifndef W4A4_B200_H_
#define W4A4_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define W4A4_ABI_VERSION 1

enum {
  W4A4_OK = 0,
  W4A4_ERR_BAD_ARG = 1,      /* null pointer, bad size, K % 128 != 0 ...           */
  W4A4_ERR_ALIGNMENT = 2,    /* a pointer or stride misses the alignment it needs  */
  W4A4_ERR_WORKSPACE = 3,    /* workspace NULL or smaller than w4a4_workspace_bytes */
  W4A4_ERR_LAUNCH = 4,       /* CUDA reported an error at launch                   */
  W4A4_ERR_DEVICE = 5,       /* a bounded device-side wait gave up (see w4a4_device_error) */
  W4A4_ERR_UNSUPPORTED = 6   /* shape outside what the selected kernel supports    */
};

/* flags for the GEMM entry points */
#define W4A4_FLAG_OUT_TOKEN_MAJOR 0x1  /* write Y as (T, N) instead of (N, T)          */
#define W4A4_FLAG_FORCE_STREAM    0x2  /* force the weight-streaming split-K kernel     */
#define W4A4_FLAG_FORCE_TENSOR    0x4  /* force the tcgen05 tensor-core kernel          */
#define W4A4_FLAG_CODES_E4M3      0x8  /* *_expanded entry points: XE holds W4A4_CODES_E4M3 bytes (for prepared weights) */
#define W4A4_FLAG_CODES_E4M3_PACKED 0x10 /* *_expanded entry points: XE holds W4A4_CODES_E4M3_PACKED bytes (for packed
                                            weights); w4a4_dump_accumulators: run the fp8 instantiation on packed weights */

int w4a4_abi_version(void);
const char* w4a4_status_string(int status);
const char* w4a4_last_error(void);

/* Reads and clears the device error word of the current device (synchronises
 * `stream`).  *word == 0 means no bounded wait has given up since the last call. */
int w4a4_device_error(int* word /* host */, void* stream);

/* Self-test of the bounded device-side waits (no counterpart in the reference): launches a
 * one-CTA kernel in which one thread waits on a barrier nobody arrives on, gives up after
 * `polls` polls (1..2^20), records the device error word and returns normally.  A later
 * w4a4_device_error then returns W4A4_ERR_DEVICE with word = 0x40000000 | (0x7e << 8), and the
 * context stays usable. */
int w4a4_selftest_bounded_wait(int polls, void* stream);

/* Replaces activation_quant_launch (bindings.cc:113-122; kernel
 * cuda_kernel/csrc/activation_quant/activation_quant.cu:699-865).
 * No workspace. */
int w4a4_activation_quant(const void* X, long long ldx, const int32_t* perm, void* X_s4,
                          void* scale_x, int32_t* sum_X, int T, int K, void* stream);

/* Quantisation fused with the element-wise step that precedes it in a decoder layer, so that the
 * intermediate fp16 activations never travel through memory and a linear costs two launches (this
 * one and the GEMM on the expanded codes).  They remove the seam the reference leaves between its
 * PyTorch glue and activation_quant (triton_kernel/v9_linear.py:106-170 on the output side; on the
 * input side the reference has no fused form).  Outputs as w4a4_activation_quant (X_s4 + sum_X,
 * may both be NULL) and/or the expanded layout (XE + sumxf, may both be NULL; code_format as
 * w4a4_expand_activations_fmt; sizes from w4a4_expanded_codes_bytes / _sums_bytes; sumxf must be
 * zero-initialised when T is not a multiple of 16); scale_x always.
 *
 * w4a4_rmsnorm_quant quantises  y[t,k] = fp16( fp16( x[t,k] * r[t] ) * w[k] ),
 *   r[t] = 1 / sqrt( fp32( sum_k x[t,k]^2 / K ) + eps )   (sum exact, IEEE sqrt and division).
 * w4a4_silu_mul_quant reads rows [gate (K) | up (K)] (ldgu >= 2K) and quantises
 *   y[t,k] = fp16( fp16( silu(gate[t,k]) ) * up[t,k] ),  silu(g) = g / (1 + exp(-g)). */
int w4a4_rmsnorm_quant(const void* X, long long ldx, const void* norm_weight, float eps, const int32_t* perm,
                       void* X_s4, void* scale_x, int32_t* sum_X, void* XE, float* sumxf, int code_format, int T,
                       int K, void* stream);
int w4a4_silu_mul_quant(const void* GU, long long ldgu, const int32_t* perm, void* X_s4, void* scale_x,
                        int32_t* sum_X, void* XE, float* sumxf, int code_format, int T, int K, void* stream);

/* Scratch bytes the GEMM entry points below need for (T, K, N, nnz); the same
 * size serves all of them.  The scratch holds the activations in the layout the
 * kernels read (expanded codes, transposed group sums, and the per-token scales
 * when the library quantises); its contents need no initialisation and calls
 * that share one scratch buffer must be ordered on one stream. */
size_t w4a4_workspace_bytes(int T, int K, int N, int nnz);

/* Replaces fused_dense_sparse_mma_int4_launch, fused_gemv_decode_launch and
 * fused_gemv_smallT_launch (bindings.cc:187-235; kernels
 * fused_dense_sparse_mma_int4.cu:184-1190, fused_gemv_decode.cu:54-191,
 * fused_gemv_smallT.cu:47-221).  nnz may be 0 (W_high/hp_col_indices then unused). */
int w4a4_fused_dense_sparse(const void* W_low, const void* W_high, const int32_t* hp_row_offsets,
                            const int32_t* hp_col_indices, const void* X_s4, const void* scale_u4,
                            const void* zero_u4, const int32_t* sum_X, const void* scale_x, void* Y,
                            int T, int K, int N, int nnz, int flags, void* workspace,
                            size_t workspace_bytes, void* stream);

/* Activations in the layout the GEMM kernels consume ("expanded"): XE, one int8
 * per code, group-major [K/128][T rounded up to 16][128 bytes] (+ slack; ask
 * w4a4_expanded_codes_bytes for the size): the 128 bytes of one (group, token)
 * hold the group's packed words in order, each 32-bit word of X_s4 turned into
 * its four even-indexed codes followed by its four odd-indexed ones, with the
 * line's eight 16-byte chunks stored at chunk ^ (token & 7); sumxf
 * [ceil(T/16)][K/128][16] float = sum_X transposed per 16-token tile.
 * w4a4_fused_dense_sparse builds both internally on every call; a caller that
 * feeds several linears from one activation (q/k/v, gate/up) can build them once
 * with w4a4_expand_activations and call w4a4_fused_dense_sparse_expanded.  No
 * counterpart in the reference's bindings (its kernels read X_s4 directly). */
size_t w4a4_expanded_codes_bytes(int T, int K);
size_t w4a4_expanded_sums_bytes(int T, int K);
int w4a4_expand_activations(const void* X_s4, const int32_t* sum_X, void* XE, float* sumxf, int T, int K,
                            void* stream);
int w4a4_fused_dense_sparse_expanded(const void* W_low, const void* W_high, const int32_t* hp_row_offsets,
                                     const int32_t* hp_col_indices, const void* XE, const float* sumxf,
                                     const void* scale_u4, const void* zero_u4, const void* scale_x, void* Y,
                                     int T, int K, int N, int nnz, int flags, void* workspace,
                                     size_t workspace_bytes, void* stream);

/* Replaces dense_gemm_mma_int4_launch and dense_gemv_decode_launch
 * (bindings.cc:124-148; dense_gemm_mma_int4.cu:39-431, dense_gemv_decode.cu:86-182). */
int w4a4_dense_gemm(const void* W_low, const void* X_s4, const void* scale_u4, const void* zero_u4,
                    const int32_t* sum_X, const void* scale_x, void* Y_low, int T, int K, int N,
                    int flags, void* workspace, size_t workspace_bytes, void* stream);

/* Replaces sparse_gemm_mma_int4_launch (bindings.cc:150-161;
 * sparse_gemm_mma_int4.cu:25-253): Y_high = sx * sum_blk s[n,bc] * acc_hi, WITHOUT the
 * factor 16 (the caller applies it, triton_kernel/v9_linear.py:148).  Rows of
 * block-rows without blocks are written as zero. */
int w4a4_sparse_gemm(const void* W_high, const int32_t* hp_row_offsets, const int32_t* hp_col_indices,
                     const void* X_s4, const void* scale_u4, const void* scale_x, void* Y_high, int T,
                     int K, int N, int nnz, int flags, void* workspace, size_t workspace_bytes,
                     void* stream);

/* Replaces fused_quant_gemv_launch and fused_quant_dense_sparse_mma_int4_launch
 * (bindings.cc:204-251; fused_quant_gemv.cu:64-266,
 * fused_quant_dense_sparse_mma_int4.cu:179-483): fp16 activations in, fp16 out.
 * Quantisation and GEMM are two launches chained with programmatic dependent
 * launch so the weight prefetch overlaps the quantisation. */
int w4a4_fused_quant_dense_sparse(const void* X, long long ldx, const int32_t* perm, const void* W_low,
                                  const void* W_high, const int32_t* hp_row_offsets,
                                  const int32_t* hp_col_indices, const void* scale_u4,
                                  const void* zero_u4, void* Y, int T, int K, int N, int nnz,
                                  int flags, void* workspace, size_t workspace_bytes, void* stream);

/* Parity aid with no counterpart in the reference's bindings: runs the same
 * MMA path as w4a4_fused_dense_sparse and stores the exact int32 accumulators,
 * acc (ng, N, T) per group (the workspace the reference defines in
 * fused_dense_sparse/cutlass_dequant.cu:7-16) and acc_hi (nnz, 128, T) per residual
 * block.  Either output may be NULL. */
int w4a4_dump_accumulators(const void* W_low, const void* W_high, const int32_t* hp_row_offsets,
                           const int32_t* hp_col_indices, const void* X_s4, int32_t* acc,
                           int32_t* acc_hi, int T, int K, int N, int nnz, int flags, void* workspace,
                           size_t workspace_bytes, void* stream);

/* Prepared weights for many-token calls (prefill).  sm_100a tensor cores have no
 * 4-bit integer MMA, so the many-token kernel widens every weight nibble on the SM
 * on every call, and that widening - not the tensor pipe - bounds it.  A caller
 * with memory to spare can widen ONCE, after loading the weights (a load-time step,
 * where the reference has its adapter backend/weight_loader.py:111
 * pack_v9_weights_for_cutlass; no counterpart in its bindings):
 * w4a4_prepare_weights turns a packed array (W_low, or W_high) into one byte per
 * code - the e4m3 encoding of the code, exact for -8..7, codes in their natural
 * order, row shape kept - of w4a4_prepared_weights_bytes(packed_bytes) = 2 x packed_bytes
 * bytes.  The *_prepared entry points take the packed arrays AND the prepared ones:
 * calls that go to the tensor-core kernel then run e4m3 x e4m3 MMAs with fp32
 * accumulation on the prepared bytes (the products and sums are small integers,
 * exact in fp32, so every accumulator and every output bit equals the packed
 * path's); calls with few tokens stream the packed arrays as before.  NULL
 * prepared pointers (both, or the one of an operand in use) select the packed path.
 * Prepared pointers must be 16-byte aligned. */
/* Dense fp16 copy of the low-precision weights, out (N, K) row-major = fp16( fp16( fp16(code) - zero ) * scale ): the
 * dequantisation step of the reference's W4A16 route for long prompts without residual blocks
 * (triton_kernel/dequant_w4_to_fp16.py:131-172, used by backend/dispatcher.py:228-238; the fp16 GEMM that follows is
 * a plain library GEMM and is not part of this library). */
int w4a4_dequant_weights_fp16(const void* W_low, const void* scale_u4, const void* zero_u4, void* out_fp16, int N, int K,
                              void* stream);

size_t w4a4_prepared_weights_bytes(size_t packed_bytes);
int w4a4_prepare_weights(const void* packed, void* prepared, size_t packed_bytes, void* stream);
int w4a4_fused_dense_sparse_prepared(const void* W_low, const void* W_high, const void* W_low_prepared,
                                     const void* W_high_prepared, const int32_t* hp_row_offsets,
                                     const int32_t* hp_col_indices, const void* X_s4, const void* scale_u4,
                                     const void* zero_u4, const int32_t* sum_X, const void* scale_x, void* Y,
                                     int T, int K, int N, int nnz, int flags, void* workspace,
                                     size_t workspace_bytes, void* stream);
int w4a4_fused_quant_dense_sparse_prepared(const void* X, long long ldx, const int32_t* perm, const void* W_low,
                                           const void* W_high, const void* W_low_prepared,
                                           const void* W_high_prepared, const int32_t* hp_row_offsets,
                                           const int32_t* hp_col_indices, const void* scale_u4,
                                           const void* zero_u4, void* Y, int T, int K, int N, int nnz,
                                           int flags, void* workspace, size_t workspace_bytes, void* stream);
/* The same with activations expanded once for several linears.  w4a4_expand_activations_fmt writes the
 * codes in one of three forms (same group-major, chunk-swizzled layout, one byte per code):
 *   W4A4_CODES_S8           sign-extended s8, inside a packed word the four even-indexed codes then the four
 *                           odd-indexed ones (what w4a4_expand_activations writes).  Read by the streaming
 *                           kernel and by the tensor-core kernel's integer MMAs on the packed weights.
 *   W4A4_CODES_E4M3         e4m3 encodings of the same integers in their natural order.  Read by fp8 MMAs
 *                           against PREPARED weights: pass the buffer to
 *                           w4a4_fused_dense_sparse_expanded_prepared with W4A4_FLAG_CODES_E4M3.
 *   W4A4_CODES_E4M3_PACKED  e4m3 encodings in the even-then-odd order.  Read by fp8 MMAs against the PACKED
 *                           weights, whose nibbles the kernel turns into e4m3 numbers on the SM with three
 *                           logic operations per eight codes (a nibble with bit 3 flipped, alone in its
 *                           byte, is the e4m3 value (code + 8) * 2^-9; the offset leaves with the zero-point
 *                           term, which is why this form needs the group sums).  Pass the buffer with
 *                           W4A4_FLAG_CODES_E4M3_PACKED and NULL prepared pointers.
 * The flags alone say which bytes XE holds and a mismatch is W4A4_ERR_BAD_ARG, never a silent
 * reinterpretation: prepared pointers without W4A4_FLAG_CODES_E4M3, W4A4_FLAG_CODES_E4M3 without
 * prepared weights for every operand in use, both flags at once.  A call with e4m3 codes of either form
 * always runs the tensor-core kernel, whatever the token count (the streaming kernel reads s8 codes;
 * W4A4_FLAG_FORCE_STREAM with e4m3 codes is W4A4_ERR_BAD_ARG).  The entry points that expand the codes
 * themselves pick W4A4_CODES_E4M3 when prepared weights are given, else W4A4_CODES_S8 - or
 * W4A4_CODES_E4M3_PACKED when the environment variable W4A4_PREFILL_F8=1 is set and the call carries
 * the group sums. */
#define W4A4_CODES_S8   0
#define W4A4_CODES_E4M3 1
#define W4A4_CODES_E4M3_PACKED 2
int w4a4_expand_activations_fmt(const void* X_s4, const int32_t* sum_X, void* XE, float* sumxf, int T, int K,
                                int code_format, void* stream);
int w4a4_fused_dense_sparse_expanded_prepared(const void* W_low, const void* W_high, const void* W_low_prepared,
                                              const void* W_high_prepared, const int32_t* hp_row_offsets,
                                              const int32_t* hp_col_indices, const void* XE, const float* sumxf,
                                              const void* scale_u4, const void* zero_u4, const void* scale_x,
                                              void* Y, int T, int K, int N, int nnz, int flags, void* workspace,
                                              size_t workspace_bytes, void* stream);
int w4a4_dump_accumulators_prepared(const void* W_low, const void* W_high, const void* W_low_prepared,
                                    const void* W_high_prepared, const int32_t* hp_row_offsets,
                                    const int32_t* hp_col_indices, const void* X_s4, int32_t* acc,
                                    int32_t* acc_hi, int T, int K, int N, int nnz, int flags, void* workspace,
                                    size_t workspace_bytes, void* stream);

/* Output exchange of a column-parallel (row-sharded) linear over peer memory, for one process per GPU on one
 * node.  No counterpart in the reference, which is single-GPU.  Set-up (these four calls allocate or map memory
 * and are NOT stream-ordered; call them once, outside any capture): every rank allocates a buffer with
 * w4a4_peer_alloc (zero-filled), exports a 64-byte handle with w4a4_peer_export, the host code passes the
 * handles between the processes, and every rank maps its peers' buffers with w4a4_peer_open (close with
 * w4a4_peer_close before the owner frees).
 *
 * w4a4_peer_push_wait(src, ...) is the per-step call: one kernel copies this rank's shard (`rows` rows of
 * `row_bytes` bytes, `src_pitch` apart) into EVERY rank's full-output buffer dst[i] (host array of `world` device
 * pointers, own buffer included) at byte offset dst_offset with row pitch dst_pitch, using plain 16-byte stores
 * to peer-mapped memory; raises flags[i][rank] (host array of `world` pointers to each rank's array of `world`
 * 32-bit flags); and then waits until all `world` flags of THIS rank have arrived, so that when the kernel has
 * finished the full output is complete in this rank's buffer.  The wait is bounded: after poll_limit polls per
 * flag the kernel records the device error word (w4a4_device_error) and returns.  `state` is (1 + 2 * world)
 * zero-initialised 32-bit words of LOCAL device memory that belong to this (buffer set, rank); every rank must
 * make the same sequence of calls on a buffer set.  Reusing a destination buffer is safe once every rank has
 * completed a later w4a4_peer_push_wait (alternate between two buffer sets). */
int w4a4_peer_alloc(size_t bytes, void** ptr /* host */);
int w4a4_peer_free(void* ptr);
int w4a4_peer_export(const void* ptr, void* handle /* host, 64 bytes */);
int w4a4_peer_open(const void* handle /* host, 64 bytes */, void** ptr /* host */);
int w4a4_peer_close(void* ptr);
int w4a4_peer_push_wait(const void* src, long long src_pitch, void* const* dst /* host */, void* const* flags /* host */,
                        long long dst_pitch, long long dst_offset, int rows, int row_bytes, int world, int rank,
                        void* state, int poll_limit, void* stream);

/* No counterpart in the reference (its launchers allocate split-K partials with
 * torch::empty, fused_dense_sparse_mma_int4.cu:1873-1879).
 *
 * Same computation and arguments as w4a4_fused_dense_sparse, for callers that
 * cannot allocate device memory and therefore have no workspace to pass: code
 * that runs inside someone else's CUDA-graph capture or allocator-free serving
 * loop, a plugin whose host owns every allocation, a process whose memory pool is
 * already carved up.  The scratch the call needs (the activations in the layout
 * the GEMM reads) lives in an array that is part of the library image instead,
 * so the size is capped: T <= W4A4_NOALLOC_MAX_T tokens and
 * K <= W4A4_NOALLOC_MAX_K features (about 544 KiB, held by every GPU that loads
 * the library until the process exits).  Larger shapes return
 * W4A4_ERR_UNSUPPORTED with a message naming the limits.  The call itself never
 * calls cudaMalloc / cudaFree or any allocating routine.
 *
 * The first call on a device looks up the device address of that array (one
 * cudaGetSymbolAddress with that device current); make that first call outside
 * any stream capture.  All calls on a device share the one array and it keeps
 * the previous call's contents (the part that must start clean is cleared on
 * every call): two calls whose GPU work overlaps - different streams without an
 * ordering between them - race on it.  Order them on one stream. */
#define W4A4_NOALLOC_MAX_T 16
#define W4A4_NOALLOC_MAX_K 32768
int w4a4_fused_dense_sparse_noalloc(const void* W_low, const void* W_high, const int32_t* hp_row_offsets,
                                    const int32_t* hp_col_indices, const void* X_s4, const void* scale_u4,
                                    const void* zero_u4, const int32_t* sum_X, const void* scale_x, void* Y,
                                    int T, int K, int N, int nnz, int flags, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* W4A4_B200_H_ */
