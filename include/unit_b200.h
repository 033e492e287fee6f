/*
 * unit_b200 -- C ABI of the B200 (sm_100a) implementation of the contractions
 * that were/UNIT tensorizes: u8 x s8 -> s32 conv2d / dense (its AVX-512 VNNI
 * path) and fp16 -> fp32 conv2d / GEMM (its wmma path).
 *
 * Conventions
 *   - every pointer named d_* is a DEVICE pointer, 16-byte aligned;
 *   - the caller owns every buffer; the library reads inputs and writes only
 *     the output (and, for the pack calls, the destination);
 *   - the first contraction call on a device, and the first use of each kernel variant, make
 *     one-off runtime queries (a symbol address, a kernel attribute): make a warm-up call of each
 *     shape before capturing calls into a CUDA graph;
 *   - `stream` is a cudaStream_t passed as void*; calls are asynchronous on it;
 *   - every function returns a unit_status; nothing throws, aborts or prints;
 *   - weights are consumed in a tensor-core-ready copy ("packed weights") that
 *     the caller produces once per weight tensor with the unit_pack_weights_*
 *     calls into a buffer of unit_packed_weights_bytes_* bytes.  The packed
 *     form depends only on the arguments of the pack call.
 *
 * Each entry point names the reference interface it replaces (paths inside
 * were/UNIT).  The reference JIT-compiles a TVM module and calls it as
 * module(a, b, c) with the caller-allocated output last
 * (poc/vnni/vnni_dense.py:66, apps/gpu/conv-fused.py:155); the functions
 * below keep that argument order: inputs, weights, output.
 */
#ifndef UNIT_B200_H_
#define UNIT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum unit_status {
  UNIT_OK = 0,
  UNIT_ERR_NULL = -1,        /* a required pointer is NULL */
  UNIT_ERR_SHAPE = -2,       /* a dimension is out of the supported range */
  UNIT_ERR_ALIGN = -3,       /* a pointer or leading dimension is not 16-byte aligned */
  UNIT_ERR_LAYOUT = -4,      /* channel block / tile size not supported */
  UNIT_ERR_ARCH = -5,        /* the current device is not compute capability 10.0 */
  UNIT_ERR_LAUNCH = -6,      /* the CUDA runtime refused the launch or a copy */
  UNIT_ERR_DEVICE_WAIT = -7, /* a kernel gave up on an internal wait and flagged it */
  UNIT_ERR_TOO_LARGE = -8    /* beyond a stated fixed capacity */
} unit_status;

/* Geometry of one convolution.  Channels are the stored (blocked) counts:
 * c_in is a multiple of c_block, c_out a multiple of 16.
 * Data layout  [n][c_in/c_block][h][w][c_block]   (NCHW16c, or NCHW4c when
 * c_block == 4: apps/cpu/kernel/conv2d.py:18-30).
 * Output layout [n][c_out/16][oh][ow][16], oh = (h + 2 pad_h - kh)/stride_h + 1.
 * The reference convolves a pre-padded input with padding 0
 * (apps/cpu/kernel/conv2d.py:50); pad_h/pad_w here are implicit zero padding
 * with the same result as padding the input first. */
typedef struct unit_conv_desc {
  int32_t n, c_in, h, w;
  int32_t c_block; /* 16, or 4 (int8 only) */
  int32_t c_out;
  int32_t kh, kw;
  int32_t stride_h, stride_w;
  int32_t pad_h, pad_w;
} unit_conv_desc;

/* The int8 convolution's epilogue, applied to the s32 accumulator acc of every output element:
 *     t = acc + d_bias[oc]            (wrapping s32; d_bias may be NULL)
 *     t = t * mul                     (wrapping s32)
 *   out_u8 == 0:  the s32 output is t.  With mul = 11 this is the fused operator of the
 *                 reference's graph flow, multiply(add(conv, bias), 11)
 *                 (apps/cpu/relay/conv2d.py:21-23, fused as apps/cpu/relay/result.log:35).
 *                 shift must be 0 and d_residual NULL.
 *   out_u8 != 0:  q = (t + 2^(shift-1)) >> shift  (arithmetic shift, 1 <= shift <= 31),
 *                 q = q + d_residual[same index as the output]   (u8, may be NULL),
 *                 output = clamp(q, 0, 255) as u8.  mul must be 1.  The clamp at 0 is the ReLU of
 *                 a residual block, so a bottleneck block chains u8 NCHW16c -> u8 NCHW16c with no
 *                 repack.  The reference fixes no rounding rule for this form; this is the
 *                 library's own requantisation.
 * x_signed != 0: the activations are s8 instead of u8.  The reference converts s8 activations to
 *                 u8 by adding 128 and subtracts 128 * sum(weights) per output channel afterwards
 *                 (apps/cpu/relay/result.log:4-6,15-21) because its instruction multiplies
 *                 u8 x s8; the tensor core multiplies s8 x s8 directly, which gives the same
 *                 numbers, and padding is s8 zero. */
typedef struct unit_epilogue {
  const int32_t *d_bias;
  int32_t mul;
  int32_t shift;
  int32_t out_u8;
  const uint8_t *d_residual;
  int32_t x_signed;
} unit_epilogue;

/* Geometry of one three-dimensional convolution (apps/cpu/kernel/conv3d.py:39-64).
 * Data   [n][c_in/16][d][h][w][16] u8 (or s8), weights [c_out/16][c_in/16][kd][kh][kw][4][16][4] s8,
 * output [n][c_out/16][od][oh][ow][16].  The reference convolves pre-padded inputs without padding
 * (conv3d.py:60); pad_* here is implicit zero padding with the same result. */
typedef struct unit_conv3d_desc {
  int32_t n, c_in, d, h, w;
  int32_t c_out;
  int32_t kd, kh, kw;
  int32_t stride_d, stride_h, stride_w;
  int32_t pad_d, pad_h, pad_w;
} unit_conv3d_desc;

/* A prepared launch (see unit_conv2d_plan_int8): plain bytes owned by the caller, valid in this
 * process for the device that was current when it was made, until the buffers it names are freed.
 * May be copied; holds no resource. */
typedef struct unit_conv_plan {
  uint64_t opaque[128];
} unit_conv_plan;

/* Keys of unit_debug_set. */
enum {
  UNIT_DEBUG_WAIT_LIMIT_NS = 1,       /* bound of every device-side wait, nanoseconds (default 1e9) */
  UNIT_DEBUG_STALL_WEIGHT_COPIES = 2  /* non-zero: contraction kernels issue no weight copies, so
                                         their waits run out and they report UNIT_ERR_DEVICE_WAIT */
};

/* Library version, major*10000 + minor*100 + patch. */
int unit_version(void);
/* Static string for a unit_status value. */
const char *unit_status_string(int status);
/* Synchronises `stream`, then reports (and clears) the device-side error word:
 * UNIT_OK, UNIT_ERR_DEVICE_WAIT if a kernel abandoned a bounded wait, or
 * UNIT_ERR_LAUNCH for a CUDA error. */
int unit_device_status(void *stream);
/* Number of kernels this library has launched in this process (monotonic). */
uint64_t unit_launch_count(void);
/* Tile trace for tuning (the counterpart of the reference's per-pass / per-op timers,
 * apps/cpu/relay/conv2d.py:31-49).  While a buffer is attached, the first thread block of
 * every contraction kernel writes 16 u64 timestamps per tile it processes,
 * for its first capacity_tiles tiles:  [0] A producer starts the tile, [1] A producer has
 * issued all copies, [2] B producer has issued all copies, [3] MMA issuer owns an
 * accumulator, [4] first stage landed, [5] last MMA issued, [6] drain sees the accumulator
 * complete, [7] drain has stored the tile; the rest unused.  Timestamps are SM cycle counts
 * (clock64) of the SM that runs that block.  d_buf: capacity_tiles * 128 bytes of device
 * memory owned by the caller; NULL detaches.  Not for use while kernels are running. */
int unit_trace_attach(void *d_buf, int32_t capacity_tiles);

/* Tensor-core peak probe, the counterpart of the reference's instruction-rate microbenchmark
 * (poc/vnni/micro.cc:16-51).  Every SM runs `issuers` (1-4) threads that each issue `iters`
 * back-to-back tcgen05.mma of 128 x n x 32 bytes on operands resident in shared memory
 * (f16 == 0: u8 x s8 -> s32; otherwise fp16 -> fp32); issuers * n <= 512.  Synchronous; writes
 * operations per second (2 per multiply-accumulate) of the whole device to *ops_per_second. */
int unit_tensor_peak(int32_t f16, int32_t n, int32_t issuers, int32_t iters, double *ops_per_second,
                     void *stream);

/* Per-shape tile table, the counterpart of the reference's tuning logs (cpu-tune.log, gpu-tune.log:
 * shape -> index of the best schedule, loaded by python/tensorizer/tune.py:20-51).  An entry names an
 * int8 NCHW16c convolution by its weight-side geometry and, optionally, one input size (n > 0), and
 * overrides what the library's heuristics would choose:
 *   bn      width of a column block (multiple of 16, <= 256; 0 = heuristic), and
 *   kc      16-byte K columns per pipeline stage (even, <= 16; 0 = heuristic): these two shape the
 *           packed weights, so they are taken only from entries with n = 0 (every input size), and the
 *           table must be the same when weights are packed and when they are used;
 *   mt      sub-tiles per tile (1, 2; 0 = heuristic);
 *   ksplit  largest split-K cluster (2-8), 1 = never split, 0 = heuristic.
 * unit_tile_table_set replaces the process-wide table (n = 0 clears it).  unit_b200/tune.py fills a
 * table by timing the candidates over the reference's shape corpus. */
typedef struct unit_tile_entry {
  int32_t c_in, c_block, c_out, kh, kw, stride_h, stride_w;
  int32_t n, h, w; /* n = 0: any input size (h, w ignored) */
  int32_t bn, kc, mt, ksplit;
} unit_tile_entry;
int unit_tile_table_set(const unit_tile_entry *entries, int32_t n);

/* Which kernel variant ran: the contraction kernel exists in one compiled variant per (operand
 * path, epilogue, data type, sub-tiles per tile).  unit_variant_count() is the size of the index
 * space; unit_variant_name(i) is NULL for indices without a compiled variant, otherwise a static
 * string such as "igemm_kernel<A_CONV_BOX, EPI_REQ_NCHWC, i8, MT=2>"; unit_variant_launches(i)
 * counts this process's launches of it.  The counterpart of the schedule index the reference logs
 * per shape (cpu-tune.log, python/tensorizer/tune.py:20-51). */
int unit_variant_count(void);
const char *unit_variant_name(int index);
uint64_t unit_variant_launches(int index);
/* Diagnostics for testing the error path without faulting the device (no counterpart in the
 * reference).  Every device-side wait is bounded; a kernel whose wait runs out stops, frees what
 * it holds and sets the error word that unit_device_status reports.  Process-wide; applies to
 * launches made afterwards. */
int unit_debug_set(int key, long long value);

/* ---- packed weights ------------------------------------------------------ */

/* Replaces: the reference hands its packed weight array straight to the
 * generated kernel (apps/cpu/kernel/conv2d.py:26,30).  Source layout
 * [c_out/16][c_in/c_block][kh][kw][c_block/4][16][4] s8.  The packed form depends on
 * c_in, c_block, c_out, kh, kw and the strides (the column-block width is chosen per stride) and,
 * for c_block == 4 and for strides other than 1, on the padding too (a stride-2 kernel carries a
 * copy for pixel-pair rows, whose taps sit by the parity of the horizontal padding): pack with
 * the descriptor fields the convolution will use (n, h and w may differ). */
size_t unit_packed_weights_bytes_conv_i8(const unit_conv_desc *desc);
int unit_pack_weights_conv_i8(const unit_conv_desc *desc, const int8_t *d_w,
                              void *d_packed, void *stream);

/* Source layout [c_out/16][c_in/16][kh][kw][16 i][16 o] fp16
 * (python/tensorizer/ops/gpu.py:29-31). */
size_t unit_packed_weights_bytes_conv_f16(const unit_conv_desc *desc);
int unit_pack_weights_conv_f16(const unit_conv_desc *desc, const void *d_w,
                               void *d_packed, void *stream);

/* Source layout [n/tile][k/4][tile][4] s8 (apps/cpu/kernel/int8-gemm.py:11-14). */
size_t unit_packed_weights_bytes_dense_i8(int32_t n, int32_t k);
int unit_pack_weights_dense_i8(int32_t n, int32_t k, int32_t tile, const int8_t *d_b,
                               void *d_packed, void *stream);

/* Source layout B[k][n] fp16 row-major (apps/gpu/gemm.py:8). */
size_t unit_packed_weights_bytes_gemm_f16(int32_t n, int32_t k);
int unit_pack_weights_gemm_f16(int32_t n, int32_t k, const void *d_b,
                               void *d_packed, void *stream);

/* ---- contractions -------------------------------------------------------- */

/* Scratch memory the int8 convolution can use for this geometry (0 for most).  A stride-2
 * convolution on NCHW4c data (the 3-channel stem) is fastest when it may first fold 2 x 2
 * pixel blocks into a 16-channel image of half the size in scratch memory; without scratch
 * (d_workspace NULL or too small) the same call runs a slower in-place gather.  No
 * counterpart in the reference, whose generated kernels use no scratch. */
size_t unit_conv2d_workspace_bytes(const unit_conv_desc *desc);

/* Replaces topi.nn.conv2d_NCHWc_int8(..., out_dtype='int32') scheduled with
 * INTRINSICS['vnni'] (apps/cpu/kernel/conv2d.py:50-54).  d_out is s32
 * [n][c_out/16][oh][ow][16]; d_bias (c_out s32) may be NULL.  d_workspace: device
 * scratch of workspace_bytes (see unit_conv2d_workspace_bytes), may be NULL. */
int unit_conv2d_u8s8s32_nchwc(const unit_conv_desc *desc, const uint8_t *d_x,
                              const void *d_packed_w, const int32_t *d_bias,
                              int32_t *d_out, void *d_workspace, size_t workspace_bytes,
                              void *stream);

/* Same contraction with the fused epilogue
 *   q = clamp((acc + bias[oc] + 2^(shift-1)) >> shift, 0, 255)  -> u8 NCHW16c.
 * This is the library's own requantisation (the reference's graph flow fuses bias and an s32
 * multiply instead, apps/cpu/relay/conv2d.py:21-23: see unit_epilogue).  1 <= shift <= 31. */
int unit_conv2d_u8s8_requant_nchwc(const unit_conv_desc *desc, const uint8_t *d_x,
                                   const void *d_packed_w, const int32_t *d_bias,
                                   int32_t shift, uint8_t *d_out, void *d_workspace,
                                   size_t workspace_bytes, void *stream);

/* The general int8 convolution: u8 or s8 activations and the whole epilogue family of
 * unit_epilogue.  d_out is s32 (out_u8 == 0) or u8 NCHW16c.  The two entry points above are
 * this one with {bias, 1, 0, 0, NULL, 0} and {bias, 1, shift, 1, NULL, 0}.  Replaces the fused
 * conv2d_NCHWc + subtract + add + multiply operator of apps/cpu/relay/result.log:21-24,35. */
int unit_conv2d_int8_nchwc(const unit_conv_desc *desc, const void *d_x, const void *d_packed_w,
                           const unit_epilogue *epilogue, void *d_out, void *d_workspace,
                           size_t workspace_bytes, void *stream);

/* The same call split in two, the way the reference builds a module once and then calls it
 * (poc/vnni/vnni_dense.py:40-66: tvm.build, then module(a, b, c) under time_evaluator).
 * unit_conv2d_plan_int8 checks the arguments, selects the kernel variant and tile shape and
 * encodes the tensor map into *plan; unit_conv2d_run launches it on `stream` (one kernel; two
 * for a folded stem) with no further host work.  The plan names the buffers it was made for. */
int unit_conv2d_plan_int8(const unit_conv_desc *desc, const void *d_x, const void *d_packed_w,
                          const unit_epilogue *epilogue, void *d_out, void *d_workspace,
                          size_t workspace_bytes, unit_conv_plan *plan);
int unit_conv2d_run(const unit_conv_plan *plan, void *stream);

/* Three-dimensional int8 convolution on NCDHW16c (replaces the compute of
 * apps/cpu/kernel/conv3d.py:58-64, scheduled by INTRINSICS['vnni'] like the two-dimensional one).
 * Same contraction kernel: the depth axis takes the place of the batch axis (a tile runs over
 * (od, oh, ow) of one image, one launch per image), the kernel depth adds a third tap index.
 * Epilogue as for unit_conv2d_int8_nchwc; the reference's form is the plain s32 output
 * {NULL, 1, 0, 0, NULL, 0}.  The packed weights depend on c_in, c_out, the kernel size and the
 * strides. */
size_t unit_packed_weights_bytes_conv3d_i8(const unit_conv3d_desc *desc);
int unit_pack_weights_conv3d_i8(const unit_conv3d_desc *desc, const int8_t *d_w, void *d_packed,
                                void *stream);
int unit_conv3d_int8_ncdhwc(const unit_conv3d_desc *desc, const void *d_x, const void *d_packed_w,
                            const unit_epilogue *epilogue, void *d_out, void *stream);

/* Requantising convolution for callers that may not allocate.  No counterpart in the
 * reference.  It is unit_conv2d_u8s8_requant_nchwc with the scratch taken from a fixed array
 * inside the library instead of a caller-provided workspace.  Some hosts of this library have
 * no way to obtain device memory at call time: an operator invoked from a runtime whose buffers
 * are all planned before execution (as the reference's graph runtime does) receives only its
 * input and output tensors, and a serving loop that must never trigger the device-wide
 * synchronisation of cudaMalloc / cudaFree cannot allocate either.  This entry point calls no
 * cudaMalloc, cudaFree or other allocating routine.
 *   - Limit: the scratch a geometry needs (unit_conv2d_workspace_bytes) must not exceed
 *     unit_noalloc_scratch_capacity() = 8 MiB, e.g. a 224 x 224 NCHW4c stem up to batch 41;
 *     larger requests return UNIT_ERR_TOO_LARGE and nothing is launched.  Geometries that need
 *     no scratch are simply forwarded.
 *   - Every GPU that loads the library holds the 8 MiB until the process exits.
 *   - The first call on each device looks up the array's device address (one runtime query,
 *     no allocation); make that first call before any stream capture begins.
 *   - All calls share the one array, which keeps whatever the last call wrote.  Nothing in it
 *     has to start at zero: each call overwrites the part it reads.  Calls that can overlap on
 *     the GPU (different streams, or one stream's call not yet finished when another begins
 *     elsewhere) race on it; issue them on one stream or serialise them yourself. */
size_t unit_noalloc_scratch_capacity(void);
int unit_conv2d_u8s8_requant_nchwc_noalloc(const unit_conv_desc *desc, const uint8_t *d_x,
                                           const void *d_packed_w, const int32_t *d_bias,
                                           int32_t shift, uint8_t *d_out, void *stream);

/* Replaces topi.x86.dense_dotprod(a, b_packed, None, 'int32')
 * (apps/cpu/kernel/int8-gemm.py:16).  A is u8 [m][k] with row pitch lda
 * bytes, C is s32 [m][n] with row pitch ldc elements. */
int unit_dense_u8s8s32(int32_t m, int32_t n, int32_t k, const uint8_t *d_a, int64_t lda,
                       const void *d_packed_w, int32_t *d_c, int64_t ldc, void *stream);

/* Replaces conv2d_NCHW16c_OHWI16o (python/tensorizer/ops/gpu.py:8-58).
 * d_x fp16 NCHW16c, d_out fp32 NCHW16c; desc->c_block must be 16. */
int unit_conv2d_f16f32_nchw16c(const unit_conv_desc *desc, const void *d_x,
                               const void *d_packed_w, float *d_out, void *stream);

/* Replaces the tensor-core GEMM of apps/gpu/gemm.py:6-19 and
 * poc/tensorcore/gemm-prefetch.cu:66-164.  A fp16 [m][k] (row pitch lda
 * bytes), C fp32 [m][n] (row pitch ldc elements). */
int unit_gemm_f16f32(int32_t m, int32_t n, int32_t k, const void *d_a, int64_t lda,
                     const void *d_packed_w, float *d_c, int64_t ldc, void *stream);

/* ---- layout transforms --------------------------------------------------- */

/* Replaces the in-graph pack of python/tensorizer/ops/gpu.py:26-28 and the
 * layout_transform chain of the graph flow.  NCHW (c channels) ->
 * [n][ceil(c/c_block)][h][w][c_block], missing channels zero; elem_bytes is
 * 1 (u8) or 2 (fp16) or 4 (s32 / fp32). */
int unit_pack_data_nchw_to_nchwc(const void *d_src, void *d_dst, int32_t n, int32_t c,
                                 int32_t h, int32_t w, int32_t c_block, int32_t elem_bytes,
                                 void *stream);
/* Inverse: blocked -> NCHW, keeping the first c channels. */
int unit_unpack_data_nchwc_to_nchw(const void *d_src, void *d_dst, int32_t n, int32_t c,
                                   int32_t h, int32_t w, int32_t c_block, int32_t elem_bytes,
                                   void *stream);
/* OIHW s8 -> [o/16][i/c_block][kh][kw][c_block/4][16][4], zero padded
 * (the array apps/cpu/kernel/conv2d.py:26,30 declares). */
int unit_pack_weights_oihw_to_ref_i8(const int8_t *d_src, int8_t *d_dst, int32_t o, int32_t i,
                                     int32_t kh, int32_t kw, int32_t c_block, void *stream);
/* OIHW fp16 -> [o/16][i/16][kh][kw][16 i][16 o] (python/tensorizer/ops/gpu.py:29-31). */
int unit_pack_weights_oihw_to_ref_f16(const void *d_src, void *d_dst, int32_t o, int32_t i,
                                      int32_t kh, int32_t kw, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* UNIT_B200_H_ */
