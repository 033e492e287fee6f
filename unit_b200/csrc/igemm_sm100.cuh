// Implicit-GEMM contraction kernel for sm_100a: tcgen05.mma with the accumulator
// in tensor memory, a warp-specialised producer / issuer / drain pipeline, and a
// persistent tile loop (one CTA per SM).
//
// GEMM view of every operator this library offers:
//   D[m][n] = sum_k A[m][k] * B[n][k]
//   m : output pixel (n_img, oh, ow) flattened, or a row of a plain matrix
//   n : output channel
//   k : (kh, kw, input channel), or the K index of a plain matrix
// K is cut into 16-byte "columns" (16 u8 or 8 fp16 values of one m or n row).
//
// Shared-memory operand format: the tensor core's K-major, no-swizzle layout.
// A "core matrix" is 8 rows x 16 bytes stored as 128 contiguous bytes; a tile
// of R rows and KC columns is stored column by column, [KC][R][16 B], so
//   stride between 8-row groups (SBO)     = 128 bytes
//   stride between adjacent K columns (LBO) = R * 16 bytes.
// NCHW16c activations fit this format natively: 16 channels of one u8 pixel
// are one 16-byte core-matrix row and consecutive pixels of an image row are
// consecutive rows.  The A tile is filled by tensor copies (TMA): whole-row
// boxes for stride 1, im2col-mode copies for other strides, column copies for
// plain matrices; 16-byte cp.async gathers with zero fill remain as the path
// for small tensors and NCHW4c without scratch.  Weights are repacked once on
// the device into ready-made [KC][BN][16 B] stage blocks and arrive with a
// single bulk copy (cp.async.bulk, no tensor map, no multicast) per stage.
//
// Two operands have K contiguous in memory in runs longer than 16 bytes and use the tensor
// core's swizzled K-major layouts instead, written directly by the copy engine: plain matrices
// (rows of 128 bytes, SWIZZLE_128B) and fp16 pixels (rows of 32 bytes = one K step, SWIZZLE_32B).
//
// A CTA tile is MT x 128 rows by BN columns (MT = 1 or 2): with MT = 2 one B
// stage feeds two accumulators, which halves the weight bytes fetched per MAC.
//
// Warp roles (736 threads):
//   warps 0-15  drain: tcgen05.ld the finished accumulator (warp w may touch
//               TMEM lanes 32(w%4)..+31 = tile rows), requantise or copy, store.
//               With two accumulator sets in TMEM the warps form two groups of
//               eight, one per set, that drain alternate tiles independently.
//               They also prepare the bias of the tile that will use their set
//               next: as s8 digits that one extra MMA K step adds to the
//               accumulator (so the drain itself only shifts, clamps and stores),
//               or as integers to add where the values do not fit that form
//   warps 16-19 A producers: lanes issue the tensor copies of a stage (or 128
//               threads gather columns with cp.async, whose copies arrive on the
//               stage barrier by themselves)
//   warp  20    B producer: one lane issues the bulk copies
//   warp  21    TMEM allocation; runs the issue loop of sub-tile 0 converged, one elected lane
//               executes tcgen05.mma / tcgen05.commit
//   warp  22    (MT = 2) the same for sub-tile 1: one warp cannot issue MMAs fast enough to
//               keep the tensor core busy on narrow column blocks
// When two accumulator sets fit in the 512 TMEM columns, the drain of tile i
// overlaps the main loop of tile i+1.
//
// The kernel is launched with programmatic stream serialisation: barrier set-up
// and TMEM allocation may overlap the previous kernel's tail; griddepcontrol.wait
// precedes the first access to global memory.
//
// Every wait on an mbarrier is bounded in time.  A wait that runs out sets a
// CTA-wide abort flag and a global error word; all roles then leave their
// loops, let their own copies land, and the CTA frees its TMEM and returns.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace unit {

enum AMode : int {
  A_CONV_I8 = 0,   // u8 NCHW16c: one 16-byte column = one channel chunk of one tap
  A_CONV_F16 = 1,  // fp16 NCHW16c: one chunk = two 16-byte columns
  A_STEM_I8 = 2,   // u8 NCHW4c: one column = 4 consecutive kw taps x 4 channels
  A_DENSE = 3,     // plain row-major matrix, K contiguous
  A_CONV_TMA = 4,  // NCHW16c (u8 or fp16) fetched by im2col-mode TMA: one bulk tensor copy per K column
  A_CONV_BOX = 5,  // u8 NCHW16c, stride 1: each sub-tile is a box of (images x output rows x
                   // row segment) fetched by tiled-mode TMA, whole pixel rows at a time
  A_DENSE_TMA = 6, // plain row-major matrix fetched by tiled-mode TMA: one copy = 128 rows x 16 bytes
  A_CONV_WIN = 7   // u8 NCHW16c, stride 1, kernels larger than 1x1: a tile is a run of consecutive positions of
                   // the zero-padded image; the rows it touches are copied ONCE per channel chunk and every tap
                   // of the kernel reads them as a shifted window (see the kernel)
};
__host__ __device__ constexpr bool a_mode_uses_tma(int m) {
  return m == A_CONV_TMA || m == A_CONV_BOX || m == A_DENSE_TMA || m == A_CONV_WIN;
}
enum EpiMode : int {
  EPI_RAW_NCHWC = 0,  // 32-bit accumulator (+ s32 bias) -> [n][oc/16][oh][ow][16]
  EPI_REQ_NCHWC = 1,  // + bias, round-shift, clamp -> u8 [n][oc/16][oh][ow][16]
  EPI_RAW_ROWS = 2,   // 32-bit accumulator -> row-major [m][n]
  EPI_MUL_NCHWC = 3,  // (accumulator + s32 bias) * mul, wrapping -> s32 [n][oc/16][oh][ow][16]
  EPI_RES_NCHWC = 4   // EPI_REQ_NCHWC with a u8 residual tensor added after the shift, before the clamp
};
__host__ __device__ constexpr bool epi_requantises(int e) { return e == EPI_REQ_NCHWC || e == EPI_RES_NCHWC; }

constexpr int kTileM = 128;
constexpr int kMaxStages = 12;
constexpr int kNumThreads = 736;
constexpr int kDrainWarps = 16, kFirstProducerWarp = 16, kBWarp = 20, kMmaWarp = 21, kMmaWarp2 = 22;
constexpr uint32_t kFoldBBytes = 4096;  // one accumulator set's bias digits: 256 channels x 16 bytes
constexpr uint32_t kFoldBytes = 2 * kFoldBBytes + 2 * 128 * 16;  // two sets + the constant A block (2 columns)
#ifndef UNIT_WAIT_HINT_NS
#define UNIT_WAIT_HINT_NS 100
#endif
constexpr uint32_t kWaitHintNs = UNIT_WAIT_HINT_NS;  // longest suspension of one mbarrier probe
constexpr int kBiasSmem = 256;  // bias values of the current N tile, staged in shared memory per accumulator set
constexpr uint32_t kErrWaitFull = 1, kErrWaitEmpty = 2, kErrWaitTmemFull = 3, kErrWaitTmemEmpty = 4, kErrWaitBias = 5, kErrWaitPeer = 6;

// n / d for 0 <= n < 2^31 with a host-computed multiplier (mul == 0: d is a power of two).
struct FastDiv {
  uint32_t mul, shr;
};
__device__ __forceinline__ uint32_t fast_div(uint32_t n, FastDiv f) {
  return f.mul != 0u ? (__umulhi(n, f.mul) >> f.shr) : (n >> f.shr);
}

struct IgemmParams {
  const uint8_t *a;   // activations / A matrix
  const uint8_t *b;   // packed weights
  void *out;
  const int32_t *bias;
  unsigned int *err;  // global error word (0 = fine)
  long long m_total;  // GEMM rows
  int n_total;        // GEMM columns actually stored (multiple of 16)
  int bn;             // N tile (multiple of 16, <= 256)
  int kc;             // 16-byte K columns per pipeline stage (even)
  int cols;           // real K columns
  int k_stages;       // ceil(cols_padded / kc)
  int last_ksteps;    // MMA K-steps (2 columns each) in the last stage
  int stages;         // pipeline depth
  int m_tiles, n_tiles;
  // convolution geometry (unused by A_DENSE)
  int H, W, Cc, OH, OW, KH, KW, sh, sw, ph, pw;
  int kwg;            // A_STEM_I8: groups of 4 kw taps per kh
  long long img_bytes;  // bytes of one input image
  long long lda;      // A_DENSE: row pitch in bytes
  long long ldc;      // EPI_RAW_ROWS: row pitch in elements
  int shift;          // EPI_REQ_NCHWC
  FastDiv div_ohw, div_ow;  // divisions by OH*OW and OW (A_CONV_TMA)
  int cols_per_chunk;       // A_CONV_TMA: 16-byte columns per channel chunk (1 for u8, 2 for fp16)
  // A_CONV_BOX: a 128-row sub-tile holds box_n images x box_h output rows x box_w output columns,
  // rows ordered (image, row, column); sub-tile index = (n block, h block, w block), w fastest
  int box_n, box_h, box_w, blocks_h, blocks_w, n_img;
  long long sub_tiles;      // number of sub-tiles
  FastDiv div_box_hw, div_box_w, div_blocks_w, div_blocks_h;
  // Row form of A_CONV_BOX (row_kw > 0): a sub-tile is one row segment of one image and one
  // channel chunk, so the KW taps of a kernel row are the same pixels shifted by 16 bytes each.
  // One copy of box_w + KW - 1 pixels then serves all KW columns of that kernel row: the MMA
  // reads column (kh, kw) at the row buffer's address + 16 kw, and the two columns of a K step
  // are 16 bytes apart (overlapping core matrices).
  int a_sw32;     // A_CONV_BOX with 32-byte rows = one K step each, 32-byte swizzled, one box copy per K step: fp16 pixels,
                  // or pairs of u8 pixels (horizontal stride 2: KW then counts the pair offsets a kernel row touches,
                  // pw is minus the first offset, and the weights hold zeros where half of a pair is no tap)
  int a_sw128;    // A_DENSE_TMA: 1 = the A tile lies in the 128-byte-swizzled K-major layout (rows of 128 bytes)
  int row_kw;     // 0, or KW (even) when the row form is in use
  int row_bytes;  // bytes one row copy delivers: (box_w + KW - 1) * 16
  FastDiv div_n_tiles;      // tile index -> (row block, column block)
  long long acc_bound;  // EPI_REQ_NCHWC: upper bound of |accumulator| (255 * 128 * reduction length)
  int fold_bias;  // 0: the drain always adds the bias
  int a_signed;   // int8 kinds: 1 = the A operand is s8 (0 = u8)
  int mul;        // EPI_MUL_NCHWC: the s32 multiplier
  const uint8_t *residual;  // EPI_RES_NCHWC: u8 tensor in the output's layout
  int tmem_cols;  // TMEM columns to allocate: a power of two >= 32 that holds the accumulator sets
  unsigned long long wait_limit_ns;  // bound of every mbarrier wait
  int inject;     // diagnostics: 1 = the B producer issues nothing (the waits then run out)
  // Split-K (kernel template parameter SPLITK): the CTAs of one thread-block cluster of ksplit CTAs
  // share one tile; CTA `rank` accumulates pipeline stages [rank * ks_per, (rank + 1) * ks_per) and the
  // partial accumulators are exchanged through distributed shared memory (see the kernel)
  int ksplit, ks_per;
  // A_CONV_WIN.  Positions q = oh * win_wp + ow' run over the padded width win_wp = W + 2 pw (the last
  // KW - 1 positions of a row are not outputs); a tile is MT x 128 consecutive positions of one image
  // (win_tpi tiles per image).  For one channel chunk the tile's operand for tap (kh, kw) is the 16-byte
  // pixels q + kh * win_wp + kw of the padded image, so one box copy of win_rows rows of win_wp pixels
  // (zero fill outside the image) serves all taps.  A pipeline stage holds the windows of two chunks
  // (win_bytes each); an MMA K step pairs the same tap of both chunks.
  int win_wp, win_rows, win_bytes, win_tpi;  // win_bytes: distance between the two windows of a stage (a multiple of 128)
  int win_box_bytes;                         // bytes one window copy delivers: win_rows * win_wp * 16
  FastDiv div_wp, div_tpi;
  // Convolution in three dimensions (one image, [c/16][D][H][W][16]): the depth axis takes the place of
  // the image axis of the two-dimensional kernel (a 128-row tile then runs over (od, oh, ow)), kernel
  // depth KD adds a third tap index, and the output strides below place (od, channel group).
  // Two-dimensional calls use KD = 1, sd = 1, pd = 0, out_img_stride = (c_out / 16) * OH * OW,
  // out_grp_stride = OH * OW, src_img_bytes = img_bytes, src_chunk_bytes = H * W * (bytes per chunk pixel).
  int KD, sd, pd;
  long long out_img_stride, out_grp_stride;  // in units of 16 output elements
  long long src_img_bytes, src_chunk_bytes;  // gather paths: bytes between images (depth slices) and channel chunks
  int src_imgs;                              // images (depth slices) of the input
  unsigned long long *trace;  // optional: 8 timestamps (ns) per tile of CTA 0, see unit_trace_attach
  int trace_cap;              // tiles the trace buffer holds
};

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Same test with acquire semantics at cluster scope (the barrier is arrived on by other CTAs).
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Same test, but the thread may stay suspended for up to `hint_ns` before it reports "not yet".
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
// What a bounded wait needs besides the barrier: the CTA's abort flag, the global error word and
// the time limit (1 s in production; the diagnostics hook of the C ABI can shorten it).
struct WaitCtx {
  volatile int *abort_flag;
  unsigned int *err;
  unsigned long long limit_ns;
};
#ifndef UNIT_SPIN_PROBES
#define UNIT_SPIN_PROBES 1
#endif
// Bounded wait: gives up after the limit (or when another role already aborted).  After the first
// probe, retries back off (suspended try_wait plus a short sleep) so that waiting threads leave the
// issue slots and the shared-memory pipe to the warps that have work.  (Measured: eight or
// thirty-two spinning probes before the back-off cost 1.8 % on the batch-256 and batch-32 sweeps.)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx &wc, uint32_t code) {
#pragma unroll 1
  for (int i = 0; i < UNIT_SPIN_PROBES; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t it = 0; it < (1u << 26); ++it) {
    if (mbar_try_wait_hint(bar, parity, kWaitHintNs)) return true;
    __nanosleep(32);
    if ((it & 15u) == 15u) {
      if (*wc.abort_flag) return false;
      if (global_timer_ns() - t0 > wc.limit_ns) break;
    }
  }
  *wc.abort_flag = 1;
  atomicCAS(wc.err, 0u, code);
  return false;
}
// Warp-collective form, called by all 32 lanes together.  Every lane probes the barrier (one
// warp-wide instruction on one address) and the lanes agree by vote, so the warp stays converged.
// Measured: a warp whose lane 0 polls while the other lanes are parked at a warp-level
// synchronisation point runs that lane markedly slower (10-20 % on whole K-loop-bound layers).
// (cluster_scope: the barrier is arrived on by other CTAs of the cluster, whose writes to this CTA's
// shared memory the wait has to acquire.)
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const WaitCtx &wc, uint32_t code,
                                               bool cluster_scope = false) {
#pragma unroll 1
  for (int i = 0; i < UNIT_SPIN_PROBES; ++i)
    if (__all_sync(0xffffffffu, (cluster_scope ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)) ? 1 : 0)) return true;
  const unsigned long long t0 = global_timer_ns();
  bool timed_out = true;
  for (uint32_t it = 0; it < (1u << 26); ++it) {
    if (__all_sync(0xffffffffu, (cluster_scope ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait_hint(bar, parity, kWaitHintNs)) ? 1 : 0))
      return true;
    __nanosleep(32);
    if ((it & 15u) == 15u) {
      if (__any_sync(0xffffffffu, *wc.abort_flag)) { timed_out = false; break; }
      if (__any_sync(0xffffffffu, global_timer_ns() - t0 > wc.limit_ns ? 1 : 0)) break;
    }
  }
  if (timed_out && (threadIdx.x & 31) == 0) {
    *wc.abort_flag = 1;
    atomicCAS(wc.err, 0u, code);
  }
  return false;
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// The barrier receives one arrival from this thread once all of the thread's earlier
// cp.async copies have landed (the pending count is not raised: the arrival is part of
// the count the barrier was initialised with).
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// im2col-mode tensor copy: `pixelsPerColumn` consecutive output positions, starting at the
// filter-window origin (w, h, d) of the first one, tap offset (woff, hoff), channel c of chunk n.
__device__ __forceinline__ void tma_im2col_5d(uint32_t dst, const CUtensorMap *tmap, int c, int w, int h, int d, int n,
                                              uint16_t woff, uint16_t hoff, uint16_t doff, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, "
      "%5, %6}], [%7], {%8, %9, %10};" ::"r"(dst),
      "l"(tmap), "r"(c), "r"(w), "r"(h), "r"(d), "r"(n), "r"(bar), "h"(woff), "h"(hoff), "h"(doff)
      : "memory");
}
// tiled-mode tensor copy of one box of the 4-D tensor (x, y, z, w) = (16-byte units of a pixel row,
// image row, channel chunk, image)
__device__ __forceinline__ void tma_tile_4d(uint32_t dst, const CUtensorMap *tmap, int x, int y, int z, int w,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, "
      "%5}], [%6];" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar)
      : "memory");
}
// tiled-mode tensor copy of one box of a 5-D tensor
__device__ __forceinline__ void tma_tile_5d(uint32_t dst, const CUtensorMap *tmap, int c0, int c1, int c2, int c3, int c4,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], "
      "[%7];" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
      : "memory");
}
// tiled-mode tensor copy of one box of the 2-D tensor (byte of a row, row)
__device__ __forceinline__ void tma_tile_2d(uint32_t dst, const CUtensorMap *tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
// tiled-mode tensor copy of one box of the 3-D tensor (8-byte half of a 16-byte column, column, row)
__device__ __forceinline__ void tma_tile_3d(uint32_t dst, const CUtensorMap *tmap, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], "
      "[%5];" ::"r"(dst),
      "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
template <bool F16>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  if constexpr (F16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
      "%14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
      "%14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
// d = (sat_u16(a) << 16) | sat_u16(b)
__device__ __forceinline__ uint32_t pack_sat_u16(int32_t a, int32_t b) {
  uint32_t d;
  asm("cvt.pack.sat.u16.s32 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// d = (c << 16) | (sat_u8(a) << 8) | sat_u8(b)
__device__ __forceinline__ uint32_t pack_sat_u8(int32_t a, int32_t b, uint32_t c) {
  uint32_t d;
  asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
// true in exactly one lane of the (converged) warp
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0u;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- thread-block cluster / distributed shared memory (split-K) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// 16 bytes into another CTA's shared memory; the copy's completion is counted (as 16 transaction
// bytes) on an mbarrier of that same CTA, so neither a fence nor a separate signal is needed
__device__ __forceinline__ void st_async_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d,
                                            uint32_t cluster_mbar) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];" ::"r"(cluster_addr),
               "r"(a), "r"(b), "r"(c), "r"(d), "r"(cluster_mbar)
               : "memory");
}
// one arrival on an mbarrier of another CTA of the cluster; releases this thread's earlier writes at cluster scope
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void fence_cluster() { asm volatile("fence.acq_rel.cluster;" ::: "memory"); }
// every thread of every CTA of the cluster: nobody leaves while a peer may still touch its shared memory
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Tile trace: CTA 0 records when each role passes a point of tile `lt` (slot 0-7).
__device__ __forceinline__ void trace_mark(const IgemmParams &p, uint32_t lt, int slot) {
  if (p.trace != nullptr && blockIdx.x == 0 && lt < (uint32_t)p.trace_cap) p.trace[lt * 16u + slot] = (unsigned long long)clock64();
}

// Kernel-level marks of CTA 0 in nanoseconds of the global timer (row 0 of the trace, slots 8-11):
// kernel entry, prologue done, predecessor's memory visible, teardown done.
__device__ __forceinline__ void trace_mark_ns(const IgemmParams &p, int slot) {
  if (p.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0 && p.trace_cap > 0) {
    p.trace[slot] = global_timer_ns();
    p.trace[slot + 4] = (unsigned long long)clock64();  // the same moment in SM cycles (slots 12-15)
  }
}

// Shared-memory matrix descriptor, K-major, no swizzle.
//   bits  0-13 start address >> 4      bits 16-29 leading-dimension byte offset >> 4
//   bits 32-45 stride byte offset >> 4 bits 46-47 descriptor version (1 on sm_100)
//   bits 61-63 swizzle mode (0 = none)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
// Shared-memory matrix descriptor, K-major, 128-byte swizzle: a row is 128 bytes of K, eight rows
// form a 1 KB atom whose 16-byte chunks are XOR-permuted by the row number (the layout the copy
// engine writes with CU_TENSOR_MAP_SWIZZLE_128B); consecutive atoms along M are 1 KB apart (SBO).
// A K step of 32 bytes inside the atom is addressed by advancing the start address by 32 bytes.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// The same with 32-byte rows (32-byte swizzle): eight rows form a 256-byte atom; one row is one
// K step (a 32-byte fp16 pixel chunk).
__device__ __forceinline__ uint64_t make_smem_desc_sw32(uint32_t addr) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(256u >> 4) << 32) | (1ull << 46) | (6ull << 61);
}
// Instruction descriptor: D format bits 4-5 (1 = f32, 2 = s32), A format bits 7-9,
// B format bits 10-12 (i8 kinds: 0 = u8, 1 = s8; f16 kind: 0 = fp16), both operands
// K-major (bits 15, 16 = 0), N >> 3 in bits 17-22, M >> 4 in bits 24-28.
template <bool F16>
__device__ __forceinline__ uint32_t make_idesc(int bn, int a_signed) {
  uint32_t d = F16 ? (1u << 4) : ((2u << 4) | ((a_signed ? 1u : 0u) << 7) | (1u << 10));
  d |= (uint32_t)(bn >> 3) << 17;
  d |= (uint32_t)(kTileM >> 4) << 24;
  return d;
}

struct alignas(16) PipeShared {
  int32_t bias[2][2][kBiasSmem];  // [accumulator set][version]: bias (+ rounding constant) where the drain adds it
  int bias_mma[2];                // per accumulator set: the bias goes in through one more MMA K step
  unsigned long long full[kMaxStages];
  unsigned long long empty[kMaxStages];
  unsigned long long tfull[2];
  unsigned long long tempty[2];
  unsigned long long bready[2];  // per accumulator set: the bias of the set's next tile is staged
  unsigned long long xfree[8];   // split-K: peer CTA r's operand ring may be overwritten with partial sums
  unsigned long long xfull;      // split-K: every peer's partial sums for this CTA's columns have arrived
  uint32_t tmem_base;
  int abort_flag;
};

// ---------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------
// Final step of the epilogue for 16 consecutive columns of one row: t = accumulator + bias
// (+ rounding constant), o = the row's element offset in the output (and residual) tensor.
// The sums cannot leave the s32 range in the requantising modes (host-side bound on |acc| plus
// the staging check); in the s32 modes they wrap like the reference's s32 arithmetic.
template <int EPI>
__device__ __forceinline__ void finish_group16(const IgemmParams &p, const uint32_t *t, long long o) {
  if constexpr (!epi_requantises(EPI)) {
    uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<uint32_t *>(p.out) + o);
    if constexpr (EPI == EPI_MUL_NCHWC) {
      const uint32_t m = (uint32_t)p.mul;
#pragma unroll
      for (int q = 0; q < 4; ++q) dst[q] = make_uint4(t[4 * q] * m, t[4 * q + 1] * m, t[4 * q + 2] * m, t[4 * q + 3] * m);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) dst[q] = make_uint4(t[4 * q], t[4 * q + 1], t[4 * q + 2], t[4 * q + 3]);
    }
  } else {
    uint32_t w[4];
    if constexpr (EPI == EPI_RES_NCHWC) {
      // the u8 residual joins after the shift; the saturating pack is the clamp (and the ReLU)
      const uint4 r = *reinterpret_cast<const uint4 *>(p.residual + o);
      const uint32_t res[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int32_t x0 = ((int32_t)t[4 * q] >> p.shift) + (int32_t)(res[q] & 0xffu);
        const int32_t x1 = ((int32_t)t[4 * q + 1] >> p.shift) + (int32_t)((res[q] >> 8) & 0xffu);
        const int32_t x2 = ((int32_t)t[4 * q + 2] >> p.shift) + (int32_t)((res[q] >> 16) & 0xffu);
        const int32_t x3 = ((int32_t)t[4 * q + 3] >> p.shift) + (int32_t)(res[q] >> 24);
        w[q] = pack_sat_u8(x1, x0, pack_sat_u8(x3, x2, 0u));
      }
    } else if (p.shift == 8) {
      // clamp to [0, 65535] while packing pairs, then keep the high byte of each half-word:
      // min(max(x, 0), 65535) >> 8 == min(max(x >> 8, 0), 255)
#pragma unroll
      for (int q = 0; q < 4; ++q)
        w[q] = __byte_perm(pack_sat_u16((int32_t)t[4 * q + 1], (int32_t)t[4 * q]),
                           pack_sat_u16((int32_t)t[4 * q + 3], (int32_t)t[4 * q + 2]), 0x7531);
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        w[q] = pack_sat_u8((int32_t)t[4 * q + 1] >> p.shift, (int32_t)t[4 * q] >> p.shift,
                           pack_sat_u8((int32_t)t[4 * q + 3] >> p.shift, (int32_t)t[4 * q + 2] >> p.shift, 0u));
    }
    *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.out) + o) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

// The 32-bit epilogues' store of one 16-column group, regrouped through shared memory.  A thread
// holds 64 bytes of its own row; stored as they are, one warp instruction would touch 32 separate
// rows with 16 bytes each.  Instead the rows go through a 1 KB scratch block of the warp, sixteen
// at a time, and come back so that four neighbouring lanes hold one row's 64 bytes: a warp
// instruction then writes eight rows' 64-byte runs (a quarter of the cache lines touched).
//   xs    : the warp's scratch block (shared-memory address)
//   v     : this lane's 16 words;  o_k / ok_k: for k = half * 2 + j, the element offset in the output
//           of row 16 * half + 8 * j + lane / 4 plus 4 * (lane % 4), and whether that row exists
// The 16-byte chunks of a row are stored at chunk ^ ((row / 2) % 4), which keeps both the row-wise
// writes and the regrouped reads free of bank conflicts.
__device__ __forceinline__ void store_group16_regrouped(uint32_t *out, uint32_t xs, int lane, const uint32_t *v,
                                                        const long long (&o_k)[4], const bool (&ok_k)[4], long long goff) {
  const uint32_t wr = xs + (uint32_t)(lane & 15) * 64u;
  const uint32_t wsw = (uint32_t)(lane >> 1) & 3u;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    if ((lane >> 4) == half) {
#pragma unroll
      for (uint32_t c = 0; c < 4u; ++c) st_shared_v4(wr + ((c ^ wsw) << 4), v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const uint32_t row = (uint32_t)(8 * j + (lane >> 2));
      const uint4 t = ld_shared_v4(xs + row * 64u + ((((uint32_t)lane & 3u) ^ ((row >> 1) & 3u)) << 4));
      if (ok_k[half * 2 + j]) *reinterpret_cast<uint4 *>(out + o_k[half * 2 + j] + goff) = t;
    }
    __syncwarp();
  }
}

// The requantising epilogue's commonest case in one piece: shift 8, bias and rounding constant
// already inside the accumulator.  16 s32 sums -> 16 u8, clamp(x >> 8, 0, 255).
__device__ __forceinline__ uint4 pack16_shift8(const uint32_t *t) {
  uint32_t w[4];
#pragma unroll
  for (int q = 0; q < 4; ++q)
    w[q] = __byte_perm(pack_sat_u16((int32_t)t[4 * q + 1], (int32_t)t[4 * q]),
                       pack_sat_u16((int32_t)t[4 * q + 3], (int32_t)t[4 * q + 2]), 0x7531);
  return make_uint4(w[0], w[1], w[2], w[3]);
}
// The same with a u8 residual added after the shift: clamp((x >> 8) + r, 0, 255) = clamp((x + 256 r) >> 8, 0, 255),
// so the residual byte joins its sum one byte up and the pack stays as it is.  (x + 256 r cannot leave s32: the
// host bounds |x| below 2^30 on this path.)
__device__ __forceinline__ uint4 pack16_shift8_res(const uint32_t *t, uint4 r) {
  const uint32_t res[4] = {r.x, r.y, r.z, r.w};
  uint32_t w[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t x0 = t[4 * q] + __byte_perm(res[q], 0u, 0x4404), x1 = t[4 * q + 1] + __byte_perm(res[q], 0u, 0x4414);
    const uint32_t x2 = t[4 * q + 2] + __byte_perm(res[q], 0u, 0x4424), x3 = t[4 * q + 3] + __byte_perm(res[q], 0u, 0x4434);
    w[q] = __byte_perm(pack_sat_u16((int32_t)x1, (int32_t)x0), pack_sat_u16((int32_t)x3, (int32_t)x2), 0x7531);
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// Epilogue for 16 consecutive columns of one row: v = accumulator words, bias_s = this
// group's 16 staged bias values in shared memory (bias + rounding constant for the
// requantising epilogues).
template <int EPI>
__device__ __forceinline__ void store_group16(const IgemmParams &p, const int32_t *bias_s, bool folded, bool wide,
                                              const uint32_t *v, long long o) {
  if (EPI == EPI_RAW_ROWS || folded) {
    // the accumulator is final: bias and rounding constant, if any, came in through the MMA
    finish_group16<EPI>(p, v, o);
    return;
  }
  int32_t bv[16];
  const int4 *bp = reinterpret_cast<const int4 *>(bias_s);
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int4 t = bp[q];  // same address in every lane: a broadcast read
    bv[4 * q] = t.x; bv[4 * q + 1] = t.y; bv[4 * q + 2] = t.z; bv[4 * q + 3] = t.w;
  }
  if (!epi_requantises(EPI) || !wide) {
    uint32_t t[16];
#pragma unroll
    for (int q = 0; q < 16; ++q) t[q] = v[q] + (uint32_t)bv[q];
    finish_group16<EPI>(p, t, o);
    return;
  }
  if constexpr (epi_requantises(EPI)) {
    // bv holds the plain bias: 64-bit sum, for shifts and magnitudes the 32-bit path cannot take
    const long long rnd = 1ll << (p.shift - 1);
    uint32_t res[4] = {0u, 0u, 0u, 0u};
    if constexpr (EPI == EPI_RES_NCHWC) {
      const uint4 r = *reinterpret_cast<const uint4 *>(p.residual + o);
      res[0] = r.x; res[1] = r.y; res[2] = r.z; res[3] = r.w;
    }
    uint32_t w[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t packed = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        long long t = (long long)(int32_t)v[4 * q + e] + (long long)bv[4 * q + e] + rnd;
        t >>= p.shift;
        if constexpr (EPI == EPI_RES_NCHWC) t += (long long)((res[q] >> (8 * e)) & 0xffu);
        t = t < 0 ? 0 : (t > 255 ? 255 : t);
        packed |= (uint32_t)t << (8 * e);
      }
      w[q] = packed;
    }
    *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.out) + o) = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// Prepares the bias of one accumulator set's columns for the tile that will use the set next.
// Called with all lanes by each of the `gw` drain warps that serve the set (wl = 0 .. gw-1); the
// warps work independently (no CTA barrier).
//
// Preferred form: bias (plus the rounding constant 2^(shift-1) when requantising) enters the
// accumulator as one more K step of the MMA.  The A side of that step is a constant block whose
// every row holds the bytes {1, 128, 128, ... 128} (second 16-byte column: zeros); the B side
// holds, per output channel, sixteen s8 digits {d0, d1 ... d15} with
//     d0 + 128 * (d1 + ... + d15) == value,   0 <= d0 < 128,  -128 <= dj <= 127,
// which exists for -245760 <= value <= 243967.  The drain then stores the accumulator as it is.
// If a value of the block does not fit (or the 64-bit requantisation is needed) the values go to
// ps->bias[slot][version] as integers and the drain adds them.
//
// Every warp reads all of the block's values to reach the same verdict (folded / wide) by warp
// votes; warp wl then writes its 256 / gw channels.  The writes become visible to the MMA
// warp through this warp's arrival on the set's "empty" barrier.
template <int EPI>
__device__ __forceinline__ void stage_bias(const IgemmParams &p, PipeShared *ps, uint8_t *fold_mem, uint32_t slot,
                                           uint32_t version, int n_tile, int wl, int gw, int lane, bool &folded,
                                           bool &wide) {
  constexpr bool kReq = epi_requantises(EPI);
  if (!kReq && p.bias == nullptr) {  // nothing to add at all: the accumulator is final without an extra step
    folded = true;
    wide = false;
    if (wl == 0 && lane == 0) ps->bias_mma[slot] = 0;
    return;
  }
  const bool static_wide = kReq && (p.shift > 23 || p.acc_bound >= (1ll << 30));
  const long long rnd = kReq ? (1ll << (p.shift - 1)) : 0ll;
  const int col0 = n_tile * p.bn;
  bool fits = !static_wide && p.fold_bias != 0, need_wide = static_wide;
#pragma unroll
  for (int i = 0; i < kBiasSmem / 32; ++i) {
    const int ch = lane + 32 * i;
    const int32_t b = (ch < p.bn && p.bias != nullptr && col0 + ch < p.n_total) ? __ldg(p.bias + col0 + ch) : 0;
    const long long v = (long long)b + rnd;
    const long long hi = v >> 7;
    fits = fits && hi >= -1920 && hi <= 1905;
    if (kReq) {
      const long long mag = v < 0 ? -v : v;
      need_wide = need_wide || (mag + p.acc_bound >= (1ll << 31));
    }
  }
  fits = __all_sync(0xffffffffu, fits ? 1 : 0) != 0;
  need_wide = __any_sync(0xffffffffu, need_wide ? 1 : 0) != 0;
  const int per_warp = kBiasSmem / gw;  // 16 or 32 channels
  const int ch = wl * per_warp + lane;
  if (lane < per_warp && ch < p.bn) {
    const int32_t b = (p.bias != nullptr && col0 + ch < p.n_total) ? __ldg(p.bias + col0 + ch) : 0;
    if (fits) {
      const int v = b + (int)rnd;
      const int hi = v >> 7, d0 = v & 127;
      const int q = hi / 15, rem = hi - 15 * q;  // hi = 15 q + rem, |rem| < 15, rem has the sign of hi
      const int extra = rem < 0 ? -rem : rem, step = rem < 0 ? -1 : 1;
      uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int d = j == 0 ? d0 : q + (j <= extra ? step : 0);
        w[j >> 2] |= (uint32_t)(d & 0xff) << (8 * (j & 3));
      }
      *reinterpret_cast<uint4 *>(fold_mem + (size_t)slot * kFoldBBytes + (size_t)ch * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      ps->bias[slot][version][ch] = (kReq && !need_wide) ? (int32_t)((long long)b + rnd) : b;
    }
  }
  if (wl == 0 && lane == 0) ps->bias_mma[slot] = fits ? 1 : 0;
  fence_proxy_async();  // the digits are read by the tensor core (async proxy)
  folded = fits;
  wide = need_wide;
}

template <int AMODE, int EPI, bool F16, int MT, bool SPLITK = false>
__global__ void __launch_bounds__(kNumThreads, 1)
    igemm_kernel(const IgemmParams p, const __grid_constant__ CUtensorMap tmap) {
  static_assert(!SPLITK || (MT == 1 && ((a_mode_uses_tma(AMODE) && AMODE != A_CONV_WIN) || AMODE == A_CONV_I8)),
                "split-K: single sub-tiles; tensor-copy-fed A operand (not the window form) or the u8 gather");
  extern __shared__ __align__(1024) uint8_t smem[];  // (1 KB: a swizzled operand atom is 8 rows x 128 bytes)
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  trace_mark_ns(p, 8);

  constexpr uint32_t kSubBytes = kTileM * 16u;                       // one K column of one 128-row sub-tile
  // (window form: a stage's A part is the two chunk windows; the sub-tiles are 128-row slices of them)
  const uint32_t a_sub_bytes = AMODE == A_CONV_WIN ? kSubBytes : (uint32_t)p.kc * kSubBytes;  // one sub-tile of one stage
  const uint32_t a_stage_bytes = AMODE == A_CONV_WIN ? 2u * (uint32_t)p.win_bytes : (uint32_t)MT * a_sub_bytes;
  const uint32_t b_stage_bytes = (uint32_t)p.kc * (uint32_t)p.bn * 16u;
  const uint32_t stage_bytes = a_stage_bytes + b_stage_bytes;
  PipeShared *ps = reinterpret_cast<PipeShared *>(smem + (size_t)p.stages * stage_bytes + kFoldBytes);
  const uint32_t smem_base = smem_u32(smem);
  volatile int *abort_flag = &ps->abort_flag;
  const WaitCtx wc{abort_flag, p.err, p.wait_limit_ns};
  // accumulator sets that fit in the 512 TMEM columns (2 = drain overlaps the next main loop)
  // (split-K: a CTA has one tile only, so one set and all sixteen warps drain it)
  const uint32_t nslots = (!SPLITK && (512u / ((uint32_t)MT * (uint32_t)p.bn)) >= 2u) ? 2u : 1u;
  // Split-K: the cluster's CTAs share tile (cluster index); this CTA's stages are [ks_begin, ks_end).
  // Otherwise tiles are dealt round-robin over the grid.
  const uint32_t crank = SPLITK ? cluster_ctarank() : 0u;
  const int tile0 = SPLITK ? (int)(blockIdx.x / (uint32_t)p.ksplit) : (int)blockIdx.x;
  const int ks_begin = SPLITK ? (int)crank * p.ks_per : 0;
  const int ks_end = SPLITK ? min(ks_begin + p.ks_per, p.k_stages) : p.k_stages;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      // 128 A-producer threads + the B producer; with TMA-fed A only the thread that issues all copies
      mbar_init(smem_u32(&ps->full[s]), a_mode_uses_tma(AMODE) ? 2 : 128 + 1);
      mbar_init(smem_u32(&ps->empty[s]), MT);      // one tcgen05.commit per MMA-issuing thread
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&ps->tfull[i]), 1 + MT);        // the first issuing thread's arrival + one commit per issuer
      mbar_init(smem_u32(&ps->tempty[i]), kDrainWarps / nslots);  // the drain warps that serve the set
      mbar_init(smem_u32(&ps->bready[i]), kDrainWarps / nslots);
    }
    if constexpr (SPLITK) {
      for (int i = 0; i < 8; ++i) mbar_init(smem_u32(&ps->xfree[i]), 1);
      mbar_init(smem_u32(&ps->xfull), 1);  // this CTA's own arrival, which also announces the bytes to come
    }
    ps->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&ps->tmem_base), (uint32_t)p.tmem_cols);
    tmem_relinquish();
    if constexpr (!F16 && EPI != EPI_RAW_ROWS) {
      // the constant A block of the bias step: column 0 = bytes {1, 128 x 15} in every row, column 1 = zeros
      uint4 *ac = reinterpret_cast<uint4 *>(smem + (size_t)p.stages * stage_bytes + 2 * kFoldBBytes);
      for (int i = lane; i < 2 * kTileM; i += 32)
        ac[i] = i < kTileM ? make_uint4(0x80808001u, 0x80808080u, 0x80808080u, 0x80808080u) : make_uint4(0u, 0u, 0u, 0u);
      fence_proxy_async();
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ps->tmem_base;
  if constexpr (SPLITK) cluster_sync_all();  // every peer's barriers exist before anybody arrives on them
  // From here on this CTA holds its tensor memory, so a dependent kernel's CTA that becomes
  // resident on the same SM can never be the one that keeps this CTA waiting in tcgen05.alloc:
  // let the next kernel of the stream start its own prologue as soon as SMs become free.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  trace_mark_ns(p, 9);
  // Programmatic dependent launch: everything above touched only this CTA's shared memory and
  // TMEM, so it may run while the previous kernel in the stream is still finishing; from here
  // on global memory is read and written, which has to wait for that kernel's completion.
  // (A no-op when the kernel was launched without the attribute.)
  asm volatile("griddepcontrol.wait;" ::: "memory");
  trace_mark_ns(p, 10);

  const int total_tiles = p.m_tiles * p.n_tiles;
  const int tstep = SPLITK ? total_tiles : (int)gridDim.x;  // split-K: exactly one tile per CTA

  if (!a_mode_uses_tma(AMODE) && warp >= kFirstProducerWarp && warp < kFirstProducerWarp + 4) {
    // ===================== A producers =====================
    const int pw = warp - kFirstProducerWarp;
    uint32_t s = 0, ring_phase = 0;  // ring position and the number of wraps (mod 2)
    uint32_t lt = 0;
    bool alive = true;
    for (int tile = tile0; tile < total_tiles && alive; tile += tstep, ++lt) {
      const int m_tile = (int)fast_div((uint32_t)tile, p.div_n_tiles);
      const long long m0 = (long long)m_tile * (kTileM * MT);

      // rows this lane feeds (per sub-tile) and their decoded positions
      constexpr int RPT = (AMODE == A_CONV_I8 || AMODE == A_STEM_I8) ? 1 : (AMODE == A_CONV_F16 ? 2 : 4);
      int row[RPT];
      bool rvalid[MT][RPT];
      const uint8_t *rbase[MT][RPT];
      int ih0[MT][RPT], iw0[MT][RPT], id0[MT][RPT];
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        if constexpr (AMODE == A_CONV_I8 || AMODE == A_STEM_I8) row[i] = pw * 32 + lane;
        else if constexpr (AMODE == A_CONV_F16) row[i] = pw * 32 + i * 16 + (lane >> 4) * 8 + (lane & 7);
        else row[i] = pw * 32 + i * 8 + (lane & 7);
#pragma unroll
        for (int t = 0; t < MT; ++t) {
          const long long m = m0 + t * kTileM + row[i];
          rvalid[t][i] = m < p.m_total;
          if constexpr (AMODE == A_DENSE) {
            rbase[t][i] = p.a + (rvalid[t][i] ? m : 0) * p.lda;
            ih0[t][i] = iw0[t][i] = id0[t][i] = 0;
          } else {
            // m_total < 2^31 is checked on the host: 32-bit divisions
            const unsigned mm = rvalid[t][i] ? (unsigned)m : 0u;
            const unsigned ohw = (unsigned)(p.OH * p.OW);
            const int n_img = (int)(mm / ohw);
            const int rem = (int)(mm - (unsigned)n_img * ohw);
            const int oh = rem / p.OW, ow = rem - oh * p.OW;
            ih0[t][i] = oh * p.sh - p.ph;
            iw0[t][i] = ow * p.sw - p.pw;
            // (three dimensions: n_img is the output depth; the first input slice is n_img * sd - pd)
            id0[t][i] = n_img * p.sd - p.pd;
            rbase[t][i] = p.a + (long long)id0[t][i] * p.src_img_bytes;
          }
        }
      }

      if (threadIdx.x == kFirstProducerWarp * 32) trace_mark(p, lt, 0);
      int ci = 0, kh = 0, kw = 0, kd = 0;  // position of the next K column (conv modes)
      if constexpr (AMODE == A_CONV_I8) {
        // (split-K: this CTA's part of the reduction starts at column ks_begin * kc)
        const int col0 = ks_begin * p.kc, tap = col0 / p.Cc;
        ci = col0 - tap * p.Cc;
        kw = tap % p.KW;
        kh = (tap / p.KW) % p.KH;
        kd = tap / (p.KW * p.KH);
      }
      for (int ks = ks_begin; ks < ks_end; ++ks) {
        if (!mbar_wait_warp(smem_u32(&ps->empty[s]), ring_phase ^ 1u, wc, kErrWaitEmpty)) {
          alive = false;
          break;
        }
        const uint32_t a_dst = smem_base + s * stage_bytes;
        if constexpr (AMODE == A_CONV_I8) {
          for (int jj = 0; jj < p.kc; ++jj) {
            const int j = ks * p.kc + jj;
#pragma unroll
            for (int t = 0; t < MT; ++t) {
              const int ih = ih0[t][0] + kh, iw = iw0[t][0] + kw;
              const bool ok = rvalid[t][0] && j < p.cols && (unsigned)ih < (unsigned)p.H && (unsigned)iw < (unsigned)p.W &&
                              (unsigned)(id0[t][0] + kd) < (unsigned)p.src_imgs;
              const uint8_t *src = ok ? rbase[t][0] + (long long)kd * p.src_img_bytes + (long long)ci * p.src_chunk_bytes +
                                            ((long long)ih * p.W + iw) * 16
                                      : p.a;
              cp_async16(a_dst + (uint32_t)t * a_sub_bytes + (uint32_t)jj * kSubBytes + (uint32_t)row[0] * 16u, src,
                         ok ? 16u : 0u);
            }
            if (++ci == p.Cc) { ci = 0; if (++kw == p.KW) { kw = 0; if (++kh == p.KH) { kh = 0; ++kd; } } }
          }
        } else if constexpr (AMODE == A_CONV_F16) {
          const int half = (lane >> 3) & 1;
          for (int jj = 0; jj < p.kc; jj += 2) {
            const int j = ks * p.kc + jj;
#pragma unroll
            for (int t = 0; t < MT; ++t) {
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                const int ih = ih0[t][i] + kh, iw = iw0[t][i] + kw;
                const bool ok =
                    rvalid[t][i] && j < p.cols && (unsigned)ih < (unsigned)p.H && (unsigned)iw < (unsigned)p.W;
                const uint8_t *src = ok ? rbase[t][i] + ((long long)(ci * p.H + ih) * p.W + iw) * 32 + half * 16 : p.a;
                cp_async16(a_dst + (uint32_t)t * a_sub_bytes + (uint32_t)(jj + half) * kSubBytes + (uint32_t)row[i] * 16u,
                           src, ok ? 16u : 0u);
              }
            }
            if (++ci == p.Cc) { ci = 0; if (++kw == p.KW) { kw = 0; ++kh; } }
          }
        } else if constexpr (AMODE == A_STEM_I8) {
          // column = (ci, kh, group of 4 kw taps); ci / kh / kw track (chunk, kh, group)
          for (int jj = 0; jj < p.kc; ++jj) {
            const int j = ks * p.kc + jj;
#pragma unroll
            for (int t = 0; t < MT; ++t) {
              const int ih = ih0[t][0] + kh;
              const bool rok = rvalid[t][0] && j < p.cols && (unsigned)ih < (unsigned)p.H;
              const uint32_t dst = a_dst + (uint32_t)t * a_sub_bytes + (uint32_t)jj * kSubBytes + (uint32_t)row[0] * 16u;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int tap = kw * 4 + q;
                const int iw = iw0[t][0] + tap;
                const bool ok = rok && tap < p.KW && (unsigned)iw < (unsigned)p.W;
                const uint8_t *src = ok ? rbase[t][0] + ((long long)(ci * p.H + ih) * p.W + iw) * 4 : p.a;
                cp_async4(dst + q * 4u, src, ok ? 4u : 0u);
              }
            }
            if (++kw == p.kwg) { kw = 0; if (++kh == p.KH) { kh = 0; ++ci; } }
          }
        } else {  // A_DENSE: 8 rows x 4 columns per warp instruction
          const int csub = lane >> 3;
          for (int jj = 0; jj < p.kc; jj += 4) {
            const int jl = jj + csub;
            const int j = ks * p.kc + jl;
            if (jl < p.kc) {
#pragma unroll
              for (int t = 0; t < MT; ++t) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const bool ok = rvalid[t][i] && j < p.cols;
                  const uint8_t *src = ok ? rbase[t][i] + (long long)j * 16 : p.a;
                  cp_async16(a_dst + (uint32_t)t * a_sub_bytes + (uint32_t)jl * kSubBytes + (uint32_t)row[i] * 16u, src,
                             ok ? 16u : 0u);
                }
              }
            }
          }
        }
        cp_async_arrive_noinc(smem_u32(&ps->full[s]));
        if (++s == (uint32_t)p.stages) { s = 0; ring_phase ^= 1u; }
      }
      if (threadIdx.x == kFirstProducerWarp * 32) trace_mark(p, lt, 1);
    }
    cp_async_wait<0>();  // nothing of this thread is in flight when the CTA winds down
  } else if (a_mode_uses_tma(AMODE) && warp >= kFirstProducerWarp && warp < kFirstProducerWarp + 4) {
    // ===================== A copies by TMA =====================
    // One tensor copy brings one K column of one sub-tile (2 KB at most).  Measured: a thread
    // needs ~330 cycles per copy and a warp ~70, so the copies of a stage (column x sub-tile)
    // are dealt round-robin to the four producer warps and, within a warp, to its lanes; each
    // warp then issues its share with one instruction.
    const int copy_id = lane * 4 + (warp - kFirstProducerWarp);
    const int jj = copy_id / MT, t = copy_id % MT;
    const bool lane_active = jj < p.kc;
    const bool tx_poster = warp == kFirstProducerWarp && lane == 0;  // announces the stage's A bytes
    uint32_t s = 0, ring_phase = 0;
    uint32_t lt = 0;
    bool alive = true;
    // What does not depend on the tile is computed once (a short-reduction layer has thousands of tiles per
    // CTA, and the integer divisions below cost this warp more than issuing a tile's copies does).
    // This lane's K column: chunk position (ci, kw, kh, kd) of its first column and, for fp16, which 16-byte
    // half (box mode: jj counts chunks, which for fp16 are whole K steps of two columns).
    // Row form: jj counts kernel rows of the stage, each copied once into the slot of its first column.
    const bool row_form = AMODE == A_CONV_BOX && p.row_kw > 0;
    const int rows_per_stage = row_form ? p.kc / p.row_kw : 0;
    const int cpc = (AMODE == A_CONV_BOX || AMODE == A_DENSE_TMA || AMODE == A_CONV_WIN) ? 1 : p.cols_per_chunk;
    const int half = jj % cpc;
    const bool rows32 = AMODE == A_CONV_BOX && (F16 || p.a_sw32 != 0);  // one copy per K step of 32-byte rows
    const int chunk_step = rows32 ? p.kc / 2 : p.kc / cpc;
    int kh0 = 0, kw0 = 0, ci0 = 0, kd0 = 0;
    if (AMODE != A_DENSE_TMA && AMODE != A_CONV_WIN && !row_form) {
      const int q0 = jj / cpc + ks_begin * chunk_step;  // chunk index along K of this lane's first column
      const int tap = q0 / p.Cc;                        // taps run (kd, kh, kw), kw fastest
      ci0 = q0 - tap * p.Cc;
      kw0 = tap % p.KW;
      kh0 = (tap / p.KW) % p.KH;
      kd0 = tap / (p.KW * p.KH);
    }
    const uint32_t box_copy_bytes = AMODE == A_CONV_BOX ? (uint32_t)(p.box_n * p.box_h * p.box_w) * 16u : kSubBytes;
    for (int tile = tile0; tile < total_tiles && alive; tile += tstep, ++lt) {
      const int m_tile = (int)fast_div((uint32_t)tile, p.div_n_tiles);
      if constexpr (AMODE == A_CONV_WIN) {
        // two box copies per stage (one per channel chunk), issued by lane 0 of the first two producer warps
        const uint32_t img = fast_div((uint32_t)m_tile, p.div_tpi);
        const uint32_t q0 = ((uint32_t)m_tile - img * (uint32_t)p.win_tpi) * (uint32_t)(kTileM * MT);
        const int y0 = (int)fast_div(q0, p.div_wp) - p.ph;
        for (int ks = ks_begin; ks < ks_end; ++ks) {
          if (!mbar_wait_warp(smem_u32(&ps->empty[s]), ring_phase ^ 1u, wc, kErrWaitEmpty)) {
            alive = false;
            break;
          }
          const uint32_t bar = smem_u32(&ps->full[s]);
          if (tx_poster) mbar_arrive_expect_tx(bar, 2u * (uint32_t)p.win_box_bytes);
          __syncwarp();
          if (lane == 0 && copy_id < 2)
            tma_tile_4d(smem_base + s * stage_bytes + (uint32_t)copy_id * (uint32_t)p.win_bytes, &tmap, -2 * p.pw, y0,
                        2 * ks + copy_id, (int)img, bar);
          if (++s == (uint32_t)p.stages) { s = 0; ring_phase ^= 1u; }
        }
        if (tx_poster) trace_mark(p, lt, 1);
        continue;
      }
      // origin of this lane's sub-tile
      int c0 = 0, c1 = 0, c2 = 0;  // BOX: x (8-byte units), y, first image; TMA: w, h, image
      bool sub_ok = true;
      if constexpr (AMODE == A_DENSE_TMA) {
        c0 = (m_tile * MT + t) * kTileM;  // first row of this lane's sub-tile; rows past the end are zero-filled
      } else if constexpr (AMODE == A_CONV_BOX) {
        long long st = (long long)m_tile * MT + t;
        sub_ok = st < p.sub_tiles;
        if (!sub_ok) st = 0;
        const uint32_t q = fast_div((uint32_t)st, p.div_blocks_w);
        const uint32_t wb = (uint32_t)st - q * (uint32_t)p.blocks_w;
        const uint32_t nb = fast_div(q, p.div_blocks_h);
        const uint32_t hb = q - nb * (uint32_t)p.blocks_h;
        c0 = ((int)wb * p.box_w - p.pw) * (rows32 ? 1 : 2);  // u8: 8-byte units of a pixel row; 32-byte rows: pixels (pairs)
        c1 = (int)hb * p.box_h * p.sh - p.ph;                 // (vertical stride: the box takes every sh-th row)
        c2 = (int)nb * p.box_n - p.pd;
      } else {
        long long m = ((long long)m_tile * MT + t) * kTileM;
        if (m >= p.m_total) m = 0;  // a sub-tile past the end: fetch valid data, nothing of it is stored
        const uint32_t n_img = fast_div((uint32_t)m, p.div_ohw);
        const uint32_t rem = (uint32_t)m - n_img * (uint32_t)(p.OH * p.OW);
        const uint32_t oh = fast_div(rem, p.div_ow);
        const uint32_t ow = rem - oh * (uint32_t)p.OW;
        c0 = (int)ow * p.sw - p.pw;
        c1 = (int)oh * p.sh - p.ph;
        c2 = (int)n_img * p.sd - p.pd;
      }
      // sub-tiles that exist in this tile, and the bytes one copy delivers
      int nsub = MT;
      const uint32_t copy_bytes = box_copy_bytes;
      if constexpr (AMODE == A_CONV_BOX) {
        const long long left = p.sub_tiles - (long long)m_tile * MT;
        nsub = left < MT ? (int)left : MT;
      }
      int kh = kh0, kw = kw0, ci = ci0, kd = kd0;
      for (int ks = ks_begin; ks < ks_end; ++ks) {
        if (!mbar_wait_warp(smem_u32(&ps->empty[s]), ring_phase ^ 1u, wc, kErrWaitEmpty)) {
          alive = false;
          break;
        }
        const uint32_t bar = smem_u32(&ps->full[s]);
        int real = p.cols - ks * p.kc;  // columns of this stage that exist (the rest only meets zero weights)
        real = real < 0 ? 0 : (real > p.kc ? p.kc : real);
        if (AMODE == A_DENSE_TMA && p.a_sw128 != 0) {
          // one copy = 128 rows x 128 bytes of K (8 columns) of one sub-tile, written swizzled
          const int atoms = p.kc >> 3;
          if (tx_poster) mbar_arrive_expect_tx(bar, (uint32_t)(atoms * nsub) * 16384u);
          __syncwarp();
          if (jj < atoms) {
            const uint32_t dst = smem_base + s * stage_bytes + (uint32_t)t * a_sub_bytes + (uint32_t)jj * 16384u;
            tma_tile_2d(dst, &tmap, (ks * p.kc + jj * 8) * 16, c0, bar);
          }
        } else if (rows32) {
          // fp16 pixels or u8 pixel pairs: one copy per K step (32 bytes per row), written swizzled
          const int steps = real >> 1;
          if (tx_poster) mbar_arrive_expect_tx(bar, (uint32_t)(steps * nsub) * copy_bytes * 2u);
          __syncwarp();
          if (jj < steps && sub_ok) {
            const uint32_t dst = smem_base + s * stage_bytes + (uint32_t)t * a_sub_bytes + (uint32_t)jj * 2u * kSubBytes;
            tma_tile_5d(dst, &tmap, 0, c0 + kw, c1 + kh, ci, c2 + kd, bar);
          }
        } else if (row_form) {
          if (tx_poster) mbar_arrive_expect_tx(bar, (uint32_t)(rows_per_stage * nsub) * (uint32_t)p.row_bytes);
          __syncwarp();
          if (jj < rows_per_stage && sub_ok) {
            const uint32_t dst = smem_base + s * stage_bytes + (uint32_t)t * a_sub_bytes +
                                 (uint32_t)(jj * p.row_kw) * kSubBytes;
            tma_tile_4d(dst, &tmap, c0, c1 + ks * rows_per_stage + jj, 0, c2, bar);
          }
        } else {
          if (tx_poster) mbar_arrive_expect_tx(bar, (uint32_t)(real * nsub) * copy_bytes);
          __syncwarp();
          if (lane_active && jj < real && (AMODE != A_CONV_BOX || sub_ok)) {
            const uint32_t dst = smem_base + s * stage_bytes + (uint32_t)t * a_sub_bytes + (uint32_t)jj * kSubBytes;
            if constexpr (AMODE == A_DENSE_TMA)
              tma_tile_3d(dst, &tmap, 0, ks * p.kc + jj, c0, bar);
            else if constexpr (AMODE == A_CONV_BOX)
              tma_tile_4d(dst, &tmap, c0 + kw * 2, c1 + kh, ci, c2 + kd, bar);
            else
              tma_im2col_5d(dst, &tmap, half * 8, c0, c1, c2, ci, (uint16_t)kw, (uint16_t)kh, (uint16_t)kd, bar);
          }
        }
        // advance this lane's column by one stage
        if (AMODE != A_DENSE_TMA && !row_form) {
          ci += chunk_step;
          while (ci >= p.Cc) { ci -= p.Cc; if (++kw == p.KW) { kw = 0; if (++kh == p.KH) { kh = 0; ++kd; } } }
        }
        if (++s == (uint32_t)p.stages) { s = 0; ring_phase ^= 1u; }
      }
      if (tx_poster) trace_mark(p, lt, 1);
    }
  } else if (warp == kBWarp) {
    // ===================== B producer =====================
    // (p.inject: diagnostics.  The producer issues nothing, so no stage ever completes and the
    // bounded waits of the other roles run out: the path that reports UNIT_ERR_DEVICE_WAIT.)
    if (lane == 0 && p.inject == 0) {
      uint32_t s = 0, ring_phase = 0;
      uint32_t lt = 0;
      bool alive = true;
      for (int tile = tile0; tile < total_tiles && alive; tile += tstep, ++lt) {
        const int n_tile = tile - (int)fast_div((uint32_t)tile, p.div_n_tiles) * p.n_tiles;
        const uint8_t *src = p.b + (size_t)n_tile * p.k_stages * b_stage_bytes;
        for (int ks = ks_begin; ks < ks_end; ++ks) {
          if (!mbar_wait(smem_u32(&ps->empty[s]), ring_phase ^ 1u, wc, kErrWaitEmpty)) {
            alive = false;
            break;
          }
          const uint32_t bar = smem_u32(&ps->full[s]);
          mbar_arrive_expect_tx(bar, b_stage_bytes);
          bulk_copy_g2s(smem_base + s * stage_bytes + a_stage_bytes, src + (size_t)ks * b_stage_bytes,
                        b_stage_bytes, bar);
          if (++s == (uint32_t)p.stages) { s = 0; ring_phase ^= 1u; }
        }
        trace_mark(p, lt, 2);
      }
    }
  } else if (warp == kMmaWarp || (MT == 2 && warp == kMmaWarp2)) {
    // ===================== MMA issuers =====================
    // One warp per sub-tile issues that sub-tile's MMAs (two warps issue independently: a 128 x 64 x 32 MMA
    // is 32 cycles of math, less than one warp's issue interval).  The warp runs the loop converged
    // (UNIT_MMA_CONVERGED): all 32 lanes wait on the barriers together and compute the same descriptor
    // addresses, and one elected lane executes the MMA, commit and arrive instructions.  Measured against
    // the earlier form, where lane 0 ran the loop alone inside a lane-divergent branch while the other lanes
    // waited at the final CTA barrier: 10-30 % less time per tile on short reductions (descriptor arithmetic
    // that is provably warp-uniform does not pass through per-lane registers on its way to the instruction).
    // (A third form, the other lanes parked at a warp-level synchronisation point while lane 0 polls, was
    // 10-20 % slower than either.)
    constexpr bool kCanFold = !F16 && EPI != EPI_RAW_ROWS;
    // Operand descriptors carry the shared-memory address as a 14-bit field (bits 4-17 of the offset in
    // this CTA's window).  In a thread-block cluster the 32-bit shared address of a CTA other than the
    // first has higher bits set (the CTA's place in the cluster's window), which must not leak into
    // the neighbouring descriptor fields: descriptor arithmetic uses the offset alone.
    const uint32_t desc_base = smem_base & 0x3FFFFu;
    const uint32_t fold_base = desc_base + (uint32_t)p.stages * stage_bytes;  // [B digits set 0][set 1][A constants]
    const uint32_t my_t = warp == kMmaWarp ? 0u : 1u;  // the sub-tile this thread issues for
#ifndef UNIT_MMA_CONVERGED
#define UNIT_MMA_CONVERGED 1
#endif
    // UNIT_MMA_CONVERGED: all 32 lanes run the issue loop together (waits are warp-collective, addresses are
    // warp-uniform) and one elected lane executes the MMA, commit and arrive instructions.
    constexpr bool kConv = UNIT_MMA_CONVERGED != 0;
    const bool one = kConv ? elect_one() : true;
    if (kConv || lane == 0) {
      const uint32_t idesc = make_idesc<F16>(p.bn, p.a_signed);
      const uint64_t a_desc0 = make_smem_desc(0u, kSubBytes, 128u);
      const uint64_t a_desc_row = make_smem_desc(0u, 16u, 128u);  // row form: K columns 16 bytes apart
      const uint64_t a_desc_sw = make_smem_desc_sw128(0u);         // dense matrices in the swizzled layout
      // the ordinary loop: column-by-column layout, or fp16 pixel boxes as 32-byte-swizzled rows
      const uint64_t a_desc_std = (AMODE == A_CONV_BOX && (F16 || p.a_sw32 != 0)) ? make_smem_desc_sw32(0u) : a_desc0;
      const uint64_t b_desc0 = make_smem_desc(0u, (uint32_t)p.bn * 16u, 128u);
      const uint32_t a_step = (2u * kSubBytes) >> 4;               // one MMA K-step = two 16-byte columns
      const uint32_t b_step = (2u * (uint32_t)p.bn * 16u) >> 4;
      const uint32_t a_sub_enc = a_sub_bytes >> 4;
      uint32_t s = 0, ring_phase = 0;
      uint32_t lt = 0;  // tiles done by this CTA
      bool alive = true;
      const bool bias_static = p.n_tiles == 1;  // every tile of this CTA has the same bias
      int bias_flag0 = 0, bias_flag1 = 0;        // the sets' "bias goes in through an MMA" flags, once read
      for (int tile = tile0; tile < total_tiles && alive; tile += tstep, ++lt) {
        const uint32_t slot = nslots == 2u ? (lt & 1u) : 0u;
        const uint32_t use = nslots == 2u ? (lt >> 1) : lt;
        // the drain warps arrive on "empty" after every drain of the set: its first use needs no wait
        if (use > 0u && !(kConv ? mbar_wait_warp(smem_u32(&ps->tempty[slot]), (use - 1u) & 1u, wc, kErrWaitTmemEmpty)
                                 : mbar_wait(smem_u32(&ps->tempty[slot]), (use - 1u) & 1u, wc, kErrWaitTmemEmpty))) {
          alive = false;
          break;
        }
        tc_fence_after();
        if (one && my_t == 0u) trace_mark(p, lt, 3);
        const uint32_t d_tmem = tmem_base + (slot * (uint32_t)MT + my_t) * (uint32_t)p.bn;  // this thread's accumulator
        uint32_t started = 0u;
        uint32_t win_off0 = 0u;  // window form: this sub-tile's first position inside the stage's windows
        if constexpr (AMODE == A_CONV_WIN) {
          const uint32_t m_t = fast_div((uint32_t)tile, p.div_n_tiles);
          const uint32_t img = fast_div(m_t, p.div_tpi);
          const uint32_t q0 = (m_t - img * (uint32_t)p.win_tpi) * (uint32_t)(kTileM * MT);
          win_off0 = q0 - fast_div(q0, p.div_wp) * (uint32_t)p.win_wp + my_t * (uint32_t)kTileM;
        }
        const uint64_t a_desc_win = make_smem_desc(0u, (uint32_t)p.win_bytes, 128u);
        for (int ks = ks_begin; ks < ks_end; ++ks) {
          if (!(kConv ? mbar_wait_warp(smem_u32(&ps->full[s]), ring_phase, wc, kErrWaitFull)
                      : mbar_wait(smem_u32(&ps->full[s]), ring_phase, wc, kErrWaitFull))) {
            alive = false;
            break;
          }
          tc_fence_after();
          if (one && ks == 0 && my_t == 0u) trace_mark(p, lt, 4);
          // descriptors differ only in the start-address field (address >> 4, 14 bits)
          const uint32_t stage_enc = (desc_base + s * stage_bytes) >> 4;
          const uint32_t a_enc = stage_enc + my_t * a_sub_enc;  // this thread's sub-tile of the stage
          const uint32_t b_enc = stage_enc + (a_stage_bytes >> 4);
          const int nk = (ks == p.k_stages - 1) ? p.last_ksteps : (p.kc >> 1);
          if constexpr (AMODE == A_CONV_WIN) {
            // K step = one tap of the two chunks of this stage: both columns are the tile's 128 positions
            // shifted by the tap, win_bytes apart (the second chunk's window)
            int kh = 0, kw = 0;
            for (int k = 0; k < nk; ++k) {
              const uint64_t bdesc = b_desc0 | (uint64_t)(b_enc + (uint32_t)k * b_step);
              const uint64_t adesc = a_desc_win | (uint64_t)(stage_enc + win_off0 + (uint32_t)(kh * p.win_wp + kw));
              if (one) tc_mma<F16>(d_tmem, adesc, bdesc, idesc, started);
              started = 1u;
              if (++kw == p.KW) { kw = 0; ++kh; }
            }
          } else if (AMODE == A_DENSE_TMA && p.a_sw128 != 0) {
            // swizzled A: K step k is 32 bytes further inside its 128-byte atom; atoms are 16 KB apart
            for (int k = 0; k < nk; ++k) {
              const uint64_t bdesc = b_desc0 | (uint64_t)(b_enc + (uint32_t)k * b_step);
              const uint64_t adesc = a_desc_sw | (uint64_t)(a_enc + (uint32_t)(k >> 2) * (16384u >> 4) + (uint32_t)(k & 3) * 2u);
              if (one) tc_mma<F16>(d_tmem, adesc, bdesc, idesc, started);
              started = 1u;
            }
          } else if (AMODE == A_CONV_BOX && p.row_kw > 0) {
            // row form: the columns of a kernel row share one row buffer, 16 bytes apart
            uint32_t a_row = a_enc;  // row buffer of the current kernel row (encoded address)
            int pr = 0;              // pair of columns within the row
            for (int k = 0; k < nk; ++k) {
              const uint64_t bdesc = b_desc0 | (uint64_t)(b_enc + (uint32_t)k * b_step);
              const uint64_t adesc = a_desc_row | (uint64_t)(a_row + (uint32_t)pr * 2u);
              if (one) tc_mma<F16>(d_tmem, adesc, bdesc, idesc, started);
              started = 1u;
              if (++pr == (p.row_kw >> 1)) { pr = 0; a_row += ((uint32_t)p.row_kw * kSubBytes) >> 4; }
            }
          } else {
            for (int k = 0; k < nk; ++k) {
              const uint64_t bdesc = b_desc0 | (uint64_t)(b_enc + (uint32_t)k * b_step);
              const uint64_t adesc = a_desc_std | (uint64_t)(a_enc + (uint32_t)k * a_step);
              if (one) tc_mma<F16>(d_tmem, adesc, bdesc, idesc, started);
              started = 1u;
            }
          }
          if (one) tc_commit(smem_u32(&ps->empty[s]));  // frees the stage when these MMAs have read it
          if (++s == (uint32_t)p.stages) { s = 0; ring_phase ^= 1u; }
        }
        if (alive) {
          if constexpr (kCanFold) {
            // The bias step comes last: the drain warps stage the set's bias while the main loop
            // runs (for a CTA's first tiles that is the whole of global-memory latency), and integer
            // sums do not depend on the order of their terms.
            // With one column block the set's bias is staged once, before its first tile, and never
            // rewritten: later tiles reuse it without waiting (the drain warps' later arrivals
            // complete phases nobody looks at).
            int with_bias = slot == 0u ? bias_flag0 : bias_flag1;
            if (!bias_static || use == 0u) {
              if (!(kConv ? mbar_wait_warp(smem_u32(&ps->bready[slot]), use & 1u, wc, kErrWaitBias)
                          : mbar_wait(smem_u32(&ps->bready[slot]), use & 1u, wc, kErrWaitBias))) {
                alive = false;
                break;
              }
              tc_fence_after();
              with_bias = *reinterpret_cast<volatile int *>(&ps->bias_mma[slot]);
              if (slot == 0u) bias_flag0 = with_bias; else bias_flag1 = with_bias;
            }
            // (split-K: the bias enters the first CTA's partial sum only)
            if (with_bias != 0 && (!SPLITK || crank == 0u)) {
              const uint64_t adesc = a_desc0 | (uint64_t)((fold_base + 2u * kFoldBBytes) >> 4);
              const uint64_t bdesc = b_desc0 | (uint64_t)((fold_base + slot * kFoldBBytes) >> 4);
              if (one) tc_mma<F16>(d_tmem, adesc, bdesc, idesc, started);
            }
          }
          // "accumulators ready" completes with every issuer's commit plus one plain arrival (a
          // release that passes the drain warps' bias integers on to whichever warp reads them)
          if (one && my_t == 0u) mbar_arrive(smem_u32(&ps->tfull[slot]));
          if (one) tc_commit(smem_u32(&ps->tfull[slot]));
        }
        if (one && my_t == 0u) trace_mark(p, lt, 5);
      }
    }
  } else if (warp < kDrainWarps) {
    // ===================== drain (warps 0-15) =====================
    // With two accumulator sets the warps split into two groups of eight, one per set: group 0
    // drains the CTA's even tiles, group 1 the odd ones, each at its own pace, so that one
    // group's stores overlap the other's per-tile bookkeeping and waiting.  With one set all
    // sixteen warps drain every tile.
    constexpr bool kCanFold = !F16 && EPI != EPI_RAW_ROWS;
    uint8_t *fold_mem = smem + (size_t)p.stages * stage_bytes;
    const int gw = kDrainWarps / (int)nslots;      // warps per group
    const uint32_t slot = (uint32_t)(warp / gw);   // the group's accumulator set
    const int wl = warp % gw;                      // warp within the group
    const int ohw = p.OH * p.OW;
    const int quad = warp & 3;   // TMEM lane quadrant this warp may read
    const int part = wl >> 2;    // which sub-tile / share of the column groups
    const int groups = p.bn >> 4;
    const int nparts = (gw >> 2) / MT;  // warps that share one sub-tile's column groups
    const int sub = part / nparts;
    const int cpart = part - sub * nparts;
    const int per = (groups + nparts - 1) / nparts;
    const int g_begin = min(cpart * per, groups);
    const int g_end = min(g_begin + per, groups);
    const uint32_t r = (uint32_t)(quad * 32 + lane);  // this thread's row of the sub-tile
    // box mode: where the row sits inside its box (the same for every tile)
    uint32_t dn = 0, dh = 0, dw = 0;
    if constexpr (AMODE == A_CONV_BOX) {
      dn = fast_div(r, p.div_box_hw);
      const uint32_t rr = r - dn * (uint32_t)(p.box_h * p.box_w);
      dh = fast_div(rr, p.div_box_w);
      dw = rr - dh * (uint32_t)p.box_w;
    }
    const long long gstride = (EPI == EPI_RAW_ROWS) ? 16 : p.out_grp_stride * 16;  // between 16-column groups
    const int tile_step = (int)nslots * tstep;  // from one tile of this group to its next
    // The set's bias: the column block it is prepared for, the verdict, and which of the two
    // integer buffers holds the values (it flips at every preparation, so that a warp preparing
    // the next tile never overwrites what a slower warp still reads for this one).
    int staged_n = -1;
    bool folded = true, wide = false;
    uint32_t ver = 0;
    const int first_tile = tile0 + (int)slot * tstep;
    // before the set's first use: stage its bias (the MMA warp runs the main loop meanwhile)
    if constexpr (kCanFold) {
      if (first_tile < total_tiles) {
        staged_n = first_tile - (int)fast_div((uint32_t)first_tile, p.div_n_tiles) * p.n_tiles;
        stage_bias<EPI>(p, ps, fold_mem, slot, ver, staged_n, wl, gw, lane, folded, wide);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ps->bready[slot]));
    }
    uint32_t use = 0;  // how many tiles this group has drained
    for (int tile = first_tile; tile < total_tiles; tile += tile_step, ++use) {
      const uint32_t lt = use * nslots + slot;  // the CTA's tile counter, for the trace
      const int m_tile = (int)fast_div((uint32_t)tile, p.div_n_tiles);
      const int n_tile = tile - m_tile * p.n_tiles;
      // this row's first stored element (needs nothing of the accumulator, so it comes before the wait)
      const long long m = (long long)m_tile * (kTileM * MT) + sub * kTileM + r;
      bool mvalid = m < p.m_total;
      long long obase = 0;
      if constexpr (AMODE == A_CONV_BOX) {
        // sub-tile -> (image block, row block, column block)
        const long long st = (long long)m_tile * MT + sub;
        const uint32_t stc = st < p.sub_tiles ? (uint32_t)st : 0u;
        const uint32_t q = fast_div(stc, p.div_blocks_w);
        const uint32_t wb = stc - q * (uint32_t)p.blocks_w;
        const uint32_t nb = fast_div(q, p.div_blocks_h);
        const uint32_t hb = q - nb * (uint32_t)p.blocks_h;
        const int n_i = (int)nb * p.box_n + (int)dn, oh = (int)hb * p.box_h + (int)dh, ow = (int)wb * p.box_w + (int)dw;
        mvalid = st < p.sub_tiles && (int)dn < p.box_n && n_i < p.n_img && oh < p.OH && ow < p.OW;
        obase = ((long long)n_i * p.out_img_stride + (long long)n_tile * (p.bn >> 4) * p.out_grp_stride + (long long)oh * p.OW + ow) * 16;
      } else if constexpr (AMODE == A_CONV_WIN) {
        // row -> position of the padded image -> (oh, ow); the last KW - 1 positions of a row are no outputs
        const uint32_t img = fast_div((uint32_t)m_tile, p.div_tpi);
        const uint32_t q = ((uint32_t)m_tile - img * (uint32_t)p.win_tpi) * (uint32_t)(kTileM * MT) + (uint32_t)sub * kTileM + r;
        const uint32_t oh = fast_div(q, p.div_wp);
        const uint32_t ow = q - oh * (uint32_t)p.win_wp;
        mvalid = (int)ow < p.OW && (int)oh < p.OH && (int)img < p.n_img;
        obase = ((long long)img * p.out_img_stride + (long long)n_tile * (p.bn >> 4) * p.out_grp_stride + (long long)oh * p.OW + ow) * 16;
      } else if constexpr (EPI == EPI_RAW_ROWS) {
        obase = m * p.ldc + (long long)n_tile * p.bn;
      } else {
        const unsigned mm = mvalid ? (unsigned)m : 0u;
        const long long n_img = (long long)(mm / (unsigned)ohw);
        const long long rem = (long long)mm - n_img * ohw;
        // [n][oc/16][ohw][16] (or [oc/16][od][ohw][16]): column group g of this tile adds g * out_grp_stride * 16
        obase = (n_img * p.out_img_stride + (long long)n_tile * (p.bn >> 4) * p.out_grp_stride + rem) * 16;
      }
      const int32_t *tile_bias = &ps->bias[slot][ver][0];
      const int g_stop = min(g_end, (p.n_total - n_tile * p.bn + 15) >> 4);  // groups that hold real columns
      if constexpr (EPI == EPI_RES_NCHWC) {
        // the residual values this thread will add: asked into L2 now, while the tile's MMAs still run
        // (one lane per 128-byte line; read straight from HBM inside the loop they cost a group its whole latency)
        if (mvalid && (lane & 7) == 0)
          for (int g = g_begin; g < g_stop; ++g)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.residual + obase + (long long)g * gstride));
      }
      if (!mbar_wait_warp(smem_u32(&ps->tfull[slot]), use & 1u, wc, kErrWaitTmemFull)) break;
      tc_fence_after();
      if (wl == 0 && lane == 0) trace_mark(p, lt, 6);
      const uint32_t t_row =
          tmem_base + ((uint32_t)(quad * 32) << 16) + (slot * (uint32_t)MT + (uint32_t)sub) * (uint32_t)p.bn;
      if constexpr (SPLITK) {
        // ---- split-K: reduce-scatter of the cluster's partial accumulators through distributed
        // shared memory.  Column group g (16 columns) belongs to CTA g % S: every CTA sends the
        // groups it does not own to their owners (into the owner's operand ring, which is idle once
        // the owner's MMAs have completed), then adds what it received to its own partial sums,
        // which never leave tensor memory, and runs the epilogue on the groups it owns.
        const uint32_t S = (uint32_t)p.ksplit;
        const uint32_t n_own = ((uint32_t)groups + S - 1u) / S;     // groups a CTA owns at most
        // this CTA's MMAs are complete: its ring may be overwritten.  It announces how many bytes it
        // is going to receive: 8 KB from each peer for each group it owns.
        if (warp == 0 && (uint32_t)lane < S && (uint32_t)lane != crank)
          mbar_arrive_remote(map_to_cta(smem_u32(&ps->xfree[crank]), (uint32_t)lane));
        if (warp == 0 && lane == 0) {
          const uint32_t real_groups = (uint32_t)min(groups, (p.n_total - n_tile * p.bn + 15) >> 4);
          const uint32_t owned = real_groups > crank ? (real_groups - crank + S - 1u) / S : 0u;
          mbar_arrive_expect_tx(smem_u32(&ps->xfull), (S - 1u) * owned * (uint32_t)(kTileM * 64));
        }
        uint32_t peer_ready = 0u;  // bit r: CTA r's ring is known to be free
        bool xok = true;
        for (int g = g_begin; g < g_stop && xok; ++g) {
          const uint32_t owner = (uint32_t)g % S;
          if (owner == crank) continue;
          uint32_t v[16];
          tmem_ld16(t_row + (uint32_t)g * 16u, v);
          tmem_ld_wait();
          if (!(peer_ready >> owner & 1u)) {
            xok = mbar_wait_warp(smem_u32(&ps->xfree[owner]), 0u, wc, kErrWaitPeer, true);
            peer_ready |= 1u << owner;
            if (!xok) break;
          }
          // slot of this CTA among the owner's S - 1 senders.  A (sender, group) block is stored as
          // four planes of 128 rows x 16 bytes, so that one warp instruction writes 512 contiguous
          // bytes of the owner's shared memory (rows 64 bytes apart were ten times slower)
          const uint32_t sender = crank - (crank > owner ? 1u : 0u);
          const uint32_t local = smem_base + (sender * n_own + (uint32_t)g / S) * (uint32_t)(kTileM * 64) + r * 16u;
          const uint32_t remote = map_to_cta(local, owner);
          const uint32_t remote_bar = map_to_cta(smem_u32(&ps->xfull), owner);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            st_async_v4(remote + (uint32_t)(q * kTileM * 16), v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3], remote_bar);
        }
        if (xok && S > 1u) xok = mbar_wait_warp(smem_u32(&ps->xfull), 0u, wc, kErrWaitPeer, true);
        if (xok) {
          for (int g = g_begin; g < g_stop; ++g) {
            if ((uint32_t)g % S != crank) continue;
            uint32_t v[16];
            tmem_ld16(t_row + (uint32_t)g * 16u, v);
            tmem_ld_wait();
            for (uint32_t sdr = 0; sdr + 1u < S; ++sdr) {
              const uint4 *src = reinterpret_cast<const uint4 *>(smem + (size_t)(sdr * n_own + (uint32_t)g / S) * (kTileM * 64) + r * 16u);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 t = src[q * kTileM];
                if constexpr (F16) {
                  v[4 * q] = __float_as_uint(__uint_as_float(v[4 * q]) + __uint_as_float(t.x));
                  v[4 * q + 1] = __float_as_uint(__uint_as_float(v[4 * q + 1]) + __uint_as_float(t.y));
                  v[4 * q + 2] = __float_as_uint(__uint_as_float(v[4 * q + 2]) + __uint_as_float(t.z));
                  v[4 * q + 3] = __float_as_uint(__uint_as_float(v[4 * q + 3]) + __uint_as_float(t.w));
                } else {
                  v[4 * q] += t.x; v[4 * q + 1] += t.y; v[4 * q + 2] += t.z; v[4 * q + 3] += t.w;
                }
              }
            }
            if (mvalid) store_group16<EPI>(p, tile_bias + g * 16, folded, wide, v, obase + g * gstride);
          }
        }
      } else {
      // software pipeline: the read of group g + 1 is in flight while group g is processed
      uint32_t va[16], vb[16];
      // The common cases as a loop of their own, with no per-group decisions and one offset that
      // advances: the accumulator is final (bias inside it, or none) and, when requantising, the
      // shift is 8.  (Measured on the 1x1 64->256 layer at batch 256: 35 -> 19 instructions per
      // group, 72 -> 52 us; the drain warps' instruction count is what bounds the write-heavy layers.)
      bool drained = false;
      // 32-bit outputs of the kernels that keep no bias in shared memory (fp16, dense): regrouped stores
      constexpr bool kRegroup = !kCanFold && (EPI == EPI_RAW_ROWS || EPI == EPI_RAW_NCHWC);
      long long o_k[4] = {0, 0, 0, 0};
      bool ok_k[4] = {false, false, false, false};
      uint32_t xs = 0u;
      if constexpr (kRegroup) {
        // the warp's scratch block: the (unused) bias-digit region, and for the last four warps the
        // (equally unused) bias integers of the pipeline state
        xs = warp < 12 ? smem_u32(fold_mem) + (uint32_t)warp * 1024u
                       : smem_u32(&ps->bias[0][0][0]) + (uint32_t)(warp - 12) * 1024u;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int src = (k >> 1) * 16 + (k & 1) * 8 + (lane >> 2);
          o_k[k] = __shfl_sync(0xffffffffu, obase, src) + 4 * (lane & 3);
          ok_k[k] = __shfl_sync(0xffffffffu, mvalid ? 1 : 0, src) != 0;
        }
      }
      if ((EPI == EPI_RAW_ROWS || folded) && (!epi_requantises(EPI) || p.shift == 8)) {
        long long o = obase + (long long)g_begin * gstride;
        uint32_t taddr = t_row + (uint32_t)g_begin * 16u;
        int left = g_stop - g_begin;
        // (residual epilogue: the residual values of a group are read one group ahead, like its accumulators)
        uint4 ra = make_uint4(0u, 0u, 0u, 0u), rb = ra;
        if (left > 0) {
          tmem_ld16(taddr, va);
          if constexpr (EPI == EPI_RES_NCHWC) {
            if (mvalid) ra = *reinterpret_cast<const uint4 *>(p.residual + o);
          }
          tmem_ld_wait();
        }
        while (left > 0) {
          if (left > 1) {
            tmem_ld16(taddr + 16u, vb);
            if constexpr (EPI == EPI_RES_NCHWC) {
              if (mvalid) rb = *reinterpret_cast<const uint4 *>(p.residual + o + gstride);
            }
          }
          if constexpr (EPI == EPI_REQ_NCHWC) {
            const uint4 w = pack16_shift8(va);
            if (mvalid) *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.out) + o) = w;
          } else if constexpr (EPI == EPI_RES_NCHWC) {
            if (mvalid) *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.out) + o) = pack16_shift8_res(va, ra);
          } else if constexpr (kRegroup) {
            store_group16_regrouped(reinterpret_cast<uint32_t *>(p.out), xs, lane, va, o_k, ok_k, o - obase);
          } else {
            if (mvalid) finish_group16<EPI>(p, va, o);
          }
          tmem_ld_wait();
          if (left > 2) {
            tmem_ld16(taddr + 32u, va);
            if constexpr (EPI == EPI_RES_NCHWC) {
              if (mvalid) ra = *reinterpret_cast<const uint4 *>(p.residual + o + 2 * gstride);
            }
          }
          if (left > 1) {
            if constexpr (EPI == EPI_REQ_NCHWC) {
              const uint4 w = pack16_shift8(vb);
              if (mvalid) *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.out) + o + gstride) = w;
            } else if constexpr (EPI == EPI_RES_NCHWC) {
              if (mvalid) *reinterpret_cast<uint4 *>(reinterpret_cast<uint8_t *>(p.out) + o + gstride) = pack16_shift8_res(vb, rb);
            } else if constexpr (kRegroup) {
              store_group16_regrouped(reinterpret_cast<uint32_t *>(p.out), xs, lane, vb, o_k, ok_k, o - obase + gstride);
            } else {
              if (mvalid) finish_group16<EPI>(p, vb, o + gstride);
            }
          }
          tmem_ld_wait();
          taddr += 32u;
          o += 2 * gstride;
          left -= 2;
        }
        drained = true;
      }
      if (!drained) {
      if (g_begin < g_stop) {
        tmem_ld16(t_row + (uint32_t)g_begin * 16u, va);
        tmem_ld_wait();
      }
      for (int g = g_begin; g < g_stop; g += 2) {
        const bool has_b = g + 1 < g_stop;
        if (has_b) tmem_ld16(t_row + (uint32_t)(g + 1) * 16u, vb);
        if (mvalid) store_group16<EPI>(p, tile_bias + g * 16, folded, wide, va, obase + g * gstride);
        tmem_ld_wait();
        if (g + 2 < g_stop) tmem_ld16(t_row + (uint32_t)(g + 2) * 16u, va);
        if (has_b && mvalid) store_group16<EPI>(p, tile_bias + (g + 1) * 16, folded, wide, vb, obase + (g + 1) * gstride);
        tmem_ld_wait();
      }
      }
      }
      // the accumulator set is free again: the MMA warp may start the set's next main loop
      tc_fence_before();
      __syncwarp();
      if (wl == 0 && lane == 0) trace_mark(p, lt, 7);
      if (lane == 0) mbar_arrive(smem_u32(&ps->tempty[slot]));
      // stage the bias of the group's next tile, unless that tile has the same column block
      if constexpr (kCanFold) {
        const int next = tile + tile_step;
        if (next < total_tiles) {
          const int nt = next - (int)fast_div((uint32_t)next, p.div_n_tiles) * p.n_tiles;
          if (nt != staged_n) {
            ver ^= 1u;
            stage_bias<EPI>(p, ps, fold_mem, slot, ver, nt, wl, gw, lane, folded, wide);
            staged_n = nt;
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&ps->bready[slot]));
      }
    }
  }

  // ===================== teardown =====================
  if (*abort_flag) {
    // let copies this CTA issued land before its shared memory is released
    cp_async_wait<0>();
    for (int i = 0; i < 50; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
  // split-K: no CTA leaves while a peer may still write into its shared memory or arrive on its barriers
  if constexpr (SPLITK) cluster_sync_all();
  trace_mark_ns(p, 11);
}

}  // namespace unit
