// C ABI of unit_b200: argument checking, tile selection, weight packing and
// layout kernels, and the launches of the implicit-GEMM kernel.
#include "../../include/unit_b200.h"

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "igemm_sm100.cuh"
#include "tensor_peak.cuh"

namespace unit {

__device__ unsigned int g_error_word = 0;

// Scratch for unit_conv2d_u8s8_requant_nchwc_noalloc: lives in the library image, so every
// GPU that loads the library holds these bytes until the process exits.
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static std::atomic<uint64_t> g_launches{0};
static std::atomic<unsigned long long *> g_trace{nullptr};
static std::atomic<int> g_trace_cap{0};

// ---------------------------------------------------------------------------
// tile selection (a pure function of the problem, shared by pack and launch)
// ---------------------------------------------------------------------------
struct TileCfg {
  int bn = 0, kc = 0, cols = 0, cols_pad = 0, k_stages = 0, last_ksteps = 0, n_tiles = 0;
  size_t b_stage_bytes = 0;
  size_t a_stage_bytes = 0;  // window form: bytes of a stage's A part (0: kc columns x 128 rows per sub-tile)
};

constexpr size_t kSmemBudget = 200 * 1024;

static int round_up(int x, int m) { return (x + m - 1) / m * m; }

// Tile-shape and path overrides exist only in experiment builds (-DUNIT_B200_TUNING): the shipped
// library reads no environment variable, so a packed weight buffer depends on nothing but the
// arguments of its pack call.
static int tuning_int(const char *name, int dflt) {
#ifdef UNIT_B200_TUNING
  const char *e = getenv(name);
  return e ? atoi(e) : dflt;
#else
  (void)name;
  return dflt;
#endif
}

// Depends on the weight tensor only (never on the batch), so packed weights stay valid
// for every input size.  kc is chosen so that four stages of the larger (two sub-tile)
// CTA tile fit in shared memory.
static TileCfg make_cfg(int n_total, int cols, bool cheap_a = false, bool dense = false, int table_bn = 0, int table_kc = 0) {
  TileCfg c;
  c.cols = cols;
  c.cols_pad = round_up(cols, 2);
  // Widest column block.  256 columns x two sub-tiles fill TMEM with one accumulator set, so
  // each tile's drain (about 2.7 k cycles) is exposed; that is paid back by the halved weight
  // traffic only when the reduction is long.  Measured at batch 256: reductions of 128..1024
  // bytes (8..64 columns) run 8-13 % faster with 128-wide blocks (two sets, drain overlapped),
  // longer ones 15-50 % slower.
  static const int forced_bn = [] {
    const int v = tuning_int("UNIT_B200_BN", 0);
    return (v >= 16 && v <= 256 && v % 16 == 0) ? v : 0;
  }();
  // (cheap_a = false: the A operand comes through the slower im2col copies, where fetching it
  // once more per extra column block costs more than the overlap gains: stride-2 layers lost 35-45 %)
  const int bn_max = table_bn ? table_bn
                     : forced_bn ? forced_bn
                                 : ((cheap_a && n_total >= 256 && c.cols_pad >= 8 && c.cols_pad <= 64) ? 128 : 256);
  c.n_tiles = (n_total + bn_max - 1) / bn_max;
  c.bn = round_up((n_total + c.n_tiles - 1) / c.n_tiles, 16);
  const int kc_max = (int)(kSmemBudget / 4 / (16 * (2 * kTileM + c.bn)));
  static const int cand[] = {8, 6, 4, 12, 10, 14, 16};
  static const int forced_kc = [] {
    const int v = tuning_int("UNIT_B200_KC", 0);
    return (v >= 2 && v <= 16 && v % 2 == 0) ? v : 0;
  }();
  c.kc = 0;
  const int kc_max2 = (int)(kSmemBudget / 2 / (16 * (2 * kTileM + c.bn)));  // two stages still fit
  if (table_kc && table_kc <= kc_max2 && table_kc % 2 == 0) c.kc = table_kc;
  if (c.kc == 0 && forced_kc && forced_kc <= kc_max2 && c.cols_pad % forced_kc == 0) c.kc = forced_kc;
  // plain matrices: stages of 8 columns = 128 bytes of K per row, the width of a swizzled operand
  // row, which lets the A tile arrive as full cache lines (three stages still fit)
  if (c.kc == 0 && dense && c.cols_pad % 8 == 0 && 8 <= (int)(kSmemBudget / 3 / (16 * (2 * kTileM + c.bn)))) c.kc = 8;
  // Narrow column blocks with a reduction of at most 16 columns (the folded stem): the whole
  // reduction in one stage.  Such tiles are bound by the per-stage work of the MMA-issuing
  // threads (wait, commit), not by bytes in flight (measured: stem 182 -> 156 us; wider blocks lose).
  if (c.kc == 0 && c.bn <= 64 && c.cols_pad > 8 && c.cols_pad <= 16 && c.cols_pad <= kc_max2) c.kc = c.cols_pad;
  for (int kc : cand)
    if (c.kc == 0 && kc <= kc_max && c.cols_pad % kc == 0) { c.kc = kc; break; }
  if (c.kc == 0) c.kc = kc_max >= 8 ? 8 : (kc_max & ~1);  // last stage is partial
  if (c.cols_pad < c.kc) c.kc = c.cols_pad;
  c.k_stages = (c.cols_pad + c.kc - 1) / c.kc;
  const int last_cols = c.cols_pad - (c.k_stages - 1) * c.kc;
  c.last_ksteps = last_cols / 2;
  c.b_stage_bytes = (size_t)c.kc * c.bn * 16;
  return c;
}

// Rows per CTA tile: two 128-row sub-tiles share each weight stage when the larger tiles
// still occupy at least half of the SMs and the reduction is long enough for the weight
// traffic to matter (measured: fewer weight bytes per MAC outweighs a partly idle GPU).
// Sub-tiles per CTA tile.  Two (one B stage feeds two accumulators, one MMA-issuing thread each)
// unless the grid would be under-filled, or the reduction is so short that a second accumulator
// set in TMEM is worth more (wide blocks only: with MT x BN <= 256 both sets fit anyway).  When
// the A operand is the bottleneck (im2col copies: slow_a) a single sub-tile costs nothing extra,
// so it is taken when it fills the last round of tiles markedly better.  Measured at batch 256.
// The fp16 kernels follow the same rule: their 32-bit drains are long, and with single sub-tiles a
// second accumulator set hides them (3x3 256->256 at 14x14, batch 256: 196 tiles of two sub-tiles
// need two rounds on 148 SMs, 392 single ones three half-sized rounds: 763 -> 857 TFLOP/s).
static int choose_mt(const TileCfg &c, long long m_total, int sms, bool slow_a) {
  static const int forced = tuning_int("UNIT_B200_MT", 0);
  if (forced == 1 || forced == 2) return forced;
  const long long tiles2 = (m_total + 2 * kTileM - 1) / (2 * kTileM) * c.n_tiles;
  const long long tiles1 = (m_total + kTileM - 1) / kTileM * c.n_tiles;
  if (2 * tiles2 < sms) return 1;
  if (c.cols_pad < 16 && c.bn > 128) return 1;
  if (slow_a) {
    const double eff2 = (double)tiles2 / (double)((tiles2 + sms - 1) / sms * sms);
    const double eff1 = (double)tiles1 / (double)((tiles1 + sms - 1) / sms * sms);
    if (eff1 > 1.25 * eff2) return 1;
  }
  return 2;
}

static int stages_for(const TileCfg &c, int mt, size_t *smem_bytes) {
  const size_t stage = c.a_stage_bytes ? c.a_stage_bytes + c.b_stage_bytes : (size_t)c.kc * 16 * ((size_t)mt * kTileM + c.bn);
  int s = (int)(kSmemBudget / stage);
  if (s > kMaxStages) s = kMaxStages;
  if (s < 2) s = 2;
  *smem_bytes = (size_t)s * stage + kFoldBytes + sizeof(PipeShared) + 128;
  return s;
}

// ---------------------------------------------------------------------------
// tile table: per-shape overrides of the tile heuristics (unit_tile_table_set)
// ---------------------------------------------------------------------------
constexpr int kMaxTileEntries = 1024;
static unit_tile_entry g_tile_table[kMaxTileEntries];
static int g_tile_entries = 0;
static std::mutex g_tile_mu;

// The entry for this convolution: weight-side fields must match; an entry with n = 0 applies to
// every input size, one with n > 0 only to that (n, h, w).  Exact-size entries win.
static bool tile_lookup(const unit_conv_desc *d, unit_tile_entry *out) {
  std::lock_guard<std::mutex> lock(g_tile_mu);
  const unit_tile_entry *any = nullptr;
  for (int i = 0; i < g_tile_entries; ++i) {
    const unit_tile_entry &e = g_tile_table[i];
    if (e.c_in != d->c_in || e.c_block != d->c_block || e.c_out != d->c_out || e.kh != d->kh || e.kw != d->kw ||
        e.stride_h != d->stride_h || e.stride_w != d->stride_w)
      continue;
    if (e.n == d->n && e.h == d->h && e.w == d->w) { *out = e; return true; }
    if (e.n == 0 && any == nullptr) any = &e;
  }
  if (any) { *out = *any; return true; }
  return false;
}

static int conv_cols_i8(const unit_conv_desc *d) {
  if (d->c_block == 16) return d->kh * d->kw * (d->c_in / 16);
  return (d->c_in / 4) * d->kh * ((d->kw + 3) / 4);
}
// stride-1 NCHW16c int8 convolutions fetch A with whole-row box copies
static bool conv_a_is_cheap(const unit_conv_desc *d) { return d->c_block == 16 && d->stride_h == 1 && d->stride_w == 1; }

static int conv_cols_f16(const unit_conv_desc *d) { return d->kh * d->kw * (d->c_in / 16) * 2; }

static bool conv_a_is_cheap(const unit_conv_desc *d);
// Tile shape of an int8 convolution's weights.  Only the weight-side fields of a table entry (bn, kc)
// enter here, and only from entries that apply to every input size, so that packed weights stay valid
// for any batch.
static TileCfg conv_cfg_i8(const unit_conv_desc *d) {
  unit_tile_entry e;
  unit_conv_desc any = *d;
  any.n = 0; any.h = 0; any.w = 0;
  if (d->c_block == 16 && tile_lookup(&any, &e) && e.n == 0 && e.bn >= 16 && e.bn <= 256 && e.bn % 16 == 0)
    return make_cfg(d->c_out, conv_cols_i8(d), conv_a_is_cheap(d), false, e.bn, e.kc);
  return make_cfg(d->c_out, conv_cols_i8(d), conv_a_is_cheap(d));
}

// ---- window form (A_CONV_WIN) ----
// Weight-side eligibility: u8 NCHW16c, stride 1, kernels of 2 to 9 taps, an even number of channel chunks.
static bool win_weights_ok(const unit_conv_desc *d) {
  static const int enabled = tuning_int("UNIT_B200_WIN", 1);
  const int taps = d->kh * d->kw;
  return enabled && d->c_block == 16 && d->stride_h == 1 && d->stride_w == 1 && taps >= 2 && taps <= 9 && (d->c_in / 16) % 2 == 0;
}
// Tile shape of the window-form copy of the weights: same column blocks as the generic form, one
// stage per pair of chunks with 2 x taps columns.
static TileCfg win_cfg(const unit_conv_desc *d) {
  TileCfg c = conv_cfg_i8(d);
  const int taps = d->kh * d->kw;
  c.kc = 2 * taps;
  c.cols_pad = c.cols;
  c.k_stages = (d->c_in / 16) / 2;
  c.last_ksteps = taps;
  c.b_stage_bytes = (size_t)c.kc * c.bn * 16;
  return c;
}
// ---- pair form: stride 2 on u8 NCHW16c ----
// With horizontal stride 2, tap kw of output column ow reads input column 2 ow + kw - pad = 2 (ow + q) + r:
// pixel r (0 or 1) of the input row's pixel PAIR ow + q.  Consecutive outputs read consecutive pairs, so the
// A operand can be fetched as dense rows of 32-byte pairs (whole cache sectors; the im2col copies fetch every
// other 16-byte pixel as its own request) and one K step = one pair = 32 bytes: both pixels' 16 channels of a
// chunk, against weights that hold tap (kh, 2 q + r + pad) in half r, or zeros where that is no tap.  A kernel
// row then takes G K steps per chunk (G = number of distinct q: 2 for a 3 x 3 kernel with pad 1, instead of 3
// taps).  Vertical stride 2 is the box copy's traversal stride.
struct PairGeom {
  bool ok = false;
  int G = 0, qmin = 0, cols = 0;
};
static int floor_div2(int v) { return v >= 0 ? v / 2 : -((-v + 1) / 2); }
static PairGeom pair_geom(const unit_conv_desc *d) {
  static const int enabled = tuning_int("UNIT_B200_PAIR", 1);
  PairGeom g;
  // (weight-side conditions only: the packed copy must not depend on the input size, which the pack call does not
  // know; the convolution call uses the copy when the width is even)
  if (!enabled || d->c_block != 16 || d->stride_h != 2 || d->stride_w != 2 || d->kw < 2) return g;
  g.qmin = floor_div2(0 - d->pad_w);
  g.G = floor_div2(d->kw - 1 - d->pad_w) - g.qmin + 1;
  g.cols = d->kh * g.G * (d->c_in / 16) * 2;
  // at least two thirds of the half-columns must carry a tap (3 x 3: 9 of 12)
  g.ok = 3 * d->kw >= 2 * 2 * g.G;
  return g;
}
// Tile shape of the pair-form copy of the weights.
static TileCfg pair_cfg(const unit_conv_desc *d, const PairGeom &g) {
  unit_tile_entry e;
  unit_conv_desc any = *d;
  any.n = 0; any.h = 0; any.w = 0;
  const bool hit = tile_lookup(&any, &e) && e.n == 0 && e.bn >= 16 && e.bn <= 256 && e.bn % 16 == 0;
  return make_cfg(d->c_out, g.cols, true, false, hit ? e.bn : 0, hit ? e.kc : 0);
}

struct WinGeom {
  bool ok = false;
  int mt = 0, wp = 0, rows = 0, bytes = 0, box_bytes = 0, tpi = 0;
};
// Input-side geometry for `mt` sub-tiles per tile; ok only if enough of the computed positions are outputs
// (the padded columns and the ragged last tile of every image are not) and the stage ring holds two stages.
static WinGeom win_geom(const unit_conv_desc *d, int mt, const TileCfg &wc) {
  WinGeom g;
  if (!win_weights_ok(d)) return g;
  const int oh = d->h + 2 * d->pad_h - d->kh + 1, ow = d->w + 2 * d->pad_w - d->kw + 1;
  g.mt = mt;
  g.wp = d->w + 2 * d->pad_w;
  const int span = kTileM * mt;
  g.tpi = (oh * g.wp + span - 1) / span;
  g.rows = (g.wp - 1 + span + (d->kh - 1) * g.wp + (d->kw - 1) + g.wp - 1) / g.wp;
  g.box_bytes = g.rows * g.wp * 16;
  g.bytes = round_up(g.box_bytes, 128);  // a tensor copy's destination in shared memory must be 128-byte aligned
  const double eff = (double)oh * ow / ((double)g.tpi * span);
  const size_t stage = 2 * (size_t)g.bytes + wc.b_stage_bytes;
  // a single sub-tile per tile re-reads the weights for every 128 positions: only where they are small
  const bool weights_small = mt == 2 || (size_t)wc.k_stages * wc.b_stage_bytes <= (64u << 10);
  g.ok = g.wp * 2 <= 256 && g.rows <= 256 && eff >= 0.85 && 2 * stage <= kSmemBudget && weights_small;
  return g;
}

static int check_conv(const unit_conv_desc *d, bool f16) {
  if (!d) return UNIT_ERR_NULL;
  if (d->n < 1 || d->c_in < 1 || d->h < 1 || d->w < 1 || d->c_out < 1 || d->kh < 1 || d->kw < 1 ||
      d->stride_h < 1 || d->stride_w < 1 || d->pad_h < 0 || d->pad_w < 0)
    return UNIT_ERR_SHAPE;
  if (d->c_block != 16 && !(d->c_block == 4 && !f16)) return UNIT_ERR_LAYOUT;
  if (d->c_in % d->c_block || d->c_out % 16) return UNIT_ERR_LAYOUT;
  if (d->h + 2 * d->pad_h < d->kh || d->w + 2 * d->pad_w < d->kw) return UNIT_ERR_SHAPE;
  if (d->kh > 64 || d->kw > 64) return UNIT_ERR_SHAPE;
  const long long img = (long long)d->c_in * d->h * d->w * (f16 ? 2 : 1);
  if (img >= (1ll << 31)) return UNIT_ERR_TOO_LARGE;
  const long long oh = (d->h + 2 * d->pad_h - d->kh) / d->stride_h + 1, ow = (d->w + 2 * d->pad_w - d->kw) / d->stride_w + 1;
  if ((long long)d->n * oh * ow >= (1ll << 31) - 512) return UNIT_ERR_TOO_LARGE;  // output pixels index in 32 bits
  return UNIT_OK;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int check_arch() {
  static std::once_flag once;
  static int cached[64];
  static int ndev = 0;
  std::call_once(once, [] {
    if (cudaGetDeviceCount(&ndev) != cudaSuccess) ndev = 0;
    if (ndev > 64) ndev = 64;
    for (int i = 0; i < ndev; ++i) {
      int major = 0, minor = 0;
      cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i);
      cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, i);
      cached[i] = (major == 10 && minor == 0) ? UNIT_OK : UNIT_ERR_ARCH;
    }
  });
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev >= ndev) return UNIT_ERR_ARCH;
  return cached[dev];
}

static int sm_count() {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 148;
}

// ---------------------------------------------------------------------------
// weight packing: reference layouts -> [n_tile][k_stage][kc][bn][16 B] blocks
// ---------------------------------------------------------------------------
enum PackMode : int { PACK_CONV_I8 = 0, PACK_STEM_I8 = 1, PACK_CONV_F16 = 2, PACK_DENSE_I8 = 3, PACK_GEMM_F16 = 4, PACK_STEM_S2D = 5, PACK_CONV_WIN = 6, PACK_CONV_PAIR = 7 };

struct PackParams {
  const uint8_t *src;
  uint4 *dst;
  int mode, n_total, bn, kc, cols, k_stages, n_tiles;
  int Cc, KH, KW, kwg;  // conv
  int tw, sft_h, sft_w;  // PACK_STEM_S2D: taps per row of the 2x2-folded kernel, tap shifts
  int pair_g, pair_qmin, pair_pad;  // PACK_CONV_PAIR: pair offsets per kernel row, the first offset, the horizontal padding
  int K, T;             // dense / gemm (K in elements)
};

__global__ void pack_weights_kernel(const PackParams p) {
  const long long total = (long long)p.n_tiles * p.k_stages * p.kc * p.bn;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(idx % p.bn);
    long long t = idx / p.bn;
    const int jj = (int)(t % p.kc);
    t /= p.kc;
    const int ks = (int)(t % p.k_stages);
    const int n_tile = (int)(t / p.k_stages);
    const int oc = n_tile * p.bn + row;
    const int j = ks * p.kc + jj;
    uint32_t w[4] = {0u, 0u, 0u, 0u};
    if (oc < p.n_total && j < p.cols) {
      if (p.mode == PACK_CONV_I8) {
        const int tap = j / p.Cc, ci = j % p.Cc;
        const int kh = tap / p.KW, kw = tap % p.KW;
        // [oc/16][ci][kh][kw][m][oc%16][r]
        const uint8_t *s = p.src + ((((size_t)(oc >> 4) * p.Cc + ci) * p.KH + kh) * p.KW + kw) * 256 + (oc & 15) * 4;
        for (int m = 0; m < 4; ++m) w[m] = *reinterpret_cast<const uint32_t *>(s + m * 64);
      } else if (p.mode == PACK_CONV_WIN) {
        // window form: stage = pair of channel chunks; within it, columns (tap, chunk 2 ks) and (tap, chunk 2 ks + 1)
        const int tap = jj >> 1, ci = 2 * ks + (jj & 1);
        const int kh = tap / p.KW, kw = tap % p.KW;
        const uint8_t *s = p.src + ((((size_t)(oc >> 4) * p.Cc + ci) * p.KH + kh) * p.KW + kw) * 256 + (oc & 15) * 4;
        for (int m = 0; m < 4; ++m) w[m] = *reinterpret_cast<const uint32_t *>(s + m * 64);
      } else if (p.mode == PACK_CONV_PAIR) {
        // column = (K step, half r); K step = ((kh, pair offset g), chunk): tap kw = 2 (qmin + g) + r + pad or none
        const int r = j & 1, step = j >> 1;
        const int tg = step / p.Cc, ci = step % p.Cc;
        const int kh = tg / p.pair_g, kw = 2 * (p.pair_qmin + tg % p.pair_g) + r + p.pair_pad;
        if (kw >= 0 && kw < p.KW) {
          const uint8_t *s = p.src + ((((size_t)(oc >> 4) * p.Cc + ci) * p.KH + kh) * p.KW + kw) * 256 + (oc & 15) * 4;
          for (int m = 0; m < 4; ++m) w[m] = *reinterpret_cast<const uint32_t *>(s + m * 64);
        }
      } else if (p.mode == PACK_STEM_I8) {
        const int g = j % p.kwg;
        const int t2 = j / p.kwg;
        const int kh = t2 % p.KH, ci = t2 / p.KH;
        for (int q = 0; q < 4; ++q) {
          const int kw = g * 4 + q;
          if (kw < p.KW) {
            // [oc/16][ci][kh][kw][0][oc%16][r]
            const uint8_t *s = p.src + ((((size_t)(oc >> 4) * p.Cc + ci) * p.KH + kh) * p.KW + kw) * 64 + (oc & 15) * 4;
            w[q] = *reinterpret_cast<const uint32_t *>(s);
          }
        }
      } else if (p.mode == PACK_STEM_S2D) {
        // column = tap (ty, tx) of the folded kernel; the 16 bytes are (dy, dx, c) with
        // kh = 2 ty + dy - sft_h, kw = 2 tx + dx - sft_w of the original kernel
        const int ty = j / p.tw, tx = j % p.tw;
        for (int q = 0; q < 4; ++q) {
          const int kh = 2 * ty + (q >> 1) - p.sft_h, kw = 2 * tx + (q & 1) - p.sft_w;
          if (kh >= 0 && kh < p.KH && kw >= 0 && kw < p.KW) {
            const uint8_t *s = p.src + (((size_t)(oc >> 4) * p.KH + kh) * p.KW + kw) * 64 + (oc & 15) * 4;
            w[q] = *reinterpret_cast<const uint32_t *>(s);
          }
        }
      } else if (p.mode == PACK_CONV_F16) {
        const int chunk = j >> 1, half = j & 1;
        const int tap = chunk / p.Cc, ci = chunk % p.Cc;
        const int kh = tap / p.KW, kw = tap % p.KW;
        // [oc/16][ci][kh][kw][i][o]
        const uint16_t *s = reinterpret_cast<const uint16_t *>(p.src) +
                            ((((size_t)(oc >> 4) * p.Cc + ci) * p.KH + kh) * p.KW + kw) * 256 + (oc & 15);
        for (int q = 0; q < 4; ++q) {
          const uint32_t lo = s[(half * 8 + 2 * q) * 16], hi = s[(half * 8 + 2 * q + 1) * 16];
          w[q] = lo | (hi << 16);
        }
      } else if (p.mode == PACK_DENSE_I8) {
        // [n/T][k/4][T][4]
        const uint8_t *s = p.src + ((size_t)(oc / p.T) * (p.K / 4)) * p.T * 4 + (size_t)(oc % p.T) * 4;
        for (int q = 0; q < 4; ++q) w[q] = *reinterpret_cast<const uint32_t *>(s + (size_t)(j * 4 + q) * p.T * 4);
      } else {  // PACK_GEMM_F16: B[k][n]
        const uint16_t *s = reinterpret_cast<const uint16_t *>(p.src);
        for (int q = 0; q < 4; ++q) {
          const uint32_t lo = s[(size_t)(j * 8 + 2 * q) * p.n_total + oc];
          const uint32_t hi = s[(size_t)(j * 8 + 2 * q + 1) * p.n_total + oc];
          w[q] = lo | (hi << 16);
        }
      }
    }
    p.dst[idx] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

static int launch_pack(const PackParams &pp, cudaStream_t st) {
  const long long total = (long long)pp.n_tiles * pp.k_stages * pp.kc * pp.bn;
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  pack_weights_kernel<<<(unsigned)blocks, 256, 0, st>>>(pp);
  g_launches.fetch_add(1);
  return cudaGetLastError() == cudaSuccess ? UNIT_OK : UNIT_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------
// layout kernels (bandwidth work)
// ---------------------------------------------------------------------------
// NCHW <-> [n][c/CB][hw][CB] as a register transpose of 4-byte words.  A thread owns one channel
// block and the P = 4 / EB pixels of one 4-byte word: on the NCHW side it touches one word per
// channel, and consecutive threads touch consecutive words of the same channel row (a warp reads
// or writes 128 contiguous bytes per instruction); on the blocked side its P pixels x CB channels
// are P * CB * EB contiguous bytes, moved as 16-byte vectors.  Needs h * w to be a multiple of P and
// 16-byte aligned tensors; other shapes take the element loops below.
template <int EB, int CB>
__device__ __forceinline__ void transpose_words(const uint32_t (&in)[CB], uint32_t (&out)[CB]) {
  // in[c] = P pixels of channel c;  out = pixel-major: P pixels x CB channels, EB bytes each
  if constexpr (EB == 4) {
#pragma unroll
    for (int c = 0; c < CB; ++c) out[c] = in[c];
  } else if constexpr (EB == 2) {
#pragma unroll
    for (int q = 0; q < CB / 2; ++q) {
      out[q] = __byte_perm(in[2 * q], in[2 * q + 1], 0x5410);           // pixel 0: low halves
      out[CB / 2 + q] = __byte_perm(in[2 * q], in[2 * q + 1], 0x7632);  // pixel 1: high halves
    }
  } else {
#pragma unroll
    for (int px = 0; px < 4; ++px)
#pragma unroll
      for (int q = 0; q < CB / 4; ++q) {
        const uint32_t sel = (uint32_t)((4 + px) << 4 | px);
        const uint32_t lo = __byte_perm(in[4 * q], in[4 * q + 1], sel);
        const uint32_t hi = __byte_perm(in[4 * q + 2], in[4 * q + 3], sel);
        out[px * (CB / 4) + q] = __byte_perm(lo, hi, 0x5410);
      }
  }
}
// the inverse: in = pixel-major words, out[c] = P pixels of channel c
template <int EB, int CB>
__device__ __forceinline__ void untranspose_words(const uint32_t (&in)[CB], uint32_t (&out)[CB]) {
  if constexpr (EB == 4) {
#pragma unroll
    for (int c = 0; c < CB; ++c) out[c] = in[c];
  } else if constexpr (EB == 2) {
#pragma unroll
    for (int q = 0; q < CB / 2; ++q) {
      out[2 * q] = __byte_perm(in[q], in[CB / 2 + q], 0x5410);
      out[2 * q + 1] = __byte_perm(in[q], in[CB / 2 + q], 0x7632);
    }
  } else {
#pragma unroll
    for (int q = 0; q < CB / 4; ++q) {
      // words of pixels 0..3 holding channels 4q .. 4q+3
      const uint32_t p0 = in[q], p1 = in[CB / 4 + q], p2 = in[2 * (CB / 4) + q], p3 = in[3 * (CB / 4) + q];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t sel = (uint32_t)((4 + k) << 4 | k);
        out[4 * q + k] = __byte_perm(__byte_perm(p0, p1, sel), __byte_perm(p2, p3, sel), 0x5410);
      }
    }
  }
}

// With 16-channel blocks a thread's result is 64 bytes (four 16-byte pieces).  Written straight
// from the thread, every store instruction of a warp would touch 32 separate half sectors; the
// pieces go through shared memory instead, so that consecutive lanes store consecutive 16 bytes
// (512 contiguous bytes per warp instruction).  kPackPad staggers the four piece planes by 32 bytes,
// which makes both the writes and the reads of the staging buffer conflict-free.
constexpr int kPackThreads = 256, kPackPad = 2;
template <int EB, int CB>
__global__ void __launch_bounds__(kPackThreads)
    nchw_to_nchwc_vec_kernel(const uint32_t *__restrict__ src, uint32_t *__restrict__ dst, int n, int c, long long hw_words) {
  constexpr int NP = CB / 4;  // 16-byte pieces per thread
  __shared__ uint4 stage[NP > 1 ? NP * (kPackThreads + kPackPad) : 1];
  const int cc = (c + CB - 1) / CB;
  const long long total = (long long)n * cc * hw_words;
  const long long span = (long long)gridDim.x * blockDim.x;
  for (long long base = blockIdx.x * (long long)blockDim.x; base < total; base += span) {
    const long long idx = base + threadIdx.x;
    uint32_t out[CB];
    if (idx < total) {
      const long long wpos = idx % hw_words;
      const long long t = idx / hw_words;
      const int chunk = (int)(t % cc);
      const long long img = t / cc;
      uint32_t in[CB];
#pragma unroll
      for (int k = 0; k < CB; ++k) {
        const int ch = chunk * CB + k;
        in[k] = ch < c ? __ldg(src + (img * c + ch) * hw_words + wpos) : 0u;
      }
      transpose_words<EB, CB>(in, out);
    }
    if constexpr (NP == 1) {
      if (idx < total) reinterpret_cast<uint4 *>(dst)[idx] = make_uint4(out[0], out[1], out[2], out[3]);
    } else {
      if (idx < total) {
#pragma unroll
        for (int q = 0; q < NP; ++q)
          stage[q * (kPackThreads + kPackPad) + threadIdx.x] = make_uint4(out[4 * q], out[4 * q + 1], out[4 * q + 2], out[4 * q + 3]);
      }
      __syncthreads();
      // piece k of the block's output (k = thread * NP + piece) is stored by thread k % 256 in round k / 256
      uint4 *d4 = reinterpret_cast<uint4 *>(dst) + base * NP;
      const long long pieces = (total - base < blockDim.x ? total - base : blockDim.x) * NP;
#pragma unroll
      for (int i = 0; i < NP; ++i) {
        const int k = i * kPackThreads + threadIdx.x;
        if (k < pieces) d4[k] = stage[(k % NP) * (kPackThreads + kPackPad) + k / NP];
      }
      __syncthreads();
    }
  }
}

template <int EB, int CB>
__global__ void nchwc_to_nchw_vec_kernel(const uint32_t *__restrict__ src, uint32_t *__restrict__ dst, int n, int c,
                                         int cb_total, long long hw_words) {
  // cb_total = stored channel blocks of the source; only the first c channels are written
  const long long total = (long long)n * cb_total * hw_words;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long wpos = idx % hw_words;
    const long long t = idx / hw_words;
    const int chunk = (int)(t % cb_total);
    const long long img = t / cb_total;
    if (chunk * CB >= c) continue;
    uint32_t in[CB], out[CB];
    const uint4 *s4 = reinterpret_cast<const uint4 *>(src + idx * CB);
#pragma unroll
    for (int q = 0; q < CB / 4; ++q) {
      const uint4 v = __ldg(s4 + q);
      in[4 * q] = v.x; in[4 * q + 1] = v.y; in[4 * q + 2] = v.z; in[4 * q + 3] = v.w;
    }
    untranspose_words<EB, CB>(in, out);
#pragma unroll
    for (int k = 0; k < CB; ++k) {
      const int ch = chunk * CB + k;
      if (ch < c) dst[(img * c + ch) * hw_words + wpos] = out[k];
    }
  }
}

// element loops: any shape
template <typename T>
__global__ void nchw_to_nchwc_kernel(const T *__restrict__ src, T *__restrict__ dst, int n, int c, int h, int w,
                                     int cb) {
  // one thread = one (pixel, channel block): reads cb strided values, writes cb contiguous
  const int cc = (c + cb - 1) / cb;
  const long long hw = (long long)h * w;
  const long long total = (long long)n * cc * hw;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long pix = idx % hw;
    const long long t = idx / hw;
    const int chunk = (int)(t % cc);
    const long long img = t / cc;
    T *d = dst + idx * cb;
    for (int k = 0; k < cb; ++k) {
      const int ch = chunk * cb + k;
      d[k] = ch < c ? src[(img * c + ch) * hw + pix] : T(0);
    }
  }
}

template <typename T>
__global__ void nchwc_to_nchw_kernel(const T *__restrict__ src, T *__restrict__ dst, int n, int c, int h, int w,
                                     int cb) {
  const int cc = (c + cb - 1) / cb;
  const long long hw = (long long)h * w;
  const long long total = (long long)n * c * hw;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long pix = idx % hw;
    const long long t = idx / hw;
    const int ch = (int)(t % c);
    const long long img = t / c;
    dst[idx] = src[((img * cc + ch / cb) * hw + pix) * cb + ch % cb];
  }
}

__global__ void oihw_to_ref_i8_kernel(const int8_t *__restrict__ src, int8_t *__restrict__ dst, int o, int i, int kh,
                                      int kw, int cb) {
  const int oc = (o + 15) / 16, icc = (i + cb - 1) / cb, c4 = cb / 4;
  const long long total = (long long)oc * icc * kh * kw * c4 * 64;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    long long t = idx;
    const int r = (int)(t % 4); t /= 4;
    const int l = (int)(t % 16); t /= 16;
    const int m = (int)(t % c4); t /= c4;
    const int x = (int)(t % kw); t /= kw;
    const int y = (int)(t % kh); t /= kh;
    const int ic = (int)(t % icc);
    const int ob = (int)(t / icc);
    const int och = ob * 16 + l, ich = ic * cb + m * 4 + r;
    dst[idx] = (och < o && ich < i) ? src[(((size_t)och * i + ich) * kh + y) * kw + x] : (int8_t)0;
  }
}

__global__ void oihw_to_ref_f16_kernel(const uint16_t *__restrict__ src, uint16_t *__restrict__ dst, int o, int i,
                                       int kh, int kw) {
  const int oc = (o + 15) / 16, icc = (i + 15) / 16;
  const long long total = (long long)oc * icc * kh * kw * 256;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    long long t = idx;
    const int ob = (int)(t % 16); t /= 16;
    const int ib = (int)(t % 16); t /= 16;
    const int x = (int)(t % kw); t /= kw;
    const int y = (int)(t % kh); t /= kh;
    const int ic = (int)(t % icc);
    const int occ = (int)(t / icc);
    const int och = occ * 16 + ob, ich = ic * 16 + ib;
    dst[idx] = (och < o && ich < i) ? src[(((size_t)och * i + ich) * kh + y) * kw + x] : (uint16_t)0;
  }
}

static unsigned grid_for(long long total) {
  long long b = (total + 255) / 256;
  if (b > 148 * 32) b = 148 * 32;
  if (b < 1) b = 1;
  return (unsigned)b;
}

// ---------------------------------------------------------------------------
// stride-2 stem on NCHW4c as a stride-1 convolution on 2x2-folded pixels
// ---------------------------------------------------------------------------
// A pixel of the folded image holds the 2 x 2 block (2y + dy, 2x + dx) of 4-channel pixels:
// 16 bytes ordered (dy, dx, c), i.e. an ordinary NCHW16c image of half the height and width.
// With pad_lo = ceil(pad / 2) and sft = 2 pad_lo - pad, tap (ty, tx) of the folded kernel
// covers the original taps kh = 2 ty + dy - sft_h, kw = 2 tx + dx - sft_w (absent taps get
// zero weights), and the convolution becomes stride 1 with low padding pad_lo; the high side
// needs no explicit padding because the tensor copy zero-fills beyond the image.
struct StemFold {
  bool ok = false;
  int h2 = 0, w2 = 0, pad_h = 0, pad_w = 0, sft_h = 0, sft_w = 0, th = 0, tw = 0;
};
static StemFold stem_fold(const unit_conv_desc *d, bool need_even_image) {
  StemFold f;
  if (d->c_block != 4 || d->c_in != 4 || d->stride_h != 2 || d->stride_w != 2) return f;
  if (need_even_image && ((d->h & 1) || (d->w & 1))) return f;
  f.pad_h = (d->pad_h + 1) / 2;
  f.pad_w = (d->pad_w + 1) / 2;
  f.sft_h = 2 * f.pad_h - d->pad_h;
  f.sft_w = 2 * f.pad_w - d->pad_w;
  f.th = (d->kh - 1 + f.sft_h) / 2 + 1;
  f.tw = (d->kw - 1 + f.sft_w) / 2 + 1;
  f.h2 = d->h / 2;
  f.w2 = d->w / 2;
  f.ok = true;
  return f;
}

// [n][1][h][w][4] -> [n][1][h/2][w/2][16]; one thread per folded pixel: two 8-byte reads, one 16-byte write
__global__ void fold2x2_kernel(const uint2 *__restrict__ src, uint4 *__restrict__ dst, int n, int h2, int w2) {
  const long long total = (long long)n * h2 * w2;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int x = (int)(idx % w2);
    const long long t = idx / w2;
    const int y = (int)(t % h2);
    const long long img = t / h2;
    // source row 2y of image img starts at ((img * 2 h2 + 2 y) * 2 w2) pixels = that many / 2 uint2
    const long long row0 = (img * 2 * h2 + 2 * y) * (long long)w2;  // in uint2 units (2 pixels each)
    const uint2 a = src[row0 + x];
    const uint2 b = src[row0 + w2 + x];
    dst[idx] = make_uint4(a.x, a.y, b.x, b.y);
  }
}

// ---------------------------------------------------------------------------
// launches of the contraction kernel
// ---------------------------------------------------------------------------
// Experiment builds: UNIT_B200_ROW=0 keeps one copy per tap for the folded stem.
static bool use_row_form() {
  static const int v = tuning_int("UNIT_B200_ROW", 1);
  return v != 0;
}

// Experiment builds: UNIT_B200_PDL=0 launches the contraction kernels fully serialised.
static bool use_pdl() {
  static const int v = tuning_int("UNIT_B200_PDL", 1);
  return v != 0;
}

// Experiment builds: UNIT_B200_FOLD=0 makes the drain add every bias; the default lets the tensor core do it.
static bool use_fold() {
  static const int v = tuning_int("UNIT_B200_FOLD", 1);
  return v != 0;
}

// ---------------------------------------------------------------------------
// kernel variants: one slot per instantiated igemm_kernel<AMODE, EPI, F16, MT>
// ---------------------------------------------------------------------------
constexpr int kNumAModes = 8, kNumEpis = 5;
constexpr int kMaxVariants = kNumAModes * kNumEpis * 2 * 2 * 2;
struct VariantSlot {
  char name[72];
  bool present;
  std::atomic<uint64_t> launches;
  std::atomic<bool> attr_done[64];  // per device: the kernel's dynamic shared-memory limit is raised
};
static VariantSlot *variant_table() {
  static VariantSlot table[kMaxVariants];  // static storage: zero-initialised
  return table;
}
static bool register_variant(int index, int amode, int epi, bool f16, int mt, bool splitk) {
  static const char *const amodes[kNumAModes] = {"A_CONV_I8", "A_CONV_F16", "A_STEM_I8", "A_DENSE", "A_CONV_TMA", "A_CONV_BOX", "A_DENSE_TMA", "A_CONV_WIN"};
  static const char *const epis[kNumEpis] = {"EPI_RAW_NCHWC", "EPI_REQ_NCHWC", "EPI_RAW_ROWS", "EPI_MUL_NCHWC", "EPI_RES_NCHWC"};
  VariantSlot &v = variant_table()[index];
  snprintf(v.name, sizeof(v.name), "igemm_kernel<%s, %s, %s, MT=%d%s>", amodes[amode], epis[epi], f16 ? "f16" : "i8", mt,
           splitk ? ", split-K" : "");
  v.present = true;
  return true;
}
template <int AMODE, int EPI, bool F16, int MT, bool SPLITK>
struct Variant {
  static constexpr int index = (((AMODE * kNumEpis + EPI) * 2 + (F16 ? 1 : 0)) * 2 + (MT - 1)) * 2 + (SPLITK ? 1 : 0);
  static const bool registered;  // set while the library is loaded, so that never-launched variants are listed too
};
template <int AMODE, int EPI, bool F16, int MT, bool SPLITK>
const bool Variant<AMODE, EPI, F16, MT, SPLITK>::registered =
    register_variant(Variant<AMODE, EPI, F16, MT, SPLITK>::index, AMODE, EPI, F16, MT, SPLITK);

// ---------------------------------------------------------------------------
// launch plans
// ---------------------------------------------------------------------------
// Everything one contraction launch needs, as plain data without pointers into the library's own
// memory except the kernel's entry and the error word: the filled kernel parameters, the tensor
// map, the grid.  Every entry point fills one on its stack and runs it; unit_conv2d_plan_int8
// hands one to the caller (unit_conv_plan), so that repeated calls on the same buffers skip the
// argument checks, the tile selection and the tensor-map encoding.
constexpr uint32_t kPlanMagic = 0x756e6974u;
struct PlanImpl {
  uint32_t magic;
  int32_t variant, device;
  uint32_t grid, smem_bytes;
  uint32_t cluster;                  // > 1: thread-block cluster size (split-K)
  int32_t table_mt, table_ksplit;    // from the tile table: 0 = heuristics (ksplit 1 = do not split)
  int32_t fold_n, fold_h2, fold_w2;  // fold_n > 0: the stem's 2 x 2 fold into scratch runs first
  const void *fold_src;
  void *fold_dst;
  const void *kernel;
  IgemmParams p;
  unsigned char map[sizeof(CUtensorMap)];
};
static_assert(sizeof(PlanImpl) <= sizeof(unit_conv_plan), "unit_conv_plan too small for the launch plan");

static std::atomic<unsigned long long> g_wait_limit_ns{1000000000ull};
static std::atomic<int> g_inject{0};

template <int AMODE, int EPI, bool F16, int MT, bool SPLITK>
static int prepare_mt(PlanImpl &pl, const TileCfg &c, int sms, int ksplit) {
  if (!Variant<AMODE, EPI, F16, MT, SPLITK>::registered) return UNIT_ERR_LAUNCH;
  IgemmParams &p = pl.p;
  pl.variant = Variant<AMODE, EPI, F16, MT, SPLITK>::index;
  pl.kernel = reinterpret_cast<const void *>(igemm_kernel<AMODE, EPI, F16, MT, SPLITK>);
  size_t smem_bytes = 0;
  p.stages = stages_for(c, MT, &smem_bytes);
  pl.smem_bytes = (uint32_t)smem_bytes;
  p.m_tiles = (int)((p.m_total + kTileM * MT - 1) / (kTileM * MT));
  const long long tiles = (long long)p.m_tiles * p.n_tiles;
  if (SPLITK) {
    p.ksplit = ksplit;
    p.ks_per = (c.k_stages + ksplit - 1) / ksplit;
    pl.grid = (unsigned)(tiles * ksplit);
    pl.cluster = (uint32_t)ksplit;
  } else {
    p.ksplit = 1;
    p.ks_per = c.k_stages;
    pl.grid = (unsigned)(tiles < sms ? tiles : sms);
    pl.cluster = 1;
  }
  // tensor memory: a power of two of columns that holds the accumulator sets (the kernel derives the
  // same number of sets from MT and bn; split-K tiles use one set)
  const int sets = (!SPLITK && (512 / (MT * c.bn)) >= 2) ? 2 : 1;
  int cols = 32;
  while (cols < sets * MT * c.bn) cols *= 2;
  p.tmem_cols = cols;
  return UNIT_OK;
}

// How many clusters of `ks` CTAs of the split-K kernel the current device holds at once (cached per
// kernel variant, size and shared-memory request).
template <int AMODE, int EPI, bool F16>
static int max_active_clusters(const TileCfg &c, int ks) {
  static std::mutex mu;
  static int cached[64][9][kMaxStages + 1] = {};
  size_t smem_bytes = 0;
  const int stages = stages_for(c, 1, &smem_bytes);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || ks < 2 || ks > 8) return 0;
  std::lock_guard<std::mutex> lock(mu);
  int &slot = cached[dev][ks][stages];
  if (slot == 0) {
    auto kern = igemm_kernel<AMODE, EPI, F16, 1, true>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
      cudaGetLastError();
      return 0;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)ks * 64);
    cfg.blockDim = dim3(kNumThreads);
    cfg.dynamicSmemBytes = 227 * 1024 - 1024;  // the largest request of any tile shape: a lower bound for smaller ones
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)ks;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
    slot = n > 0 ? n : -1;
  }
  return slot > 0 ? slot : 0;
}

// Split-K factor for grids that would leave most SMs idle: S CTAs (one thread-block cluster)
// share a tile, each accumulating a slice of the reduction, and exchange partial sums through
// distributed shared memory (integer sums do not depend on the order, so the int8 results stay
// bit-exact; the reference splits its reductions too: python/tensorizer/ops/gpu.py:83-87,134,
// poc/tensorcore/gemm-prefetch.cu:29-64).  Returns 1 when the problem should not be split.
static int choose_ksplit(const TileCfg &c, long long m_total, int sms, int table_ksplit = 0) {
  static const int forced_env = tuning_int("UNIT_B200_KSPLIT", -1);
  const int forced = table_ksplit > 0 ? table_ksplit : forced_env;  // a tile-table entry: 1 = never, n = at most n
  if (forced == 0 || forced == 1) return 1;
  const long long tiles = (m_total + kTileM - 1) / kTileM * c.n_tiles;
  if (tiles * 2 > sms || c.k_stages < 4) return 1;
  // The exchange costs about 5 us (two hops between SMs and the transfer).  A CTA streams its operands
  // at roughly 100 GB/s, so splitting pays once a tile's operands exceed some 600 KB (measured at
  // batch 32: reductions of 2048 bytes and more gain 1-6 us per layer, shorter ones lose).
  if ((size_t)c.k_stages * c.kc * 16 * (kTileM + c.bn) < (640u << 10) && forced < 2) return 1;
  int s = (int)(sms / tiles);
  if (s > 8) s = 8;                          // the portable cluster size
  if (s > c.k_stages / 2) s = c.k_stages / 2;  // at least two pipeline stages per CTA
  if (forced >= 2 && forced < s) s = forced;
  if (s < 2) return 1;
  const int per = (c.k_stages + s - 1) / s;
  s = (c.k_stages + per - 1) / per;          // no CTA without stages
  if (s < 2) return 1;
  // the partial sums a CTA receives replace its operand ring: (S - 1) senders x owned groups x 128 rows x 64 bytes
  size_t smem_bytes = 0;
  const int stages = stages_for(c, 1, &smem_bytes);
  const size_t ring = (size_t)stages * c.kc * 16 * (kTileM + c.bn);
  const size_t recv = (size_t)(s - 1) * (((c.bn >> 4) + s - 1) / s) * kTileM * 64;
  return recv <= ring ? s : 1;
}

static FastDiv make_fast_div(uint32_t d);

// Device address of the error word on the current device, looked up once per device (a launch
// then makes no runtime call besides the kernel launch itself, so it can be captured in a graph).
static unsigned int *error_word_address() {
  static std::mutex mu;
  static unsigned int *cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void *ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_error_word) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<unsigned int *>(ptr);
  }
  return cached[dev];
}

// Fills the tile fields of the plan's parameters and picks the sub-tile count.  MAX_MT = 1 for
// operand paths that only small problems reach (no two-sub-tile variant is compiled for them).
template <int AMODE, int EPI, bool F16, int MAX_MT = 2>
static int prepare(PlanImpl &pl, const TileCfg &c, const CUtensorMap *tmap_in = nullptr) {
  IgemmParams &p = pl.p;
  if (tmap_in) memcpy(pl.map, tmap_in, sizeof(CUtensorMap));
  else memset(pl.map, 0, sizeof(pl.map));
  p.bn = c.bn;
  p.kc = c.kc;
  p.cols = c.cols;
  p.k_stages = c.k_stages;
  p.last_ksteps = c.last_ksteps;
  p.n_tiles = c.n_tiles;
  p.div_n_tiles = make_fast_div((uint32_t)c.n_tiles);
  p.err = error_word_address();
  if (p.err == nullptr) return UNIT_ERR_LAUNCH;
  if (cudaGetDevice(&pl.device) != cudaSuccess) return UNIT_ERR_LAUNCH;
  if (p.a_signed == 0) p.fold_bias = use_fold() ? 1 : 0;  // (the bias step's constant block is u8)
  const int sms = sm_count();
  pl.magic = kPlanMagic;
  if constexpr (MAX_MT >= 2) {
    const int mt = (pl.table_mt == 1 || pl.table_mt == 2) ? pl.table_mt : choose_mt(c, p.m_total, sms, AMODE == A_CONV_TMA || F16);
    if (mt == 2) return prepare_mt<AMODE, EPI, F16, 2, false>(pl, c, sms, 1);
  }
  if constexpr ((a_mode_uses_tma(AMODE) && AMODE != A_CONV_WIN) || AMODE == A_CONV_I8) {  // (the window form is used on full grids only;
                                                                                        //  of the gathers, the u8 convolution's has a split-K form)
    int ks = choose_ksplit(c, p.m_total, sms, pl.table_ksplit);
    // all clusters must be resident at once: a cluster needs its CTAs on SMs of one GPC, so fewer
    // clusters fit than SMs / size suggests (measured: 49 clusters of 3 ran in two rounds)
    const long long tiles1 = (p.m_total + kTileM - 1) / kTileM * c.n_tiles;
    while (ks > 1) {
      const int per = (c.k_stages + ks - 1) / ks;
      if ((c.k_stages + per - 1) / per == ks && tiles1 <= max_active_clusters<AMODE, EPI, F16>(c, ks)) break;
      --ks;
    }
    if (ks > 1) return prepare_mt<AMODE, EPI, F16, 1, true>(pl, c, sms, ks);
    // experiment builds: the split-K kernel with clusters of one CTA
    static const int force1 = tuning_int("UNIT_B200_KSPLIT_ONE", 0);
    if (force1 && (long long)((p.m_total + kTileM - 1) / kTileM) * c.n_tiles <= sms) return prepare_mt<AMODE, EPI, F16, 1, true>(pl, c, sms, 1);
  }
  return prepare_mt<AMODE, EPI, F16, 1, false>(pl, c, sms, 1);
}

// The int8 convolution's epilogue is chosen at run time: one instantiation per mode.
template <int AMODE>
static int prepare_conv_i8(PlanImpl &pl, const TileCfg &c, int epi, const CUtensorMap *tmap = nullptr) {
  switch (epi) {
    case EPI_RAW_NCHWC: return prepare<AMODE, EPI_RAW_NCHWC, false>(pl, c, tmap);
    case EPI_REQ_NCHWC: return prepare<AMODE, EPI_REQ_NCHWC, false>(pl, c, tmap);
    case EPI_MUL_NCHWC: return prepare<AMODE, EPI_MUL_NCHWC, false>(pl, c, tmap);
    case EPI_RES_NCHWC: return prepare<AMODE, EPI_RES_NCHWC, false>(pl, c, tmap);
    default: return UNIT_ERR_SHAPE;
  }
}

static int run_plan(const PlanImpl &pl, cudaStream_t st) {
  if (pl.magic != kPlanMagic || pl.variant < 0 || pl.variant >= kMaxVariants) return UNIT_ERR_SHAPE;
  VariantSlot &v = variant_table()[pl.variant];
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev != pl.device || dev < 0) return UNIT_ERR_LAUNCH;
  if (!v.attr_done[dev & 63].load(std::memory_order_acquire)) {
    // not latched on failure: the next call tries again
    if (cudaFuncSetAttribute(pl.kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess) {
      cudaGetLastError();
      return UNIT_ERR_LAUNCH;
    }
    v.attr_done[dev & 63].store(true, std::memory_order_release);
  }
  if (pl.fold_n > 0) {
    const long long total = (long long)pl.fold_n * pl.fold_h2 * pl.fold_w2;
    fold2x2_kernel<<<grid_for(total), 256, 0, st>>>(static_cast<const uint2 *>(pl.fold_src), static_cast<uint4 *>(pl.fold_dst),
                                                    pl.fold_n, pl.fold_h2, pl.fold_w2);
    g_launches.fetch_add(1);
    if (cudaGetLastError() != cudaSuccess) return UNIT_ERR_LAUNCH;
  }
  IgemmParams p = pl.p;
  p.trace = g_trace.load();
  p.trace_cap = g_trace_cap.load();
  p.wait_limit_ns = g_wait_limit_ns.load();
  p.inject = g_inject.load();
  alignas(64) CUtensorMap map;
  memcpy(&map, pl.map, sizeof(map));
  // launched with programmatic stream serialisation: the kernel's prologue (barrier set-up,
  // TMEM allocation) may overlap the tail of the previous kernel in the stream; the kernel waits
  // for that kernel's completion (griddepcontrol.wait) before it touches global memory
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(pl.grid);
  cfg.blockDim = dim3(kNumThreads);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = use_pdl() ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (pl.cluster > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = pl.cluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  void *args[2] = {&p, &map};
  const cudaError_t le = cudaLaunchKernelExC(&cfg, pl.kernel, args);
  g_launches.fetch_add(1);
  v.launches.fetch_add(1);
  return (le == cudaSuccess && cudaGetLastError() == cudaSuccess) ? UNIT_OK : UNIT_ERR_LAUNCH;
}

// Multiplier for n / d, valid for 0 <= n < 2^31: q = umulhi(n, mul) >> shr (mul == 0: shift only).
static FastDiv make_fast_div(uint32_t d) {
  FastDiv f{0u, 0u};
  if (d == 0) d = 1;
  uint32_t l = 0;
  while ((1ull << l) < d) ++l;  // ceil(log2 d)
  if ((d & (d - 1)) == 0) {
    f.shr = l;
  } else {
    f.mul = (uint32_t)((1ull << (31 + l)) / d + 1);
    f.shr = l - 1;
  }
  return f;
}

// Tensors smaller than 128 KB are never described by a tensor map.  For such tensors, with
// drivers up to CUDA 13.1, CUTLASS edits the descriptor that cuTensorMapEncodeTiled /
// cuTensorMapEncodeIm2col return (cute/atom/copy_traits_sm90_tma.hpp and
// copy_traits_sm90_im2col.hpp clear one bit of its second word when the tensor's extent is below
// 131072 bytes); the descriptor is opaque and this library does not edit it, so operands below that
// size take the cp.async gather instead, which loses nothing on problems that small.
static bool tensor_map_allowed(long long tensor_bytes) { return tensor_bytes >= 131072; }

// im2col-mode tensor map over NCHW16c activations, seen as the 5-D tensor
//   (c = 16 channels of a chunk, w, h, d = image, n = channel chunk)
// so that one copy walks kTileM consecutive output positions (w, then h, then image) of one
// chunk.  Returns false when the driver entry point is missing or rejects the geometry; the
// caller then uses the cp.async gather.
static bool make_im2col_map(CUtensorMap *map, const unit_conv_desc *d, const void *x, bool f16) {
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const int *, const int *, cuuint32_t, cuuint32_t, const cuuint32_t *,
                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  if (!encode) return false;
  if (!tensor_map_allowed((long long)d->n * d->c_in * d->h * d->w * (f16 ? 2 : 1))) return false;
  if (d->c_block != 16 || d->pad_w > 15 || d->pad_h > 15 || d->kw > 16 || d->kh > 16 || d->stride_w > 8 || d->stride_h > 8)
    return false;
  const cuuint64_t eb = f16 ? 2 : 1;
  const cuuint64_t cc = (cuuint64_t)d->c_in / 16;
  const cuuint64_t dims[5] = {16, (cuuint64_t)d->w, (cuuint64_t)d->h, (cuuint64_t)d->n, cc};
  const cuuint64_t plane = (cuuint64_t)d->h * d->w * 16 * eb;
  const cuuint64_t strides[4] = {16 * eb, (cuuint64_t)d->w * 16 * eb, cc * plane, plane};
  const int lower[3] = {-d->pad_w, -d->pad_h, 0};
  const int upper[3] = {d->pad_w - (d->kw - 1), d->pad_h - (d->kh - 1), 0};
  const cuuint32_t estr[5] = {1, (cuuint32_t)d->stride_w, (cuuint32_t)d->stride_h, 1, 1};
  const CUresult r = encode(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 5,
                            const_cast<void *>(x), dims, strides, lower, upper, f16 ? 8 : 16, kTileM, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// The same for one three-dimensional image [c/16][D][H][W][16] (u8): the depth axis is the map's fourth
// dimension (where the two-dimensional map has the image), the channel chunk the fifth.
static bool make_im2col_map_3d(CUtensorMap *map, const unit_conv3d_desc *d, const void *x) {
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const int *, const int *, cuuint32_t, cuuint32_t, const cuuint32_t *,
                               CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  if (!encode) return false;
  if (!tensor_map_allowed((long long)d->c_in * d->d * d->h * d->w)) return false;
  if (d->pad_w > 15 || d->pad_h > 15 || d->pad_d > 15 || d->kw > 16 || d->kh > 16 || d->kd > 16 || d->stride_w > 8 ||
      d->stride_h > 8 || d->stride_d > 8)
    return false;
  const cuuint64_t cc = (cuuint64_t)d->c_in / 16;
  const cuuint64_t dims[5] = {16, (cuuint64_t)d->w, (cuuint64_t)d->h, (cuuint64_t)d->d, cc};
  const cuuint64_t plane = (cuuint64_t)d->h * d->w * 16;
  const cuuint64_t strides[4] = {16, (cuuint64_t)d->w * 16, plane, plane * d->d};
  const int lower[3] = {-d->pad_w, -d->pad_h, -d->pad_d};
  const int upper[3] = {d->pad_w - (d->kw - 1), d->pad_h - (d->kh - 1), d->pad_d - (d->kd - 1)};
  const cuuint32_t estr[5] = {1, (cuuint32_t)d->stride_w, (cuuint32_t)d->stride_h, (cuuint32_t)d->stride_d, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 5, const_cast<void *>(x), dims, strides, lower, upper, 16,
                            kTileM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Box geometry for A_CONV_BOX: a 128-row sub-tile covers box_n images x box_h output rows x box_w
// output columns.  Picks the split with the fewest sub-tiles (least idle MMA rows), preferring
// taller boxes (longer contiguous runs per image).
struct BoxGeom {
  int bw, bh, bn, blocks_w, blocks_h, blocks_n;
  long long sub_tiles;
};
static BoxGeom choose_box(int n, int oh, int ow) {
  BoxGeom g{};
  g.bw = ow < kTileM ? ow : kTileM;
  g.blocks_w = (ow + g.bw - 1) / g.bw;
  long long best = -1;
  for (int bh = 1; bh <= oh && bh * g.bw <= kTileM; ++bh) {
    int bn = kTileM / (g.bw * bh);
    if (bn > n) bn = n;
    if (bn < 1) bn = 1;
    const long long tiles = (long long)((n + bn - 1) / bn) * ((oh + bh - 1) / bh) * g.blocks_w;
    if (best < 0 || tiles <= best) {
      best = tiles;
      g.bh = bh;
      g.bn = bn;
    }
  }
  g.blocks_h = (oh + g.bh - 1) / g.bh;
  g.blocks_n = (n + g.bn - 1) / g.bn;
  g.sub_tiles = (long long)g.blocks_n * g.blocks_h * g.blocks_w;
  return g;
}

// Tiled-mode tensor map over u8 NCHW16c activations seen as (8-byte units of a pixel row, image
// row, channel chunk, image): one copy fetches box_n x box_h row segments of box_w pixels, and
// out-of-range coordinates (the zero padding) are filled with zeros by the copy engine.
// (depth > 0: one three-dimensional image [c/16][depth][h][w][16]; the map's fourth dimension is then the
// depth axis and `n` is ignored.)
static bool make_box_map(CUtensorMap *map, int n, int c_in, int h, int w, const void *x, const BoxGeom &g,
                         int extra_w = 0, int depth = 0) {
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  if (!encode || !tensor_map_allowed((long long)(depth > 0 ? depth : n) * c_in * h * w)) return false;
  const cuuint64_t cc = (cuuint64_t)c_in / 16;
  const cuuint64_t dims[4] = {(cuuint64_t)w * 2, (cuuint64_t)h, cc, (cuuint64_t)(depth > 0 ? depth : n)};
  const cuuint64_t row = (cuuint64_t)w * 16;
  const cuuint64_t strides[3] = {row, depth > 0 ? row * h * depth : row * h, depth > 0 ? row * h : row * h * cc};
  const cuuint32_t box[4] = {(cuuint32_t)(g.bw + extra_w) * 2, (cuuint32_t)g.bh, 1, (cuuint32_t)g.bn};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 4, const_cast<void *>(x), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Tiled-mode tensor map over a row-major matrix of `row_bytes` used bytes per row and `ld` bytes
// between rows, seen as (8-byte half of a K column, K column, row): one copy fetches one 16-byte K
// column of 128 consecutive rows, which lands in shared memory as that column's core matrices.
// Rows past the end of the matrix are filled with zeros by the copy engine.
static bool make_dense_map(CUtensorMap *map, const void *a, long long rows, long long row_bytes, long long ld) {
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  if (!encode || ld >= (1ll << 40) || rows > 0x7fffffffll - 512) return false;
  if (!tensor_map_allowed((rows - 1) * ld + row_bytes)) return false;
  const cuuint64_t dims[3] = {2, (cuuint64_t)(row_bytes / 16), (cuuint64_t)rows};
  const cuuint64_t strides[2] = {16, (cuuint64_t)ld};
  const cuuint32_t box[3] = {2, 1, 128};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, const_cast<void *>(a), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Tiled-mode tensor map over fp16 NCHW16c activations seen as (8-byte quarter of a pixel's 32
// bytes, image column, image row, channel chunk, image), written with the 32-byte swizzle: one
// copy fetches box_n x box_h row segments of box_w pixels of one chunk; a pixel lands as one
// 32-byte operand row = one K step.  Out-of-range coordinates (the zero padding) read as zeros.
static bool make_box_map_f16(CUtensorMap *map, int n, int c_in, int h, int w, const void *x, const BoxGeom &g) {
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  if (!encode || !tensor_map_allowed(2ll * n * c_in * h * w)) return false;
  const cuuint64_t cc = (cuuint64_t)c_in / 16;
  const cuuint64_t dims[5] = {4, (cuuint64_t)w, (cuuint64_t)h, cc, (cuuint64_t)n};
  const cuuint64_t row = (cuuint64_t)w * 32;
  const cuuint64_t strides[4] = {32, row, row * h, row * h * cc};
  const cuuint32_t box[5] = {4, (cuuint32_t)g.bw, (cuuint32_t)g.bh, 1, (cuuint32_t)g.bn};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 5, const_cast<void *>(x), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Tiled-mode tensor map over u8 NCHW16c activations seen as (8-byte quarters of a pixel pair, pair, image
// row, chunk, image): one copy fetches box_n x box_h x box_w pairs, taking every second image row, and
// writes them as 32-byte-swizzled rows (one K step of the pair form).
static bool make_pair_map(CUtensorMap *map, int n, int c_in, int h, int w, const void *x, const BoxGeom &g) {
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  if (!encode || (w & 1) || !tensor_map_allowed((long long)n * c_in * h * w)) return false;
  if (2 * g.bh - 1 > 256) return false;
  const cuuint64_t cc = (cuuint64_t)c_in / 16;
  const cuuint64_t dims[5] = {4, (cuuint64_t)w / 2, (cuuint64_t)h, cc, (cuuint64_t)n};
  const cuuint64_t row = (cuuint64_t)w * 16;
  const cuuint64_t strides[4] = {32, row, row * h, row * h * cc};
  const cuuint32_t box[5] = {4, (cuuint32_t)g.bw, (cuuint32_t)(2 * g.bh - 1), 1, (cuuint32_t)g.bn};
  const cuuint32_t estr[5] = {1, 1, 2, 1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 5, const_cast<void *>(x), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Tiled-mode tensor map over a row-major byte matrix for the 128-byte-swizzled operand layout:
// one copy fetches 128 bytes of K of 128 consecutive rows (full cache lines) and writes them as
// 1 KB atoms of 8 rows with the 16-byte chunks permuted by the row number.  Bytes and rows past
// the end of the matrix are filled with zeros.
static bool make_dense_map_sw128(CUtensorMap *map, const void *a, long long rows, long long row_bytes, long long ld) {
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      fn = nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  if (!encode || ld >= (1ll << 40) || rows > 0x7fffffffll - 512 || row_bytes >= (1ll << 31)) return false;
  if (!tensor_map_allowed((rows - 1) * ld + row_bytes)) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld};
  const cuuint32_t box[2] = {128, 128};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(a), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// Experiment builds: UNIT_B200_SW128=0 keeps the column copies for plain matrices.
static bool use_sw128() {
  static const int v = tuning_int("UNIT_B200_SW128", 1);
  return v != 0;
}

// Experiment builds: UNIT_B200_TMA=0 selects the cp.async gather everywhere.
static bool use_tma() {
  static const int v = tuning_int("UNIT_B200_TMA", 1);
  return v != 0;
}

static void fill_conv(IgemmParams &p, const unit_conv_desc *d, int elem_bytes) {
  p.H = d->h; p.W = d->w; p.Cc = d->c_in / d->c_block;
  p.KH = d->kh; p.KW = d->kw; p.sh = d->stride_h; p.sw = d->stride_w; p.ph = d->pad_h; p.pw = d->pad_w;
  p.OH = (d->h + 2 * d->pad_h - d->kh) / d->stride_h + 1;
  p.OW = (d->w + 2 * d->pad_w - d->kw) / d->stride_w + 1;
  p.kwg = (d->kw + 3) / 4;
  p.img_bytes = (long long)d->c_in * d->h * d->w * elem_bytes;
  p.m_total = (long long)d->n * p.OH * p.OW;
  p.n_total = d->c_out;
  p.div_ohw = make_fast_div((uint32_t)(p.OH * p.OW));
  p.div_ow = make_fast_div((uint32_t)p.OW);
  p.cols_per_chunk = elem_bytes;
  // the two-dimensional case of the fields that three-dimensional convolutions set differently
  p.KD = 1; p.sd = 1; p.pd = 0;
  p.out_grp_stride = (long long)p.OH * p.OW;
  p.out_img_stride = (long long)(d->c_out / 16) * p.OH * p.OW;
  p.src_img_bytes = p.img_bytes;
  p.src_chunk_bytes = (long long)d->h * d->w * d->c_block * elem_bytes;
  p.src_imgs = d->n;
}

static void set_box(IgemmParams &p, const BoxGeom &g, int n) {
  p.box_n = g.bn; p.box_h = g.bh; p.box_w = g.bw; p.blocks_h = g.blocks_h; p.blocks_w = g.blocks_w;
  p.n_img = n;
  p.sub_tiles = g.sub_tiles;
  p.div_box_hw = make_fast_div((uint32_t)(g.bh * g.bw));
  p.div_box_w = make_fast_div((uint32_t)g.bw);
  p.div_blocks_w = make_fast_div((uint32_t)g.blocks_w);
  p.div_blocks_h = make_fast_div((uint32_t)g.blocks_h);
  p.m_total = g.sub_tiles * kTileM;  // rows of the padded tiling; the kernel masks the idle ones
}

static size_t stem_workspace_bytes(const unit_conv_desc *d) {
  const StemFold f = stem_fold(d, true);
  return f.ok ? (size_t)d->n * f.h2 * f.w2 * 16 : 0;
}

// The int8 convolution's epilogue as the entry points describe it.
struct EpilogueArgs {
  const int32_t *bias = nullptr;
  int mul = 1;                      // s32 output only
  int shift = 0;                    // u8 output only
  bool out_u8 = false;
  const uint8_t *residual = nullptr;  // u8 output only
  bool x_signed = false;
};

static int plan_conv_i8(PlanImpl &pl, const unit_conv_desc *d, const void *x, const void *pw, const EpilogueArgs &e,
                        void *out, void *workspace, size_t workspace_bytes) {
  int rc = check_conv(d, false);
  if (rc) return rc;
  if (!x || !pw || !out) return UNIT_ERR_NULL;
  if (!aligned16(x) || !aligned16(pw) || !aligned16(out) || (e.bias && !aligned16(e.bias)) ||
      (workspace && !aligned16(workspace)) || (e.residual && !aligned16(e.residual)))
    return UNIT_ERR_ALIGN;
  if (e.out_u8 && (e.shift < 1 || e.shift > 31 || e.mul != 1)) return UNIT_ERR_SHAPE;
  if (!e.out_u8 && (e.residual != nullptr || e.shift != 0)) return UNIT_ERR_SHAPE;
  if ((rc = check_arch())) return rc;
  const int epi = e.out_u8 ? (e.residual ? EPI_RES_NCHWC : EPI_REQ_NCHWC) : (e.mul != 1 ? EPI_MUL_NCHWC : EPI_RAW_NCHWC);
  const TileCfg c = conv_cfg_i8(d);
  pl = PlanImpl{};
  {
    unit_tile_entry te;
    if (d->c_block == 16 && tile_lookup(d, &te)) {
      pl.table_mt = te.mt;
      pl.table_ksplit = te.ksplit;
    }
  }
  IgemmParams &p = pl.p;
  p.a = static_cast<const uint8_t *>(x); p.b = static_cast<const uint8_t *>(pw); p.out = out; p.bias = e.bias; p.shift = e.shift;
  p.mul = e.mul; p.residual = e.residual; p.a_signed = e.x_signed ? 1 : 0;
  fill_conv(p, d, 1);
  p.acc_bound = 255ll * 128ll * d->c_in * d->kh * d->kw;
  CUtensorMap map;
  if (d->c_block == 16) {
    if (use_tma() && win_weights_ok(d) && pl.table_mt == 0) {
      // stride 1, kernels of several taps: window form when its tiling of the padded image wastes little.
      // Two sub-tiles per tile if that still fills the SMs, else one; grids too small for either go on
      // to the box form below (which can split the reduction).
      const TileCfg wc = win_cfg(d);
      const int sms = sm_count();
      for (int mt = 2; mt >= 1; --mt) {
        const WinGeom g = win_geom(d, mt, wc);
        const long long tiles = (long long)d->n * g.tpi * wc.n_tiles;
        if (!g.ok || tiles < (mt == 2 ? 2 : 1) * (long long)sms) continue;
        BoxGeom bg{};
        bg.bw = g.wp; bg.bh = g.rows; bg.bn = 1;
        if (!make_box_map(&map, d->n, d->c_in, d->h, d->w, x, bg)) break;
        p.b = static_cast<const uint8_t *>(pw) + (size_t)c.n_tiles * c.k_stages * c.b_stage_bytes;  // the second packed copy
        p.win_wp = g.wp; p.win_rows = g.rows; p.win_bytes = g.bytes; p.win_box_bytes = g.box_bytes; p.win_tpi = g.tpi;
        p.div_wp = make_fast_div((uint32_t)g.wp);
        p.div_tpi = make_fast_div((uint32_t)g.tpi);
        p.n_img = d->n;
        p.m_total = (long long)d->n * g.tpi * kTileM * mt;
        pl.table_mt = mt;
        pl.table_ksplit = 1;
        TileCfg wcm = wc;
        wcm.a_stage_bytes = 2 * (size_t)g.bytes;
        return prepare_conv_i8<A_CONV_WIN>(pl, wcm, epi, &map);
      }
    }
    if (use_tma() && d->stride_h == 1 && d->stride_w == 1) {
      // stride 1: whole pixel rows per copy
      const BoxGeom g = choose_box(d->n, p.OH, p.OW);
      if (make_box_map(&map, d->n, d->c_in, d->h, d->w, x, g)) {
        set_box(p, g, d->n);
        return prepare_conv_i8<A_CONV_BOX>(pl, c, epi, &map);
      }
    }
    const PairGeom pg = pair_geom(d);
    if (use_tma() && pg.ok && d->w % 2 == 0) {
      // stride 2, several taps per kernel row, even width: dense rows of pixel pairs, one K step per pair
      const BoxGeom g = choose_box(d->n, p.OH, p.OW);
      if (make_pair_map(&map, d->n, d->c_in, d->h, d->w, x, g)) {
        const TileCfg pc = pair_cfg(d, pg);
        set_box(p, g, d->n);
        p.a_sw32 = 1;
        p.KW = pg.G;       // the producer walks (kh, pair offset, chunk)
        p.pw = -pg.qmin;   // first pair of a box row = first output column + qmin
        p.b = static_cast<const uint8_t *>(pw) + (size_t)c.n_tiles * c.k_stages * c.b_stage_bytes;  // the second packed copy
        return prepare_conv_i8<A_CONV_BOX>(pl, pc, epi, &map);
      }
    }
    if (use_tma() && make_im2col_map(&map, d, x, false)) return prepare_conv_i8<A_CONV_TMA>(pl, c, epi, &map);
    return prepare_conv_i8<A_CONV_I8>(pl, c, epi);
  }
  // NCHW4c.  With scratch memory a stride-2 stem runs as a stride-1 convolution on 2x2-folded
  // pixels (whole pixel rows per copy); otherwise the 4-byte gather does it in place.
  const StemFold f = stem_fold(d, true);
  const size_t need = stem_workspace_bytes(d);
  if (use_tma() && f.ok && workspace != nullptr && workspace_bytes >= need) {
    const TileCfg cf = make_cfg(d->c_out, f.th * f.tw);
    const size_t generic_bytes = (size_t)c.n_tiles * c.k_stages * c.b_stage_bytes;
    PlanImpl q = pl;  // OH, OW, output geometry and epilogue stay; the input side changes
    q.p.a = static_cast<const uint8_t *>(workspace);
    q.p.b = static_cast<const uint8_t *>(pw) + generic_bytes;
    q.p.H = f.h2; q.p.W = f.w2; q.p.Cc = 1; q.p.KH = f.th; q.p.KW = f.tw; q.p.sh = q.p.sw = 1; q.p.ph = f.pad_h; q.p.pw = f.pad_w;
    q.p.img_bytes = (long long)f.h2 * f.w2 * 16;
    q.p.src_img_bytes = q.p.img_bytes;
    q.p.src_chunk_bytes = q.p.img_bytes;
    const BoxGeom g = choose_box(d->n, q.p.OH, q.p.OW);
    // row form (one copy per kernel row instead of one per tap) when a sub-tile is a single row
    // segment, the kernel width is even (column pairs stay inside a kernel row) and the stages
    // hold whole kernel rows
    const bool row_form = use_row_form() && g.bn == 1 && g.bh == 1 && f.tw % 2 == 0 && cf.kc % f.tw == 0 &&
                          cf.cols % cf.kc == 0 && (g.bw + f.tw - 1) * 2 <= 256;
    if (make_box_map(&map, d->n, 16, f.h2, f.w2, workspace, g, row_form ? f.tw - 1 : 0)) {
      set_box(q.p, g, d->n);
      q.p.row_kw = row_form ? f.tw : 0;
      q.p.row_bytes = (g.bw + f.tw - 1) * 16;
      q.fold_n = d->n; q.fold_h2 = f.h2; q.fold_w2 = f.w2;
      q.fold_src = x; q.fold_dst = workspace;
      pl = q;
      return prepare_conv_i8<A_CONV_BOX>(pl, cf, epi, &map);
    }
  }
  return prepare_conv_i8<A_STEM_I8>(pl, c, epi);
}

static int conv_i8(const unit_conv_desc *d, const void *x, const void *pw, const EpilogueArgs &e, void *out,
                   void *workspace, size_t workspace_bytes, cudaStream_t st) {
  PlanImpl pl;
  const int rc = plan_conv_i8(pl, d, x, pw, e, out, workspace, workspace_bytes);
  return rc ? rc : run_plan(pl, st);
}

// ---- three-dimensional int8 convolution (one image per launch) ----
static int check_conv3d(const unit_conv3d_desc *d) {
  if (!d) return UNIT_ERR_NULL;
  if (d->n < 1 || d->c_in < 1 || d->d < 1 || d->h < 1 || d->w < 1 || d->c_out < 1 || d->kd < 1 || d->kh < 1 || d->kw < 1 ||
      d->stride_d < 1 || d->stride_h < 1 || d->stride_w < 1 || d->pad_d < 0 || d->pad_h < 0 || d->pad_w < 0)
    return UNIT_ERR_SHAPE;
  if (d->c_in % 16 || d->c_out % 16) return UNIT_ERR_LAYOUT;
  if (d->d + 2 * d->pad_d < d->kd || d->h + 2 * d->pad_h < d->kh || d->w + 2 * d->pad_w < d->kw) return UNIT_ERR_SHAPE;
  if (d->kd > 16 || d->kh > 16 || d->kw > 16) return UNIT_ERR_SHAPE;
  const long long img = (long long)d->c_in * d->d * d->h * d->w;
  if (img >= (1ll << 31)) return UNIT_ERR_TOO_LARGE;
  const long long od = (d->d + 2 * d->pad_d - d->kd) / d->stride_d + 1, oh = (d->h + 2 * d->pad_h - d->kh) / d->stride_h + 1,
                  ow = (d->w + 2 * d->pad_w - d->kw) / d->stride_w + 1;
  if (od * oh * ow >= (1ll << 31) - 512 || od * oh * ow * d->c_out >= (1ll << 31)) return UNIT_ERR_TOO_LARGE;
  return UNIT_OK;
}
static TileCfg conv3d_cfg(const unit_conv3d_desc *d) {
  const bool cheap = d->stride_d == 1 && d->stride_h == 1 && d->stride_w == 1;
  return make_cfg(d->c_out, d->kd * d->kh * d->kw * (d->c_in / 16), cheap);
}

// Plan for image `img` of the batch.  The depth axis takes the place of the two-dimensional kernel's
// image axis: a 128-row tile runs over (od, oh, ow) of one image.
static int plan_conv3d_i8(PlanImpl &pl, const unit_conv3d_desc *d, const uint8_t *x, const void *pw, const EpilogueArgs &e,
                          void *out) {
  const TileCfg c = conv3d_cfg(d);
  const int epi = e.out_u8 ? (e.residual ? EPI_RES_NCHWC : EPI_REQ_NCHWC) : (e.mul != 1 ? EPI_MUL_NCHWC : EPI_RAW_NCHWC);
  pl = PlanImpl{};
  IgemmParams &p = pl.p;
  p.a = x; p.b = static_cast<const uint8_t *>(pw); p.out = out; p.bias = e.bias; p.shift = e.shift;
  p.mul = e.mul; p.residual = e.residual; p.a_signed = e.x_signed ? 1 : 0;
  p.H = d->h; p.W = d->w; p.Cc = d->c_in / 16;
  p.KD = d->kd; p.KH = d->kh; p.KW = d->kw;
  p.sd = d->stride_d; p.sh = d->stride_h; p.sw = d->stride_w;
  p.pd = d->pad_d; p.ph = d->pad_h; p.pw = d->pad_w;
  const int OD = (d->d + 2 * d->pad_d - d->kd) / d->stride_d + 1;
  p.OH = (d->h + 2 * d->pad_h - d->kh) / d->stride_h + 1;
  p.OW = (d->w + 2 * d->pad_w - d->kw) / d->stride_w + 1;
  p.m_total = (long long)OD * p.OH * p.OW;
  p.n_total = d->c_out;
  p.div_ohw = make_fast_div((uint32_t)(p.OH * p.OW));
  p.div_ow = make_fast_div((uint32_t)p.OW);
  p.cols_per_chunk = 1;
  p.out_img_stride = (long long)p.OH * p.OW;            // one output depth position further
  p.out_grp_stride = (long long)OD * p.OH * p.OW;       // [c_out/16][OD][OH][OW][16]
  p.src_img_bytes = (long long)d->h * d->w * 16;        // one depth slice of a chunk
  p.src_chunk_bytes = p.src_img_bytes * d->d;
  p.img_bytes = p.src_img_bytes;
  p.src_imgs = d->d;
  p.n_img = OD;
  p.acc_bound = 255ll * 128ll * d->c_in * d->kd * d->kh * d->kw;
  CUtensorMap map;
  if (use_tma() && d->stride_d == 1 && d->stride_h == 1 && d->stride_w == 1) {
    const BoxGeom g = choose_box(OD, p.OH, p.OW);
    if (make_box_map(&map, 1, d->c_in, d->h, d->w, x, g, 0, d->d)) {
      set_box(p, g, OD);
      return prepare_conv_i8<A_CONV_BOX>(pl, c, epi, &map);
    }
  }
  if (use_tma() && make_im2col_map_3d(&map, d, x)) return prepare_conv_i8<A_CONV_TMA>(pl, c, epi, &map);
  return prepare_conv_i8<A_CONV_I8>(pl, c, epi);
}

// Device address of g_static_scratch on the current device.  In host code the array's name is
// only a handle for the runtime, not an address a kernel could use, so the address is looked up
// once per device (with that device current) and cached.
static int static_scratch_address(void **out) {
  static std::mutex mu;
  static void *cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return UNIT_ERR_ARCH;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void *ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) return UNIT_ERR_LAUNCH;
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return UNIT_OK;
}

template <int EB, int CB>
static void launch_pack_vec(const void *src, void *dst, int n, int c, long long hw_words, cudaStream_t st) {
  const long long total = (long long)n * ((c + CB - 1) / CB) * hw_words;
  nchw_to_nchwc_vec_kernel<EB, CB><<<grid_for(total), kPackThreads, 0, st>>>(static_cast<const uint32_t *>(src), static_cast<uint32_t *>(dst), n, c, hw_words);
}
template <int EB, int CB>
static void launch_unpack_vec(const void *src, void *dst, int n, int c, long long hw_words, cudaStream_t st) {
  const int cb_total = (c + CB - 1) / CB;
  const long long total = (long long)n * cb_total * hw_words;
  nchwc_to_nchw_vec_kernel<EB, CB><<<grid_for(total), 256, 0, st>>>(static_cast<const uint32_t *>(src), static_cast<uint32_t *>(dst), n, c, cb_total, hw_words);
}

}  // namespace unit

using namespace unit;

extern "C" {

int unit_version(void) { return 100; }

const char *unit_status_string(int s) {
  switch (s) {
    case UNIT_OK: return "ok";
    case UNIT_ERR_NULL: return "null pointer";
    case UNIT_ERR_SHAPE: return "unsupported shape";
    case UNIT_ERR_ALIGN: return "pointer or pitch not 16-byte aligned";
    case UNIT_ERR_LAYOUT: return "unsupported channel block or tile";
    case UNIT_ERR_ARCH: return "device is not compute capability 10.0 (sm_100a)";
    case UNIT_ERR_LAUNCH: return "CUDA launch or copy failed";
    case UNIT_ERR_DEVICE_WAIT: return "a kernel abandoned a bounded wait";
    case UNIT_ERR_TOO_LARGE: return "beyond a fixed capacity";
    default: return "unknown status";
  }
}

int unit_device_status(void *stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaStreamSynchronize(st) != cudaSuccess) return UNIT_ERR_LAUNCH;
  unsigned int w = 0;
  if (cudaMemcpyFromSymbol(&w, g_error_word, sizeof(w)) != cudaSuccess) return UNIT_ERR_LAUNCH;
  if (w != 0) {
    const unsigned int zero = 0;
    cudaMemcpyToSymbol(g_error_word, &zero, sizeof(zero));
    return UNIT_ERR_DEVICE_WAIT;
  }
  return UNIT_OK;
}

uint64_t unit_launch_count(void) { return g_launches.load(); }

int unit_trace_attach(void *d_buf, int32_t capacity_tiles) {
  if (d_buf != nullptr && (capacity_tiles < 1 || !aligned16(d_buf))) return UNIT_ERR_SHAPE;
  g_trace_cap.store(d_buf ? capacity_tiles : 0);
  g_trace.store(static_cast<unsigned long long *>(d_buf));
  return UNIT_OK;
}

int unit_tensor_peak(int32_t f16, int32_t n, int32_t issuers, int32_t iters, double *ops_per_second, void *stream) {
  int rc = check_arch();
  if (rc) return rc;
  unsigned int *err = error_word_address();
  if (err == nullptr) return UNIT_ERR_LAUNCH;
  return run_tensor_peak(f16 != 0, n, issuers, iters, err, ops_per_second, static_cast<cudaStream_t>(stream));
}

int unit_tile_table_set(const unit_tile_entry *entries, int32_t n) {
  if (n < 0 || n > kMaxTileEntries) return UNIT_ERR_TOO_LARGE;
  if (n > 0 && !entries) return UNIT_ERR_NULL;
  for (int i = 0; i < n; ++i) {
    const unit_tile_entry &e = entries[i];
    if (e.c_block != 16 || e.c_in < 16 || e.c_in % 16 || e.c_out < 16 || e.c_out % 16 || e.kh < 1 || e.kw < 1 || e.stride_h < 1 ||
        e.stride_w < 1 || e.n < 0 || (e.bn != 0 && (e.bn < 16 || e.bn > 256 || e.bn % 16)) || e.kc < 0 || e.kc > 16 || e.kc % 2 ||
        e.mt < 0 || e.mt > 2 || e.ksplit < 0 || e.ksplit > 8)
      return UNIT_ERR_SHAPE;
  }
  std::lock_guard<std::mutex> lock(g_tile_mu);
  for (int i = 0; i < n; ++i) g_tile_table[i] = entries[i];
  g_tile_entries = n;
  return UNIT_OK;
}

int unit_variant_count(void) { return kMaxVariants; }

const char *unit_variant_name(int index) {
  if (index < 0 || index >= kMaxVariants || !variant_table()[index].present) return nullptr;
  return variant_table()[index].name;
}

uint64_t unit_variant_launches(int index) {
  if (index < 0 || index >= kMaxVariants) return 0;
  return variant_table()[index].launches.load();
}

int unit_debug_set(int key, long long value) {
  switch (key) {
    case UNIT_DEBUG_WAIT_LIMIT_NS:
      if (value < 1000 || value > 60000000000ll) return UNIT_ERR_SHAPE;
      g_wait_limit_ns.store((unsigned long long)value);
      return UNIT_OK;
    case UNIT_DEBUG_STALL_WEIGHT_COPIES:
      g_inject.store(value != 0 ? 1 : 0);
      return UNIT_OK;
    default:
      return UNIT_ERR_SHAPE;
  }
}

// ---- packed weights --------------------------------------------------------
size_t unit_packed_weights_bytes_conv_i8(const unit_conv_desc *d) {
  if (check_conv(d, false)) return 0;
  const TileCfg c = conv_cfg_i8(d);
  size_t bytes = (size_t)c.n_tiles * c.k_stages * c.b_stage_bytes;
  if (win_weights_ok(d)) {  // second copy in the window form's column order
    const TileCfg wc = win_cfg(d);
    bytes += (size_t)wc.n_tiles * wc.k_stages * wc.b_stage_bytes;
  }
  const PairGeom pg = pair_geom(d);
  if (pg.ok) {  // second copy in the pair form's column order (stride 2)
    const TileCfg pc = pair_cfg(d, pg);
    bytes += (size_t)pc.n_tiles * pc.k_stages * pc.b_stage_bytes;
  }
  const StemFold f = stem_fold(d, false);
  if (f.ok) {  // second copy for the folded stride-1 form of a stride-2 stem
    const TileCfg cf = make_cfg(d->c_out, f.th * f.tw);
    bytes += (size_t)cf.n_tiles * cf.k_stages * cf.b_stage_bytes;
  }
  return bytes;
}

size_t unit_conv2d_workspace_bytes(const unit_conv_desc *d) {
  if (check_conv(d, false)) return 0;
  return stem_workspace_bytes(d);
}

int unit_pack_weights_conv_i8(const unit_conv_desc *d, const int8_t *w, void *packed, void *stream) {
  int rc = check_conv(d, false);
  if (rc) return rc;
  if (!w || !packed) return UNIT_ERR_NULL;
  if (!aligned16(w) || !aligned16(packed)) return UNIT_ERR_ALIGN;
  const TileCfg c = conv_cfg_i8(d);
  PackParams pp{};
  pp.src = reinterpret_cast<const uint8_t *>(w);
  pp.dst = static_cast<uint4 *>(packed);
  pp.mode = d->c_block == 16 ? PACK_CONV_I8 : PACK_STEM_I8;
  pp.n_total = d->c_out; pp.bn = c.bn; pp.kc = c.kc; pp.cols = c.cols; pp.k_stages = c.k_stages; pp.n_tiles = c.n_tiles;
  pp.Cc = d->c_in / d->c_block; pp.KH = d->kh; pp.KW = d->kw; pp.kwg = (d->kw + 3) / 4;
  rc = launch_pack(pp, static_cast<cudaStream_t>(stream));
  if (rc == UNIT_OK && win_weights_ok(d)) {
    const TileCfg wc = win_cfg(d);
    PackParams pwn = pp;
    pwn.dst = reinterpret_cast<uint4 *>(static_cast<uint8_t *>(packed) + (size_t)c.n_tiles * c.k_stages * c.b_stage_bytes);
    pwn.mode = PACK_CONV_WIN;
    pwn.bn = wc.bn; pwn.kc = wc.kc; pwn.cols = wc.cols; pwn.k_stages = wc.k_stages; pwn.n_tiles = wc.n_tiles;
    rc = launch_pack(pwn, static_cast<cudaStream_t>(stream));
  }
  const PairGeom pg = pair_geom(d);
  if (rc == UNIT_OK && pg.ok) {
    const TileCfg pc = pair_cfg(d, pg);
    PackParams ppr = pp;
    ppr.dst = reinterpret_cast<uint4 *>(static_cast<uint8_t *>(packed) + (size_t)c.n_tiles * c.k_stages * c.b_stage_bytes);
    ppr.mode = PACK_CONV_PAIR;
    ppr.bn = pc.bn; ppr.kc = pc.kc; ppr.cols = pc.cols; ppr.k_stages = pc.k_stages; ppr.n_tiles = pc.n_tiles;
    ppr.pair_g = pg.G; ppr.pair_qmin = pg.qmin; ppr.pair_pad = d->pad_w;
    rc = launch_pack(ppr, static_cast<cudaStream_t>(stream));
  }
  const StemFold f = stem_fold(d, false);
  if (rc == UNIT_OK && f.ok) {
    const size_t generic_bytes = (size_t)c.n_tiles * c.k_stages * c.b_stage_bytes;
    const TileCfg cf = make_cfg(d->c_out, f.th * f.tw);
    PackParams pf = pp;
    pf.dst = reinterpret_cast<uint4 *>(static_cast<uint8_t *>(packed) + generic_bytes);
    pf.mode = PACK_STEM_S2D;
    pf.bn = cf.bn; pf.kc = cf.kc; pf.cols = cf.cols; pf.k_stages = cf.k_stages; pf.n_tiles = cf.n_tiles;
    pf.tw = f.tw; pf.sft_h = f.sft_h; pf.sft_w = f.sft_w;
    rc = launch_pack(pf, static_cast<cudaStream_t>(stream));
  }
  return rc;
}

size_t unit_packed_weights_bytes_conv_f16(const unit_conv_desc *d) {
  if (check_conv(d, true)) return 0;
  const TileCfg c = make_cfg(d->c_out, conv_cols_f16(d), false);
  return (size_t)c.n_tiles * c.k_stages * c.b_stage_bytes;
}

int unit_pack_weights_conv_f16(const unit_conv_desc *d, const void *w, void *packed, void *stream) {
  int rc = check_conv(d, true);
  if (rc) return rc;
  if (!w || !packed) return UNIT_ERR_NULL;
  if (!aligned16(w) || !aligned16(packed)) return UNIT_ERR_ALIGN;
  const TileCfg c = make_cfg(d->c_out, conv_cols_f16(d), false);
  PackParams pp{};
  pp.src = static_cast<const uint8_t *>(w);
  pp.dst = static_cast<uint4 *>(packed);
  pp.mode = PACK_CONV_F16;
  pp.n_total = d->c_out; pp.bn = c.bn; pp.kc = c.kc; pp.cols = c.cols; pp.k_stages = c.k_stages; pp.n_tiles = c.n_tiles;
  pp.Cc = d->c_in / 16; pp.KH = d->kh; pp.KW = d->kw;
  return launch_pack(pp, static_cast<cudaStream_t>(stream));
}

size_t unit_packed_weights_bytes_dense_i8(int32_t n, int32_t k) {
  if (n < 16 || n % 16 || k < 16 || k % 16) return 0;
  const TileCfg c = make_cfg(n, k / 16, false, true);
  return (size_t)c.n_tiles * c.k_stages * c.b_stage_bytes;
}

int unit_pack_weights_dense_i8(int32_t n, int32_t k, int32_t tile, const int8_t *b, void *packed, void *stream) {
  if (n < 16 || n % 16 || k < 16 || k % 16) return UNIT_ERR_SHAPE;
  if (tile < 1 || n % tile) return UNIT_ERR_LAYOUT;
  if (!b || !packed) return UNIT_ERR_NULL;
  if (!aligned16(b) || !aligned16(packed)) return UNIT_ERR_ALIGN;
  const TileCfg c = make_cfg(n, k / 16, false, true);
  PackParams pp{};
  pp.src = reinterpret_cast<const uint8_t *>(b);
  pp.dst = static_cast<uint4 *>(packed);
  pp.mode = PACK_DENSE_I8;
  pp.n_total = n; pp.bn = c.bn; pp.kc = c.kc; pp.cols = c.cols; pp.k_stages = c.k_stages; pp.n_tiles = c.n_tiles;
  pp.K = k; pp.T = tile;
  return launch_pack(pp, static_cast<cudaStream_t>(stream));
}

size_t unit_packed_weights_bytes_gemm_f16(int32_t n, int32_t k) {
  if (n < 16 || n % 16 || k < 8 || k % 8) return 0;
  const TileCfg c = make_cfg(n, k / 8, false, true);
  return (size_t)c.n_tiles * c.k_stages * c.b_stage_bytes;
}

int unit_pack_weights_gemm_f16(int32_t n, int32_t k, const void *b, void *packed, void *stream) {
  if (n < 16 || n % 16 || k < 8 || k % 8) return UNIT_ERR_SHAPE;
  if (!b || !packed) return UNIT_ERR_NULL;
  if (!aligned16(b) || !aligned16(packed)) return UNIT_ERR_ALIGN;
  const TileCfg c = make_cfg(n, k / 8, false, true);
  PackParams pp{};
  pp.src = static_cast<const uint8_t *>(b);
  pp.dst = static_cast<uint4 *>(packed);
  pp.mode = PACK_GEMM_F16;
  pp.n_total = n; pp.bn = c.bn; pp.kc = c.kc; pp.cols = c.cols; pp.k_stages = c.k_stages; pp.n_tiles = c.n_tiles;
  pp.K = k;
  return launch_pack(pp, static_cast<cudaStream_t>(stream));
}

// ---- contractions ------------------------------------------------------------
int unit_conv2d_u8s8s32_nchwc(const unit_conv_desc *d, const uint8_t *x, const void *pw, const int32_t *bias,
                              int32_t *out, void *workspace, size_t workspace_bytes, void *stream) {
  EpilogueArgs e;
  e.bias = bias;
  return conv_i8(d, x, pw, e, out, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int unit_conv2d_u8s8_requant_nchwc(const unit_conv_desc *d, const uint8_t *x, const void *pw, const int32_t *bias,
                                   int32_t shift, uint8_t *out, void *workspace, size_t workspace_bytes,
                                   void *stream) {
  EpilogueArgs e;
  e.bias = bias; e.shift = shift; e.out_u8 = true;
  return conv_i8(d, x, pw, e, out, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

static int epilogue_from(const unit_epilogue *epi, EpilogueArgs *e) {
  if (!epi) return UNIT_ERR_NULL;
  e->bias = epi->d_bias;
  e->mul = epi->mul;
  e->shift = epi->shift;
  e->out_u8 = epi->out_u8 != 0;
  e->residual = epi->d_residual;
  e->x_signed = epi->x_signed != 0;
  return UNIT_OK;
}

int unit_conv2d_int8_nchwc(const unit_conv_desc *d, const void *x, const void *pw, const unit_epilogue *epi, void *out,
                           void *workspace, size_t workspace_bytes, void *stream) {
  EpilogueArgs e;
  const int rc = epilogue_from(epi, &e);
  if (rc) return rc;
  return conv_i8(d, x, pw, e, out, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int unit_conv2d_plan_int8(const unit_conv_desc *d, const void *x, const void *pw, const unit_epilogue *epi, void *out,
                          void *workspace, size_t workspace_bytes, unit_conv_plan *plan) {
  if (!plan) return UNIT_ERR_NULL;
  EpilogueArgs e;
  int rc = epilogue_from(epi, &e);
  if (rc) return rc;
  PlanImpl pl;
  rc = plan_conv_i8(pl, d, x, pw, e, out, workspace, workspace_bytes);
  if (rc) return rc;
  memset(plan, 0, sizeof(*plan));
  memcpy(plan, &pl, sizeof(pl));
  return UNIT_OK;
}

int unit_conv2d_run(const unit_conv_plan *plan, void *stream) {
  if (!plan) return UNIT_ERR_NULL;
  PlanImpl pl;
  memcpy(&pl, plan, sizeof(pl));
  return run_plan(pl, static_cast<cudaStream_t>(stream));
}

size_t unit_packed_weights_bytes_conv3d_i8(const unit_conv3d_desc *d) {
  if (check_conv3d(d)) return 0;
  const TileCfg c = conv3d_cfg(d);
  return (size_t)c.n_tiles * c.k_stages * c.b_stage_bytes;
}

int unit_pack_weights_conv3d_i8(const unit_conv3d_desc *d, const int8_t *w, void *packed, void *stream) {
  int rc = check_conv3d(d);
  if (rc) return rc;
  if (!w || !packed) return UNIT_ERR_NULL;
  if (!aligned16(w) || !aligned16(packed)) return UNIT_ERR_ALIGN;
  const TileCfg c = conv3d_cfg(d);
  PackParams pp{};
  pp.src = reinterpret_cast<const uint8_t *>(w);
  pp.dst = static_cast<uint4 *>(packed);
  pp.mode = PACK_CONV_I8;
  pp.n_total = d->c_out; pp.bn = c.bn; pp.kc = c.kc; pp.cols = c.cols; pp.k_stages = c.k_stages; pp.n_tiles = c.n_tiles;
  // [c_out/16][c_in/16][kd][kh][kw][4][16][4]: the depth and height taps form one axis of kd * kh entries
  pp.Cc = d->c_in / 16; pp.KH = d->kd * d->kh; pp.KW = d->kw;
  return launch_pack(pp, static_cast<cudaStream_t>(stream));
}

int unit_conv3d_int8_ncdhwc(const unit_conv3d_desc *d, const void *x, const void *pw, const unit_epilogue *epi, void *out,
                            void *stream) {
  int rc = check_conv3d(d);
  if (rc) return rc;
  EpilogueArgs e;
  if ((rc = epilogue_from(epi, &e))) return rc;
  if (!x || !pw || !out) return UNIT_ERR_NULL;
  if (!aligned16(x) || !aligned16(pw) || !aligned16(out) || (e.bias && !aligned16(e.bias)) || (e.residual && !aligned16(e.residual)))
    return UNIT_ERR_ALIGN;
  if (e.out_u8 && (e.shift < 1 || e.shift > 31 || e.mul != 1)) return UNIT_ERR_SHAPE;
  if (!e.out_u8 && (e.residual != nullptr || e.shift != 0)) return UNIT_ERR_SHAPE;
  if ((rc = check_arch())) return rc;
  const long long in_bytes = (long long)d->c_in * d->d * d->h * d->w;
  const long long od = (d->d + 2 * d->pad_d - d->kd) / d->stride_d + 1, oh = (d->h + 2 * d->pad_h - d->kh) / d->stride_h + 1,
                  ow = (d->w + 2 * d->pad_w - d->kw) / d->stride_w + 1;
  const long long out_elems = od * oh * ow * d->c_out;
  for (int img = 0; img < d->n; ++img) {  // one launch per image
    EpilogueArgs ei = e;
    if (e.residual) ei.residual = e.residual + img * out_elems;
    void *oi = e.out_u8 ? static_cast<void *>(static_cast<uint8_t *>(out) + img * out_elems)
                        : static_cast<void *>(static_cast<int32_t *>(out) + img * out_elems);
    PlanImpl pl;
    rc = plan_conv3d_i8(pl, d, static_cast<const uint8_t *>(x) + img * in_bytes, pw, ei, oi);
    if (rc == UNIT_OK) rc = run_plan(pl, static_cast<cudaStream_t>(stream));
    if (rc) return rc;
  }
  return UNIT_OK;
}

size_t unit_noalloc_scratch_capacity(void) { return kStaticScratchBytes; }

int unit_conv2d_u8s8_requant_nchwc_noalloc(const unit_conv_desc *d, const uint8_t *x, const void *pw,
                                           const int32_t *bias, int32_t shift, uint8_t *out, void *stream) {
  const int rc = check_conv(d, false);
  if (rc) return rc;
  if (!x || !pw || !out) return UNIT_ERR_NULL;
  if (shift < 1 || shift > 31) return UNIT_ERR_SHAPE;
  const size_t need = stem_workspace_bytes(d);
  if (need > kStaticScratchBytes) return UNIT_ERR_TOO_LARGE;  // beyond the built-in scratch: use the workspace form
  void *scratch = nullptr;
  if (need > 0) {
    const int rs = static_scratch_address(&scratch);
    if (rs) return rs;
  }
  EpilogueArgs e;
  e.bias = bias; e.shift = shift; e.out_u8 = true;
  return conv_i8(d, x, pw, e, out, scratch, need ? kStaticScratchBytes : 0, static_cast<cudaStream_t>(stream));
}

static int run_dense(bool f16, int32_t m, int32_t n, int32_t k, const void *a, int64_t lda, const void *pw, void *cmat,
                     int64_t ldc, cudaStream_t st) {
  const int eb = f16 ? 2 : 1;
  const int kq = 16 / eb;  // elements per 16-byte K column
  if (m < 1 || n < 16 || n % 16 || k < kq || k % kq) return UNIT_ERR_SHAPE;
  if (!a || !pw || !cmat) return UNIT_ERR_NULL;
  if (!aligned16(a) || !aligned16(pw) || !aligned16(cmat) || lda % 16 || lda < (int64_t)eb * k || ldc % 4 || ldc < n)
    return UNIT_ERR_ALIGN;
  int rc = check_arch();
  if (rc) return rc;
  const TileCfg c = make_cfg(n, k / kq, false, true);
  PlanImpl pl{};
  IgemmParams &p = pl.p;
  p.a = static_cast<const uint8_t *>(a); p.b = static_cast<const uint8_t *>(pw); p.out = cmat;
  p.m_total = m; p.n_total = n; p.lda = lda; p.ldc = ldc;
  p.OH = p.OW = 1;
  CUtensorMap map;
  if (use_tma() && use_sw128() && c.kc % 8 == 0 && make_dense_map_sw128(&map, a, m, (long long)eb * k, lda)) {
    p.a_sw128 = 1;
    rc = f16 ? prepare<A_DENSE_TMA, EPI_RAW_ROWS, true>(pl, c, &map) : prepare<A_DENSE_TMA, EPI_RAW_ROWS, false>(pl, c, &map);
  } else if (use_tma() && make_dense_map(&map, a, m, (long long)eb * k, lda)) {
    rc = f16 ? prepare<A_DENSE_TMA, EPI_RAW_ROWS, true>(pl, c, &map) : prepare<A_DENSE_TMA, EPI_RAW_ROWS, false>(pl, c, &map);
  } else {
    // matrices below the tensor-map size limit: the cp.async gather, single sub-tiles
    rc = f16 ? prepare<A_DENSE, EPI_RAW_ROWS, true, 1>(pl, c) : prepare<A_DENSE, EPI_RAW_ROWS, false, 1>(pl, c);
  }
  return rc ? rc : run_plan(pl, st);
}

int unit_dense_u8s8s32(int32_t m, int32_t n, int32_t k, const uint8_t *a, int64_t lda, const void *pw, int32_t *cmat,
                       int64_t ldc, void *stream) {
  return run_dense(false, m, n, k, a, lda, pw, cmat, ldc, static_cast<cudaStream_t>(stream));
}

int unit_conv2d_f16f32_nchw16c(const unit_conv_desc *d, const void *x, const void *pw, float *out, void *stream) {
  int rc = check_conv(d, true);
  if (rc) return rc;
  if (!x || !pw || !out) return UNIT_ERR_NULL;
  if (!aligned16(x) || !aligned16(pw) || !aligned16(out)) return UNIT_ERR_ALIGN;
  if ((rc = check_arch())) return rc;
  const TileCfg c = make_cfg(d->c_out, conv_cols_f16(d), false);
  PlanImpl pl{};
  IgemmParams &p = pl.p;
  p.a = static_cast<const uint8_t *>(x); p.b = static_cast<const uint8_t *>(pw); p.out = out;
  fill_conv(p, d, 2);
  CUtensorMap map;
  rc = -1;
  if (use_tma() && use_sw128() && d->stride_h == 1 && d->stride_w == 1 && c.kc % 2 == 0) {
    // stride 1: whole pixel rows per copy, one copy per K step
    const BoxGeom g = choose_box(d->n, p.OH, p.OW);
    if (make_box_map_f16(&map, d->n, d->c_in, d->h, d->w, x, g)) {
      set_box(p, g, d->n);
      p.a_sw32 = 1;
      rc = prepare<A_CONV_BOX, EPI_RAW_NCHWC, true>(pl, c, &map);
    }
  }
  if (rc == -1) {
    if (use_tma() && make_im2col_map(&map, d, x, true)) rc = prepare<A_CONV_TMA, EPI_RAW_NCHWC, true>(pl, c, &map);
    else rc = prepare<A_CONV_F16, EPI_RAW_NCHWC, true>(pl, c);
  }
  return rc ? rc : run_plan(pl, static_cast<cudaStream_t>(stream));
}

int unit_gemm_f16f32(int32_t m, int32_t n, int32_t k, const void *a, int64_t lda, const void *pw, float *cmat,
                     int64_t ldc, void *stream) {
  return run_dense(true, m, n, k, a, lda, pw, cmat, ldc, static_cast<cudaStream_t>(stream));
}

// ---- layout transforms ---------------------------------------------------------
int unit_pack_data_nchw_to_nchwc(const void *src, void *dst, int32_t n, int32_t c, int32_t h, int32_t w, int32_t cb,
                                 int32_t eb, void *stream) {
  if (!src || !dst) return UNIT_ERR_NULL;
  if (n < 1 || c < 1 || h < 1 || w < 1) return UNIT_ERR_SHAPE;
  if (cb != 4 && cb != 16) return UNIT_ERR_LAYOUT;
  if (eb != 1 && eb != 2 && eb != 4) return UNIT_ERR_LAYOUT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long hw = (long long)h * w;
  if (hw * eb % 4 == 0 && aligned16(src) && aligned16(dst)) {
    // register transpose of 4-byte words, 16-byte stores
    const long long hww = hw * eb / 4;
    if (cb == 16) {
      if (eb == 1) launch_pack_vec<1, 16>(src, dst, n, c, hww, st);
      else if (eb == 2) launch_pack_vec<2, 16>(src, dst, n, c, hww, st);
      else launch_pack_vec<4, 16>(src, dst, n, c, hww, st);
    } else {
      if (eb == 1) launch_pack_vec<1, 4>(src, dst, n, c, hww, st);
      else if (eb == 2) launch_pack_vec<2, 4>(src, dst, n, c, hww, st);
      else launch_pack_vec<4, 4>(src, dst, n, c, hww, st);
    }
  } else {
    const long long total = (long long)n * ((c + cb - 1) / cb) * hw;
    const unsigned g = grid_for(total);
    if (eb == 1) nchw_to_nchwc_kernel<uint8_t><<<g, 256, 0, st>>>((const uint8_t *)src, (uint8_t *)dst, n, c, h, w, cb);
    else if (eb == 2) nchw_to_nchwc_kernel<uint16_t><<<g, 256, 0, st>>>((const uint16_t *)src, (uint16_t *)dst, n, c, h, w, cb);
    else nchw_to_nchwc_kernel<uint32_t><<<g, 256, 0, st>>>((const uint32_t *)src, (uint32_t *)dst, n, c, h, w, cb);
  }
  g_launches.fetch_add(1);
  return cudaGetLastError() == cudaSuccess ? UNIT_OK : UNIT_ERR_LAUNCH;
}

int unit_unpack_data_nchwc_to_nchw(const void *src, void *dst, int32_t n, int32_t c, int32_t h, int32_t w, int32_t cb,
                                   int32_t eb, void *stream) {
  if (!src || !dst) return UNIT_ERR_NULL;
  if (n < 1 || c < 1 || h < 1 || w < 1) return UNIT_ERR_SHAPE;
  if (cb != 4 && cb != 16) return UNIT_ERR_LAYOUT;
  if (eb != 1 && eb != 2 && eb != 4) return UNIT_ERR_LAYOUT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const long long hw = (long long)h * w;
  if (hw * eb % 4 == 0 && aligned16(src) && aligned16(dst)) {
    const long long hww = hw * eb / 4;
    if (cb == 16) {
      if (eb == 1) launch_unpack_vec<1, 16>(src, dst, n, c, hww, st);
      else if (eb == 2) launch_unpack_vec<2, 16>(src, dst, n, c, hww, st);
      else launch_unpack_vec<4, 16>(src, dst, n, c, hww, st);
    } else {
      if (eb == 1) launch_unpack_vec<1, 4>(src, dst, n, c, hww, st);
      else if (eb == 2) launch_unpack_vec<2, 4>(src, dst, n, c, hww, st);
      else launch_unpack_vec<4, 4>(src, dst, n, c, hww, st);
    }
  } else {
    const unsigned g = grid_for((long long)n * c * hw);
    if (eb == 1) nchwc_to_nchw_kernel<uint8_t><<<g, 256, 0, st>>>((const uint8_t *)src, (uint8_t *)dst, n, c, h, w, cb);
    else if (eb == 2) nchwc_to_nchw_kernel<uint16_t><<<g, 256, 0, st>>>((const uint16_t *)src, (uint16_t *)dst, n, c, h, w, cb);
    else nchwc_to_nchw_kernel<uint32_t><<<g, 256, 0, st>>>((const uint32_t *)src, (uint32_t *)dst, n, c, h, w, cb);
  }
  g_launches.fetch_add(1);
  return cudaGetLastError() == cudaSuccess ? UNIT_OK : UNIT_ERR_LAUNCH;
}

int unit_pack_weights_oihw_to_ref_i8(const int8_t *src, int8_t *dst, int32_t o, int32_t i, int32_t kh, int32_t kw,
                                     int32_t cb, void *stream) {
  if (!src || !dst) return UNIT_ERR_NULL;
  if (o < 1 || i < 1 || kh < 1 || kw < 1) return UNIT_ERR_SHAPE;
  if (cb != 4 && cb != 16) return UNIT_ERR_LAYOUT;
  const long long total = (long long)((o + 15) / 16) * ((i + cb - 1) / cb) * kh * kw * (cb / 4) * 64;
  oihw_to_ref_i8_kernel<<<grid_for(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(src, dst, o, i, kh, kw, cb);
  g_launches.fetch_add(1);
  return cudaGetLastError() == cudaSuccess ? UNIT_OK : UNIT_ERR_LAUNCH;
}

int unit_pack_weights_oihw_to_ref_f16(const void *src, void *dst, int32_t o, int32_t i, int32_t kh, int32_t kw,
                                      void *stream) {
  if (!src || !dst) return UNIT_ERR_NULL;
  if (o < 1 || i < 1 || kh < 1 || kw < 1) return UNIT_ERR_SHAPE;
  const long long total = (long long)((o + 15) / 16) * ((i + 15) / 16) * kh * kw * 256;
  oihw_to_ref_f16_kernel<<<grid_for(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      (const uint16_t *)src, (uint16_t *)dst, o, i, kh, kw);
  g_launches.fetch_add(1);
  return cudaGetLastError() == cudaSuccess ? UNIT_OK : UNIT_ERR_LAUNCH;
}

}  // extern "C"
