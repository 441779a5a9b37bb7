// C ABI of the library (declared in include/gie_b200.h): problem validation, configuration selection inside the one
// sm_100a kernel family, plans, tensor-map encoding and launches.  Host code only; the kernels live in the other
// translation units of this directory.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

#include "gie_b200.h"
#include "internal.h"
#include "ptx.cuh"

namespace {

using namespace gieb;

// ---- error reporting -------------------------------------------------------------------------------------------
thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
int fail_cuda(cudaError_t e, const char* what) {
  (void)cudaGetLastError();  // clear the non-sticky error, as the reference's throw_cuda_error does (src/runtime/error.cpp:22-24)
  return fail(GIEB_CUDA_ERROR, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}
#define GIEB_CUDA(expr)                                  \
  do {                                                   \
    const cudaError_t gieb_e_ = (expr);                  \
    if (gieb_e_ != cudaSuccess) return fail_cuda(gieb_e_, #expr); \
  } while (0)

// ---- hardware constants of the one supported target (B200, sm_100a) -------------------------------------------------
constexpr size_t kMaxDynamicSmem = 232448;  // 227 KiB opt-in limit per CTA

size_t align256(size_t v) { return (v + 255) & ~size_t(255); }
int ceil_div(int64_t a, int64_t b) { return int((a + b - 1) / b); }
int round_up(int a, int b) { return (a + b - 1) / b * b; }

struct Geometry {
  int out_h, out_w, pq;
  int64_t pixels;      // B * P * Q
  int64_t y_elems, x_elems, w_elems;
  int esize;
};

Geometry geometry(const gieb_conv_desc& d) {
  Geometry g;
  g.out_h = (d.in_h + 2 * d.pad_h - d.dilation_h * (d.kernel_h - 1) - 1) / d.stride_h + 1;
  g.out_w = (d.in_w + 2 * d.pad_w - d.dilation_w * (d.kernel_w - 1) - 1) / d.stride_w + 1;
  g.pq = g.out_h * g.out_w;
  g.pixels = int64_t(d.batch) * g.pq;
  g.y_elems = g.pixels * d.out_channels;
  g.x_elems = int64_t(d.batch) * d.in_channels * d.in_h * d.in_w;
  g.w_elems = int64_t(d.out_channels) * d.in_channels * d.kernel_h * d.kernel_w;
  g.esize = (d.precision == GIEB_FP16 || d.precision == GIEB_BF16) ? 2 : 4;
  return g;
}

// validate_problem (src/runtime/conv2d.cpp:83-109)
int validate(const gieb_conv_desc* d) {
  if (d == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null problem descriptor");
  if (d->batch <= 0 || d->in_channels <= 0 || d->in_h <= 0 || d->in_w <= 0 || d->out_channels <= 0 || d->kernel_h <= 0 ||
      d->kernel_w <= 0)
    return fail(GIEB_INVALID_ARGUMENT, "all extents must be positive");
  if (d->stride_h <= 0 || d->stride_w <= 0) return fail(GIEB_INVALID_ARGUMENT, "strides must be positive");
  if (d->pad_h < 0 || d->pad_w < 0) return fail(GIEB_INVALID_ARGUMENT, "padding must be non-negative");
  if (d->dilation_h != 1 || d->dilation_w != 1) return fail(GIEB_UNSUPPORTED, "dilation != 1 is not supported");
  if (d->groups != 1) return fail(GIEB_UNSUPPORTED, "grouped convolution is not supported");
  if (d->precision < GIEB_FP32 || d->precision > GIEB_FP8_E4M3) return fail(GIEB_INVALID_ARGUMENT, "unknown precision id %d", d->precision);
  if (int64_t(d->in_h) + 2 * d->pad_h < d->kernel_h || int64_t(d->in_w) + 2 * d->pad_w < d->kernel_w)
    return fail(GIEB_INVALID_ARGUMENT, "kernel larger than padded input");
  const Geometry g = geometry(*d);
  if (g.out_h <= 0 || g.out_w <= 0) return fail(GIEB_INVALID_ARGUMENT, "empty output");
  const int64_t lim = 2147483647LL;
  const int64_t gk = int64_t(d->in_channels) * d->kernel_h * d->kernel_w;
  if (int64_t(d->batch) * g.out_h * g.out_w > lim || gk > lim) return fail(GIEB_INVALID_ARGUMENT, "GEMM extents exceed 32-bit indexing");
  if (int64_t(d->in_channels) * d->in_h * d->in_w > lim) return fail(GIEB_INVALID_ARGUMENT, "per-image input size exceeds 32-bit indexing");
  if (int64_t(d->out_channels) * g.out_h * g.out_w > lim) return fail(GIEB_INVALID_ARGUMENT, "per-image output size exceeds 32-bit indexing");
  return GIEB_OK;
}

// ---- configuration selection --------------------------------------------------------------------------------------
// The reference ranks ~115 kernels of six backends with a roofline model (src/runtime/perf_model.cpp:130-174).  Here
// the search space is one kernel family: (tile_n, tile_k, stages, split_k).  The estimate below counts SM cycles of
// the slowest CTA: per reduction slab max(tensor-pipe time, shared-memory read time), plus fixed prologue/epilogue
// cost, plus (for split-K) writing and re-reading FP32 partials and the extra launch.
struct Resolved {
  // 1 tensor path with im2col-mode TMA; 4 tensor path with tiled TMA over the NHWC copy (1x1, stride 1, pad 0);
  // 2 tensor path reading the caller's NCHW activations directly (1x1, stride 1, pad 0, H*W % 8 == 0); 3 FP32 SIMT;
  // 5 tensor path over row-gathered activations (few input channels: S*C <= 64)
  int variant;
  int boxes_per_image;  // variant 2: ceil(H*W / 64)
  int tile_m, tile_n, tile_k, stages, split_k;
  int pair;  // 1: the 256-pixel tile belongs to a pair of CTAs (tcgen05.mma.cta_group::2), each staging half of the weight tile
  // Width geometry the kernel and its tensor maps see: the problem's own, except on the row-gather route (variant 5),
  // where the S taps of a filter row have become channels of a tensor of width Q (kernel width 1, stride 1, no padding).
  int eff_in_w, eff_kernel_w, eff_stride_w, eff_pad_w;
  // A 1x1 convolution with stride > 1 and no padding over an NCHW tensor (variant 4): the repack copies only the pixels
  // it reads, and the kernel sees a stride-1 1x1 problem over that copy of out_h x out_w pixels per image.
  int subsampled;
  // Row-gather route with stride_w = 2 and at most 4 channels: the gathered tensor holds column PAIRS once (16 bytes per
  // position) and the im2col tensor map reads it with a pixel stride of one position, so that the windows of adjacent
  // output columns overlap in memory instead of being stored twice.  gp_t positions (8 values each) per window.
  int gather_pairs, gp_positions, gp_left, gp_t, gp_shift;
  int strip;  // the pair layout read as one position strip per (output row, filter row): see resolve()
  double est_cycles;  // the cost model's estimate for the chosen configuration (SM cycles; 0 on the FP32 path)
  int tma_epilogue;  // channel-contiguous output staged in shared memory and written by TMA stores
  int swap;          // transposed accumulator (lane = output channel): NCHW output staged per warp and written by TMA stores
  int reduce;  // 1 workspace partials + reduction launch, 2 cluster (distributed shared memory); 0 when split_k == 1
  int c_padded, kb_per_tap, total_kb, kb_per_split;
  int tiles_m, tiles_n;
  size_t smem;
  int epi_warps;  // 8, or 16 when the CTA has its SM to itself (see conv_tc_kernel)
  size_t ws_x, ws_w, ws_part, ws_total;  // workspace layout (bytes; offsets are cumulative in this order)
};

int pick_tile_k(int c) {
  const int base = round_up(c, 16);
  if (double(round_up(c, 64)) <= 1.15 * base) return 64;
  if (double(round_up(c, 32)) <= 1.15 * base) return 32;
  return 16;
}

// Measured on B200: with every SM pulling, one SM receives about 74 B/clk of operands from L2 through TMA, well below
// the 128 B/clk the tensor pipe of a 128x128 tile would need, so operand bytes per slab usually decide.  CTAs that fit
// together on an SM (shared memory and the 512 TMEM columns permitting) hide each other's prologue and epilogue.
constexpr double kFeedBytesPerClk = 74.0;
constexpr int kNumSmPairs = kNumSms / 2;  // SM pairs that can host a two-CTA cluster

size_t stage_bytes_of(int tile_m, int tile_n, int tile_k) { return size_t(tile_m + tile_n) * tile_k * 2; }
// bytes one CTA of a pair stages per slab: its 128 activation rows and half of the weight rows
size_t pair_stage_bytes_of(int tile_n, int tile_k) { return size_t(kTileM + tile_n / 2) * tile_k * 2; }

// TMEM columns one CTA allocates: one accumulator set per 128-pixel half, doubled when two sets fit 256 columns.
int tmem_cols_of(int tile_m, int tile_n) {
  const int one = tile_m / kTileM * tile_n;
  const int cols = one <= 256 ? 2 * one : one;
  return cols < 32 ? 32 : cols;
}

int resident_ctas(int tile_m, int tile_n, size_t smem) {
  int by_smem = int(kMaxDynamicSmem / (smem + 1024));
  int by_tmem = 512 / tmem_cols_of(tile_m, tile_n);
  int r = by_smem < by_tmem ? by_smem : by_tmem;
  return r < 1 ? 1 : (r > 2 ? 2 : r);  // 384 threads x 80 registers: two CTAs fill the register file
}

// Ring depth: deep enough to cover L2 latency, shallow enough that two CTAs share an SM when more than one wave of
// CTAs exists (their epilogues then overlap with another CTA's main loop).
int pick_stages(int tile_m, int tile_n, int tile_k, int kb_per_split, int64_t ctas, size_t extra_smem = 0) {
  const size_t sb = stage_bytes_of(tile_m, tile_n, tile_k);
  const int by_tmem = 512 / tmem_cols_of(tile_m, tile_n);
  // measured: with >= 2.5 tiles per SM three shallow CTAs per SM beat two deeper ones; between 1 and 2.5 two CTAs win
  int want = 1;
  if (ctas > kNumSms) want = 2;  // two CTAs per SM (the register file holds no more)
  if (want > by_tmem) want = by_tmem;
  const size_t budget = want == 1 ? kMaxDynamicSmem - 1024 : (kMaxDynamicSmem / want - 2048);
  int stages = budget > 3072 + extra_smem + sb ? int((budget - 3072 - extra_smem) / sb) : 1;
  if (stages > 6) stages = 6;
  if (stages > kb_per_split) stages = kb_per_split;
  if (stages < 2) stages = 2;
  return stages;
}

// Whether the split-K slices of one tile may be summed inside a cluster (distributed shared memory).
bool cluster_reduce_ok(int tile_m, int tile_n, int tile_k, int stages, int split) {
  const int chunks = tile_n / 32;
  return tile_m == kTileM && (split == 2 || split == 4 || split == 8) && chunks % split == 0 &&
         size_t(split - 1) * (tile_n / split) * kTileM * 4 <= size_t(stages) * stage_bytes_of(tile_m, tile_n, tile_k);
}

// Cost model in SM cycles, fitted to per-CTA clock stamps of the kernel on B200:
//  * a converged issuer needs >= 78 cycles per tcgen05.mma plus ~215 per wait / vote / fence / commit round (one round
//    per slab, or per two slabs of a narrow tile when they have queued up);
//    256-column instructions (128 pipe cycles each) hide all of that behind the tensor pipe;
//  * with every SM busy, L2 delivers ~74 B/clk of operands to each SM;
//  * CTAs that share an SM interleave their issue latencies but share pipe and feed;
//  * ~4500 cycles from launch to the first MMA, ~500 + 16 per accumulator column for an epilogue, which is hidden
//    behind the next tile's main loop when the accumulator is double-buffered or a second CTA shares the SM.
// reduce: 0 none, 1 FP32 partials in the workspace + reduction launch, 2 cluster.
// swap: the accumulator is transposed (the instruction's M is 128 channels, its N the tile's pixels), so the issue cost
// follows tile_m instead of tile_n, and the epilogue is short (one TMA store per 32 x 32 box).
double estimate_cycles(const gieb_conv_desc& d, const Geometry& g, int tile_m, int tile_n, int tile_k, int split, int reduce, int total_kb,
                       bool swap = false) {
  const int kb_per_split = ceil_div(total_kb, split);
  const int real_split = ceil_div(total_kb, kb_per_split);
  const int64_t ctas = int64_t(ceil_div(g.pixels, tile_m)) * ceil_div(d.out_channels, tile_n) * real_split;
  const int stages = pick_stages(tile_m, tile_n, tile_k, kb_per_split, ctas);
  const size_t smem = conv_tc_smem_bytes(tile_m, tile_n, tile_k, stages, 0);
  if (smem > kMaxDynamicSmem) return 1e300;
  const int mh = tile_m / kTileM;
  const int resident = resident_ctas(tile_m, tile_n, smem);
  const double tiles_per_sm = double((ctas + kNumSms - 1) / kNumSms);
  const double sharing = fmin(double(resident), tiles_per_sm);   // CTAs that really run side by side on an SM
  const int instr_n = swap ? tile_m : tile_n;                                                // N of one instruction
  const double mmas = (swap ? double(tile_n / kTileM) : double(mh)) * (tile_k / 16);        // instructions per slab
  const double pipe = mmas * (instr_n / 2.0);
  const double issue = instr_n >= 256 ? pipe : mmas * 78.0 + 110.0;  // narrow instructions: two slabs per wait / vote / fence when they queue up
  const double feed = double(stage_bytes_of(tile_m, tile_n, tile_k)) / kFeedBytesPerClk;
  const double slab = fmax(fmax(pipe, feed), issue / sharing);
  // transposed: eight warps, ~900 cycles per 32 x 32 box (TMEM load, rounding, one TMA store issue), (tile_n / 128) * (tile_m / 32) / 2 boxes per warp
  double epilogue = swap ? 300.0 + 900.0 * (tile_n / 128) * (tile_m / 64) : 500.0 + 16.0 * mh * tile_n;
  if (real_split > 1 && reduce == 1) epilogue *= 2.0;  // FP32 partials: twice the bytes
  const bool overlapped = sharing >= 2.0 || (mh * tile_n <= 256 && tiles_per_sm >= 2.0);
  double total = 4500.0 + tiles_per_sm * kb_per_split * slab + (overlapped ? epilogue : tiles_per_sm * epilogue);
  if (real_split > 1) {
    if (reduce == 2)  // two cluster barriers + pushing all but the own share of the FP32 tile at ~16 B/clk
      total += 2000.0 + double(real_split - 1) / real_split * (double(kTileM) * tile_n * 4.0) / 16.0;
    else total += 6000.0 + 2.0 * real_split * double(g.y_elems) * 4.0 / 1500.0;      // extra launch + partial traffic
  }
  return total;
}

// Ring depth of a CTA pair: each CTA owns its SM, so the ring takes what shared memory is left.
int pick_pair_stages(int tile_n, int tile_k, int kb_per_split, size_t extra_smem) {
  const size_t sb = pair_stage_bytes_of(tile_n, tile_k);
  int stages = int((kMaxDynamicSmem - 1024 - 3072 - extra_smem) / sb);
  if (stages > kMaxStages) stages = kMaxStages;
  if (stages > kb_per_split) stages = kb_per_split;
  if (stages < 2) stages = 2;
  return stages;
}

// The same model for 256-pixel tiles of CTA pairs: one instruction stream drives both SMs, each SM's tensor pipe works on
// 128 x tile_n x 16 per instruction and receives (128 + tile_n / 2) operand rows per slab.
double estimate_cycles_pair(const gieb_conv_desc& d, const Geometry& g, int64_t rows, int tile_n, int tile_k, int split, int total_kb) {
  const int kb_per_split = ceil_div(total_kb, split);
  const int real_split = ceil_div(total_kb, kb_per_split);
  const int64_t pairs = int64_t(ceil_div(rows, 2 * kTileM)) * ceil_div(d.out_channels, tile_n) * real_split;
  const double tiles_per_sm = double((pairs + kNumSmPairs - 1) / kNumSmPairs);
  const double mmas = tile_k / 16;
  const double pipe = mmas * (tile_n / 2.0);
  const double issue = tile_n >= 256 ? pipe : mmas * 78.0 + 110.0;
  const double feed = double(pair_stage_bytes_of(tile_n, tile_k)) / kFeedBytesPerClk;
  const double slab = fmax(fmax(pipe, feed), issue);
  double epilogue = 500.0 + 16.0 * tile_n;
  if (real_split > 1) epilogue *= 2.0;  // FP32 partials: twice the bytes
  const bool overlapped = tile_n <= 256 && tiles_per_sm >= 2.0;  // accumulators are double-buffered
  double total = 5000.0 + tiles_per_sm * kb_per_split * slab + (overlapped ? epilogue : tiles_per_sm * epilogue);
  if (real_split > 1) total += 6000.0 + 2.0 * real_split * double(g.y_elems) * 4.0 / 1500.0;  // extra launch + partial traffic
  return total;
}

// When the heuristic chooses CTA-pair tiles unasked (a configuration can always ask for them).  Measured per layer of
// the ResNet-50-shaped chain and on the benchmark shapes: pairs win on long reductions (sixteen 64-channel slabs or more)
// when there is at least one full wave of pair tiles or the reduction is very long (3x3 over 256 channels and up); short
// reductions are bound by memory or by fixed costs, where the pair's cluster launch and its two extra cluster barriers
// cost more than the halved weight traffic returns; with few output pixels split-K inside clusters does better.
bool auto_pair(const gieb_conv_desc& d, int64_t rows, int total_kb, int tile_k) {
  const int kb64 = total_kb * tile_k / 64;  // reduction length in 64-channel slabs
  if (rows < int64_t(2 * kTileM) * 16) return false;  // few pixels: split-K inside clusters fills the machine better
  return d.out_channels >= 128 && kb64 >= 16 && (rows >= int64_t(2 * kTileM) * kNumSmPairs || kb64 >= 32);
}

}  // namespace

namespace gieb {
bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("GIEB_DISABLE_PDL");
    return !(e && e[0] == '1');
  }();
  return on;
}
// GIEB_GATHER_STRIPS=0 reads the pair layout through im2col-mode loads of whole windows (a debugging aid).
bool strips_enabled() {
  static const bool on = [] {
    const char* e = getenv("GIEB_GATHER_STRIPS");
    return !(e && e[0] == '0');
  }();
  return on;
}
// GIEB_GATHER_PAIRS=0 keeps the row-gather route on its one-window-per-pixel layout (a debugging aid).
bool pairs_enabled() {
  static const bool on = [] {
    const char* e = getenv("GIEB_GATHER_PAIRS");
    return !(e && e[0] == '0');
  }();
  return on;
}
// GIEB_DISABLE_PREFETCH=1 switches the L2 prefetches that precede the dependency waits off (a debugging aid).
bool prefetch_enabled() {
  static const bool on = [] {
    const char* e = getenv("GIEB_DISABLE_PREFETCH");
    return !(e && e[0] == '1');
  }();
  return on;
}
}  // namespace gieb

namespace {

int resolve(const gieb_conv_desc& d, const gieb_conv_cfg* user, Resolved* r, char* why, size_t why_len) {
  auto no = [&](const char* m) { snprintf(why, why_len, "%s", m); return GIEB_UNSUPPORTED; };
  memset(r, 0, sizeof(*r));
  const Geometry g = geometry(d);
  gieb_conv_cfg c;
  memset(&c, 0, sizeof(c));
  if (user) c = *user;

  // TF32 (4-byte storage) and FP8 (1-byte storage) share the restrictions of a storage type that is not 2 bytes wide: their
  // tensors pass through their own repack kernels, on the im2col and tiled routes, without the extension flags.
  const bool fp8 = d.precision == GIEB_FP8_E4M3;
  const bool tf32 = d.precision == GIEB_TF32 || fp8;   // "not a 2-byte type" in every route decision below
  if (tf32 && (d.flags & (GIEB_FLAG_WEIGHTS_PREPACKED | GIEB_FLAG_INPUT_NHWC | GIEB_FLAG_OUTPUT_NHWC | GIEB_FLAG_RESIDUAL)))
    return no("prepacked weights, channel-contiguous tensors and the fused residual are offered for FP16 / BF16 only");
  if (d.precision == GIEB_FP32) {
    if (c.variant != 0 && c.variant != 3) return no("FP32 runs on the SIMT kernel only (variant 3)");
    if (d.flags & (GIEB_FLAG_WEIGHTS_PREPACKED | GIEB_FLAG_INPUT_NHWC | GIEB_FLAG_OUTPUT_NHWC | GIEB_FLAG_RESIDUAL))
      return no("prepacked weights, channel-contiguous tensors and the fused residual apply to the 16-bit tensor path only");
    r->variant = 3;
    r->tile_m = r->tile_n = conv_fp32_tile(g.pixels, d.out_channels);
    r->tile_k = 16;
    r->stages = 2;
    r->split_k = 1;
    if (ceil_div(d.out_channels, 32) > 65535) return no("grid.y limit exceeded");
    return GIEB_OK;
  }
  const bool pointwise = d.kernel_h == 1 && d.kernel_w == 1 && d.stride_h == 1 && d.stride_w == 1 && d.pad_h == 0 && d.pad_w == 0;
  const bool direct_ok = !tf32 && pointwise && (d.in_h * d.in_w) % 8 == 0;
  if (c.variant != 0 && c.variant != 1 && c.variant != 2 && c.variant != 4 && c.variant != 5)
    return no("unknown kernel variant for 16-bit precision (1 = im2col-mode TMA, 2 = direct NCHW 1x1, 4 = tiled TMA for 1x1, 5 = row gather)");
  // Row gather: the S taps of a filter row become channels (c2 = padded S*C <= 64, one slab or less per filter row).
  // Worth it when it at least halves the padded reduction length (a 7x7 stem over 3 channels: 7*32 instead of 49*16).
  const int gather_c2 = round_up(d.kernel_w * d.in_channels, 16);
  const bool gather_ok = !tf32 && !(d.flags & GIEB_FLAG_INPUT_NHWC) && d.kernel_w > 1 && gather_c2 <= 64;
  const bool gather_pays = gather_ok && 2 * gather_c2 <= d.kernel_w * round_up(d.in_channels, 16);
  if (c.variant == 5 && !gather_ok) return no("variant 5 (row gather) needs an NCHW input, a kernel wider than 1 and kernel_w * channels <= 64");
  const bool strided_pw = !tf32 && !(d.flags & GIEB_FLAG_INPUT_NHWC) && d.kernel_h == 1 && d.kernel_w == 1 && d.pad_h == 0 && d.pad_w == 0 &&
                          (d.stride_h > 1 || d.stride_w > 1);
  if (c.variant == 4 && !pointwise && !strided_pw)
    return no("variant 4 (tiled activation loads) needs a 1x1 kernel without padding (stride 1, or any stride over an NCHW 16-bit input)");
  if (c.variant == 2 && !direct_ok) return no("variant 2 (direct NCHW loads) needs a 1x1 kernel, stride 1, no padding and H*W % 8 == 0");
  const bool in_nhwc = (d.flags & GIEB_FLAG_INPUT_NHWC) != 0;
  if (in_nhwc) {
    if (d.in_channels % 16 != 0) return no("channel-contiguous input needs a channel count that is a multiple of 16");
    if (c.variant == 2) return no("variant 2 reads NCHW activations; a channel-contiguous input takes variant 1 or 4");
  }
  r->variant = c.variant ? c.variant : (in_nhwc ? (pointwise ? 4 : 1) : (direct_ok ? 2 : ((pointwise || strided_pw) ? 4 : (gather_pays ? 5 : 1))));
  r->subsampled = (r->variant == 4 && strided_pw) ? 1 : 0;
  const bool gather = r->variant == 5;
  r->eff_in_w = gather ? g.out_w : d.in_w;
  r->eff_kernel_w = gather ? 1 : d.kernel_w;
  r->eff_stride_w = gather ? 1 : d.stride_w;
  r->eff_pad_w = gather ? 0 : d.pad_w;
  r->boxes_per_image = ceil_div(int64_t(d.in_h) * d.in_w, 64);
  // GEMM rows: output pixels, or (variant 2) 64-pixel boxes that never straddle an image
  if (gather && d.stride_w == 2 && d.in_w % 2 == 0 && d.in_channels <= 4 && d.kernel_w - 1 - d.pad_w >= 0 && pairs_enabled()) {
    const int left = (d.pad_w + 1) / 2, after = (d.kernel_w - 1 - d.pad_w) / 2;
    const int t = left + after + 1;
    if (t == 2 || t == 4 || t == 8) {
      int right = (g.out_w - 1) + after - (d.in_w / 2 - 1);
      if (right < 0) right = 0;
      r->gather_pairs = 1;
      r->gp_left = left; r->gp_t = t; r->gp_shift = 2 * left - d.pad_w;
      r->gp_positions = d.in_w / 2 + left + right;
    }
  }
  // The pair layout read as STRIPS: one 128-row tile per output row, whose operand for filter row r is the strip of positions
  // of ONE input row (a single 2 KiB box instead of 128 pixels x 64 bytes), multiplied as overlapping windows through an
  // unswizzled descriptor.  Needs out_w <= 128 and a CTA that finishes its tiles alone.
  r->strip = (r->gather_pairs && g.out_w <= 128 && c.split_k <= 1 && c.reduce == 0 && c.cta_pair != 2 && (c.tile_k == 0 || c.tile_k == r->gp_t * 8) &&
              strips_enabled()) ? 1 : 0;   // (one slab per filter row: the strip is loaded once per slab)
  const int64_t rows = r->strip ? int64_t(d.batch) * g.out_h * 128 : (r->variant == 2 ? int64_t(d.batch) * r->boxes_per_image * 64 : g.pixels);

  // hardware limits of the im2col-mode tensor map (rank 4): traversal strides 1..8, corners and offsets 8-bit
  if (d.stride_h > 8 || d.stride_w > 8) return no("stride > 8 cannot be expressed by the TMA im2col traversal stride");
  if (d.pad_h > 127 || d.pad_w > 127 || d.kernel_h > 128 || d.kernel_w > 128) return no("padding/kernel extent exceeds the TMA im2col corner range");

  if (fp8) {
    // FP8 storage: a 128/64/32-byte slab row holds 128/64/32 values.  cfg.tile_k counts FP8 values; internally every tile
    // and padding quantity is kept in 2-byte units (half the FP8 counts), as for TF32.
    if (c.variant == 2 || c.variant == 5) return no("FP8 runs on the im2col (1) and tiled (4) routes");
    int tk = c.tile_k;
    if (tk == 0) {
      const int base = round_up(d.in_channels, 32);
      tk = double(round_up(d.in_channels, 128)) <= 1.15 * base ? 128 : (double(round_up(d.in_channels, 64)) <= 1.15 * base ? 64 : 32);
    }
    if (tk != 32 && tk != 64 && tk != 128) return no("tile_k must be 32, 64 or 128 for FP8 (values per slab row)");
    r->tile_k = tk / 2;
  } else if (tf32) {
    // FP32 storage: a 128/64/32-byte slab row holds 32/16/8 values.  cfg.tile_k counts FP32 values; internally every
    // tile and padding quantity is kept in 2-byte units (twice the FP32 counts) so that the byte layouts coincide.
    if (c.variant == 2 || c.variant == 5) return no("TF32 runs on the im2col (1) and tiled (4) routes");
    int tk = c.tile_k;
    if (tk == 0) {
      const int base = round_up(d.in_channels, 8);
      tk = double(round_up(d.in_channels, 32)) <= 1.15 * base ? 32 : (double(round_up(d.in_channels, 16)) <= 1.15 * base ? 16 : 8);
    }
    if (tk != 8 && tk != 16 && tk != 32) return no("tile_k must be 8, 16 or 32 for TF32 (FP32 values per slab row)");
    r->tile_k = 2 * tk;
  } else {
    r->tile_k = c.tile_k ? c.tile_k : (in_nhwc ? (d.in_channels % 64 == 0 ? 64 : (d.in_channels % 32 == 0 ? 32 : 16)) : pick_tile_k(d.in_channels));
  }
  if (r->tile_k != 16 && r->tile_k != 32 && r->tile_k != 64) return no("tile_k must be 16, 32 or 64");
  if (in_nhwc && d.in_channels % r->tile_k != 0) return no("tile_k must divide the channel count of a channel-contiguous input (it is read in place)");
  if (gather) {
    const int gc2 = r->gather_pairs ? r->gp_t * 8 : gather_c2;
    if (!c.tile_k) r->tile_k = gc2 % 64 == 0 ? 64 : (gc2 % 32 == 0 ? 32 : 16);
    if (gc2 % r->tile_k != 0) return no("tile_k must divide the gathered row length (padded kernel_w * channels)");
    r->c_padded = gc2;
  } else if (fp8) {
    r->c_padded = round_up(d.in_channels, 2 * r->tile_k) / 2;
  } else if (tf32) {
    r->c_padded = 2 * round_up(d.in_channels, r->tile_k / 2);
  } else {
    r->c_padded = round_up(d.in_channels, r->tile_k);
  }
  r->kb_per_tap = r->c_padded / r->tile_k;
  r->total_kb = d.kernel_h * r->eff_kernel_w * r->kb_per_tap;

  if (c.tile_n) {
    if (c.tile_n != 32 && c.tile_n != 64 && c.tile_n != 128 && c.tile_n != 256) return no("tile_n must be 32, 64, 128 or 256");
    r->tile_n = c.tile_n;
  }
  if (c.split_k < 0) return no("split_k must be >= 0");
  if (c.tile_m != 0 && c.tile_m != 128 && c.tile_m != 256) return no("tile_m must be 128 or 256");
  if (c.cta_pair < 0 || c.cta_pair > 2) return no("cta_pair must be 0 (auto), 1 (single CTA) or 2 (CTA pair)");
  if (c.cta_pair == 2) {
    if (d.precision == GIEB_TF32) return no("CTA-pair tiles are offered for FP16, BF16 and FP8");
    if (c.tile_m != 0 && c.tile_m != 256) return no("a CTA pair computes 256-pixel tiles (tile_m 0 or 256)");
    if (c.tile_n != 0 && c.tile_n < 64) return no("CTA-pair tiles are 64, 128 or 256 output channels wide");
    if (c.reduce == 2) return no("a CTA pair is a cluster already: its split-K slices are summed through the workspace (reduce 0 or 1)");
  }
  // NCHW output whose planes are 16-byte multiples, 16-bit types: 128- and 256-channel tiles that a CTA finishes alone
  // keep the accumulator transposed (lane = output channel) and write their boxes with TMA stores.
  bool swap_ok = !tf32 && !(d.flags & GIEB_FLAG_OUTPUT_NHWC) && g.pq % 8 == 0;
  bool swap_forced = false;
  if (const char* e = getenv("GIEB_TRANSPOSED_ACC")) {  // debugging aid: 0 = pixel-lane kernels only, 2 = transposed wherever it is possible
    swap_ok = swap_ok && e[0] != '0';
    swap_forced = e[0] == '2';
  }
  // search (tile_m, tile_n, split_k, pair) unless fixed
  double best = 1e300;
  int best_m = 0, best_n = 0, best_s = 0, best_mode = 0, best_pair = 0, best_swap = 0;
  const int n_opts[4] = {32, 64, 128, 256};
  // 256-pixel tiles of CTA pairs: only the workspace reduction for split-K
  const bool pair_unasked = c.cta_pair == 0 && !r->strip && d.precision != GIEB_TF32 && c.tile_m == 0 && c.split_k <= 1 && c.reduce == 0 && c.variant != 2 &&
                            auto_pair(d, rows, r->total_kb, r->tile_k);
  for (int ni = 1; ni < 4 && d.precision != GIEB_TF32 && (c.cta_pair == 2 || pair_unasked) && (c.tile_m == 0 || c.tile_m == 256) && c.reduce != 2; ++ni) {
    const int tn = n_opts[ni];
    if (r->tile_n && tn != r->tile_n) continue;
    if (!r->tile_n && tn / 2 >= d.out_channels) continue;
    if (c.cta_pair != 2 && rows <= kTileM) continue;  // the peer CTA would own no pixel
    for (int s = 1; s <= (pair_unasked ? 1 : 16); ++s) {
      if (c.split_k && s != c.split_k) continue;
      if (s > 1 && r->total_kb < 2 * s) break;
      if (s > 1 && size_t(s) * size_t(g.y_elems) * 4 > (size_t(1) << 31)) continue;
      const double t = estimate_cycles_pair(d, g, rows, tn, r->tile_k, s, r->total_kb);
      if (t < best) { best = t; best_m = 2 * kTileM; best_n = tn; best_s = s; best_mode = s > 1 ? 1 : 0; best_pair = 1; }
    }
  }
  for (int tm = 128; tm <= 256 && c.cta_pair != 2 && !(pair_unasked && best_pair); tm += 128) {
    if (c.tile_m && tm != c.tile_m) continue;
    if (!c.tile_m && tm == 256 && int64_t(ceil_div(g.pixels, 256)) * ceil_div(d.out_channels, 128) < 4 * kNumSms) continue;  // big tiles only where wave quantisation is negligible
    for (int ni = 0; ni < 4; ++ni) {
      const int tn = n_opts[ni];
      if (r->tile_n && tn != r->tile_n) continue;
      if (!r->tile_n && tn > 32 && tn / 2 >= d.out_channels) continue;  // never pad channels by 2x or more
      for (int s = 1; s <= (r->strip ? 1 : 16); ++s) {   // (position strips: a CTA finishes its tiles alone)
        if (c.split_k && s != c.split_k) continue;
        if (s > 1 && r->total_kb < 2 * s) break;  // reduction too short (src/kernels/tensor_core_mma.cu:292 rule)
        const int kbs = ceil_div(r->total_kb, s);
        const bool even = ceil_div(r->total_kb, kbs) == s;  // every slice non-empty
        const int64_t ctas = int64_t(ceil_div(rows, tm)) * ceil_div(d.out_channels, tn) * s;
        for (int mode = (s > 1 ? 1 : 0); mode <= (s > 1 ? 2 : 0); ++mode) {
          if (c.reduce && mode && mode != c.reduce) continue;
          if (mode == 1 && size_t(s) * size_t(g.y_elems) * 4 > (size_t(1) << 31)) continue;
          if (mode == 2) {
            const int st = c.stages ? c.stages : pick_stages(tm, tn, r->tile_k, kbs, ctas);
            if (!even || !cluster_reduce_ok(tm, tn, r->tile_k, st, s)) continue;
            // unasked, clusters are used only when the whole grid is one wave of one CTA per SM
            if (c.reduce == 0 && ctas > kNumSms) continue;
          }
          // tiles of 128 or 256 channels that a CTA finishes alone may keep the accumulator transposed: both forms compete
          const bool can_swap = swap_ok && s == 1 && tn >= 128;
          for (int sw = (can_swap && swap_forced ? 1 : 0); sw <= (can_swap ? 1 : 0); ++sw) {
            const double t = estimate_cycles(d, g, tm, tn, r->tile_k, s, mode, r->total_kb, sw != 0) +
                             (r->variant == 2 && tn < d.out_channels && tn < 256 ? 1e6 : 0.0);
            if (t < best) { best = t; best_m = tm; best_n = tn; best_s = s; best_mode = mode; best_pair = 0; best_swap = sw; }
          }
        }
      }
    }
  }
  if (best_n == 0) {
    if (c.reduce == 2) return no("cluster reduction needs tile_m 128, split_k 2, 4 or 8 dividing tile_n / 32 with no empty slice, and a ring that holds the received slices");
    if (c.split_k > 1) return no("reduction too short for this split-K factor");
    return no("no feasible tile configuration");
  }
  r->tile_m = best_m;
  r->tile_n = best_n;
  r->pair = best_pair;
  r->est_cycles = best;
  r->kb_per_split = ceil_div(r->total_kb, best_s);
  r->split_k = ceil_div(r->total_kb, r->kb_per_split);  // every slice non-empty
  r->tiles_m = ceil_div(rows, r->tile_m);
  r->tiles_n = ceil_div(d.out_channels, r->tile_n);
  if (int64_t(r->tiles_m) * r->tiles_n * r->split_k > 2147483647LL) return no("tile count exceeds 32-bit indexing");

  // Channel-contiguous output goes through shared-memory boxes and TMA stores when the rows of the [pixels][O] matrix
  // are 16-byte multiples, rows are numbered by pixel (not the direct-NCHW route) and each CTA finishes its tiles alone.
  r->tma_epilogue = (d.flags & GIEB_FLAG_OUTPUT_NHWC) && d.out_channels % 8 == 0 && r->variant != 2 && !r->strip && r->split_k == 1;
  bool swap = best_swap != 0 && !r->pair && !r->strip && r->split_k == 1;  // 2 KiB of staging per epilogue warp
  const int64_t total_tiles = int64_t(r->tiles_m) * r->tiles_n * r->split_k;
  auto stages_for = [&](size_t epi_smem) {
    int st = c.stages ? c.stages
             : r->pair ? pick_pair_stages(r->tile_n, r->tile_k, r->kb_per_split, epi_smem)
                       : pick_stages(r->tile_m, r->tile_n, r->tile_k, r->kb_per_split, total_tiles, epi_smem);
    // Activations streamed once from DRAM (direct-NCHW route) with a long reduction: one CTA per SM with a deep ring
    // keeps more loads in flight than two shallow ones (measured on 512 -> 128 channels at 28x28: 17.5 vs 18.4 us).
    if (!c.stages && !r->pair && r->variant == 2 && r->kb_per_split >= 8) {
      const size_t sb = stage_bytes_of(r->tile_m, r->tile_n, r->tile_k);
      if (3072 + 1024 + 6 * sb + epi_smem <= kMaxDynamicSmem) st = 6;
    }
    return st;
  };
  // A CTA that has its SM to itself drains its accumulators with 16 warps instead of 8: always for 256-column tiles
  // (measured 2-7 % per step), for 128-column tiles only when the CTA has a single tile, whose epilogue nothing hides
  // (with several tiles per CTA the extra polling warps cost more than the last epilogue gains).
  auto epi_warps_for = [&](size_t smem) {
    if (r->pair) return conv_tc_pair_epi_warps(r->tile_n);
    if (swap) return 8;  // the transposed epilogue is short: eight warps, 16 KiB of staging
    const bool alone = resident_ctas(r->tile_m, r->tile_n, smem) == 1;
    const bool single_tile = total_tiles <= kNumSms;
    return (alone && (r->tile_n >= 256 || (r->tile_n >= 128 && single_tile && best_mode != 2))) ? 16 : 8;
  };
  size_t epi_smem = r->tma_epilogue ? conv_tc_epilogue_staging_bytes(r->tile_n) : (swap ? size_t(8) * 2048 : 0);
  int stages = stages_for(epi_smem);
  if (stages < 2 || stages > kMaxStages) return no("stages must be in [2, 8]");
  r->smem = conv_tc_smem_bytes(r->tile_m, r->tile_n, r->tile_k, stages, epi_smem, r->pair != 0);
  r->epi_warps = epi_warps_for(r->smem);
  if (swap && r->smem > kMaxDynamicSmem) {  // a ring depth that was asked for leaves no room: the pixel-lane kernel
    swap = false;
    stages = stages_for(0);
    r->smem = conv_tc_smem_bytes(r->tile_m, r->tile_n, r->tile_k, stages, 0, r->pair != 0);
    r->epi_warps = epi_warps_for(r->smem);
  }
  r->swap = swap;
  r->stages = stages;
  if (r->smem > kMaxDynamicSmem) return no("configuration needs more shared memory than one CTA may have (227 KiB)");
  // A CTA of a pair keeps its SM to itself (the tensor-memory allocation of a pair spans two SMs): a short ring still
  // asks for more than half of an SM's shared memory.
  if (r->pair && r->smem < kMaxDynamicSmem / 2 + 2048) r->smem = kMaxDynamicSmem / 2 + 2048;

  // workspace: channel-padded NHWC activations, prepacked weights, split-K partials (ws_layout analogue,
  // src/kernels/tensor_core_mma.cu:265-278)
  r->ws_x = in_nhwc ? 0 : align256(size_t(d.batch) * (r->subsampled ? size_t(g.out_h) * g.out_w : size_t(d.in_h) * r->eff_in_w) * r->c_padded * 2);
  if (r->gather_pairs) r->ws_x = align256(size_t(d.batch) * d.in_h * r->gp_positions * 16);
  r->ws_w = (d.flags & GIEB_FLAG_WEIGHTS_PREPACKED) ? 0 : align256(size_t(d.out_channels) * d.kernel_h * r->eff_kernel_w * r->c_padded * 2);
  // how the split-K slices are summed
  if (c.reduce < 0 || c.reduce > 2) return no("reduce must be 0 (auto), 1 (workspace) or 2 (cluster)");
  r->reduce = r->split_k > 1 ? best_mode : 0;
  if (r->reduce == 2 && !cluster_reduce_ok(r->tile_m, r->tile_n, r->tile_k, stages, r->split_k))
    return no("cluster reduction needs tile_m 128, split_k 2, 4 or 8 dividing tile_n / 32, and a ring that holds the received slices");
  r->ws_part = r->split_k > 1 && r->reduce == 1 ? align256(size_t(r->split_k) * size_t((g.y_elems + 3) & ~int64_t(3)) * 4) : 0;
  r->ws_total = r->ws_x + r->ws_w + r->ws_part;
  if (r->ws_total > (size_t(180) << 30) / 4) return no("workspace exceeds a quarter of device memory");
  return GIEB_OK;
}

void fill_info(const gieb_conv_desc& d, const Resolved& r, gieb_conv_info* out) {
  const Geometry g = geometry(d);
  out->supported = 1;
  out->variant = r.variant;
  out->cfg.tile_m = r.tile_m;
  out->cfg.tile_n = r.tile_n;
  out->cfg.tile_k = d.precision == GIEB_TF32 ? r.tile_k / 2 : (d.precision == GIEB_FP8_E4M3 ? r.tile_k * 2 : r.tile_k);  // in elements of the storage type
  out->cfg.stages = r.stages;
  out->cfg.split_k = r.split_k;
  out->cfg.variant = r.variant;
  out->cfg.reduce = r.reduce;
  out->cfg.cta_pair = r.variant == 3 ? 0 : (r.pair ? 2 : 1);
  out->workspace_bytes = r.ws_total;
  out->persistent_bytes = sizeof(uint32_t);
  out->padded_channels = d.precision == GIEB_TF32 ? r.c_padded / 2 : (d.precision == GIEB_FP8_E4M3 ? r.c_padded * 2 : r.c_padded);
  if (r.variant == 3) {
    out->dynamic_smem_bytes = 0;
    out->threads_per_block = r.tile_n == 64 ? 256 : 64;
    out->num_blocks = conv_fp32_num_blocks(g.pixels, d.out_channels);
    out->launches = 1;
  } else {
    out->dynamic_smem_bytes = uint32_t(r.smem);
    out->threads_per_block = conv_tc_threads(r.epi_warps);
    out->num_blocks = int64_t(r.tiles_m) * r.tiles_n * r.split_k * (r.pair ? 2 : 1);
    // repack (activations and weights in one launch; none when both are consumed in place), convolution, reduction
    const bool x_in_place = r.variant == 2 || (d.flags & GIEB_FLAG_INPUT_NHWC);
    const bool w_in_place = (d.flags & GIEB_FLAG_WEIGHTS_PREPACKED) != 0 ||
                            (x_in_place && d.precision != GIEB_TF32 && d.kernel_h * d.kernel_w == 1 && r.c_padded == d.in_channels);  // 16-byte aligned w assumed
    out->launches = (x_in_place && w_in_place ? 0 : 1) + 1 + (r.reduce == 1 ? 1 : 0) + (d.precision == GIEB_TF32 ? 1 : 0);  // TF32: X and W repacked by two launches
  }
}

// ---- tensor-map encoding ------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
using EncodeIm2colFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;
EncodeIm2colFn g_encode_im2col = nullptr;
int g_driver_version = 0;
std::once_flag g_driver_once;
cudaError_t g_driver_err = cudaSuccess;

void load_driver_entry_points() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  g_driver_err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (g_driver_err != cudaSuccess || q != cudaDriverEntryPointSuccess) { if (g_driver_err == cudaSuccess) g_driver_err = cudaErrorSymbolNotFound; return; }
  g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  g_driver_err = cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &fn, cudaEnableDefault, &q);
  if (g_driver_err != cudaSuccess || q != cudaDriverEntryPointSuccess) { if (g_driver_err == cudaSuccess) g_driver_err = cudaErrorSymbolNotFound; return; }
  g_encode_im2col = reinterpret_cast<EncodeIm2colFn>(fn);
  (void)cudaDriverGetVersion(&g_driver_version);
}

CUtensorMapSwizzle swizzle_for(int tile_k) {
  return tile_k == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : (tile_k == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
}

// Drivers up to 13.1 mis-handle descriptors of tensors smaller than 128 KiB unless one descriptor bit is cleared; this
// is the work-around CUTLASS applies after both encode calls (cute/atom/copy_traits_sm90_tma.hpp and
// copy_traits_sm90_im2col.hpp in the CUTLASS 4.x header tree).
void small_tensor_fixup(CUtensorMap* m, size_t tensor_bytes) {
  if (g_driver_version <= 13010 && tensor_bytes < 131072) reinterpret_cast<uint64_t*>(m)[1] &= ~(1ull << 21);
}

}  // namespace

struct gieb_conv_plan {
  gieb_conv_desc desc;
  Resolved r;
  Geometry g;
  int device;
  uint32_t* d_status;
  long long wait_limit = ptx::kWaitLimitCycles;  // bound of every device-side wait, in SM cycles
  uint32_t debug_skip = 0;                       // see gieb_conv_plan_inject_stall
};

namespace {

// mode: 0 im2col over the NHWC copy `xn`, 1 tiled over the NHWC copy, 2 tiled straight over the caller's NCHW tensor `xn`.
int encode_maps(const gieb_conv_plan* pl, int mode, const void* xn, const void* wk, CUtensorMap* tm_act, CUtensorMap* tm_wgt) {
  const gieb_conv_desc& d = pl->desc;
  const Resolved& r = pl->r;
  const bool tf32 = d.precision == GIEB_TF32, fp8 = d.precision == GIEB_FP8_E4M3;
  const CUtensorMapDataType dt = tf32  ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                       : (d.precision == GIEB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  const CUtensorMapSwizzle sw = swizzle_for(r.tile_k);
  // element counts along channels from counts of 2-byte units: halved for 4-byte elements, doubled for 1-byte elements
  auto el = [&](uint64_t units) { return tf32 ? units >> 1 : (fp8 ? units << 1 : units); };
  if (mode == 2) {  // NCHW seen as {HW, C, N}: one box = 64 pixels (128 bytes, the swizzle span) x tile_k channels
    const cuuint64_t hw = cuuint64_t(d.in_h) * d.in_w;
    const cuuint64_t dims[3] = {hw, cuuint64_t(d.in_channels), cuuint64_t(d.batch)};
    const cuuint64_t strides[2] = {hw * 2, hw * d.in_channels * 2};
    const cuuint32_t box[3] = {64, cuuint32_t(r.tile_k), 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult res = g_encode_tiled(tm_act, dt, 3, const_cast<void*>(xn), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(GIEB_CUDA_ERROR, "cuTensorMapEncodeTiled (NCHW activations) failed with CUresult %d", int(res));
    small_tensor_fixup(tm_act, size_t(hw) * d.in_channels * d.batch * 2);
  } else if (mode == 3) {  // the pair layout {8 values, positions, H, N}: one box = the strip of 128 + T - 1 positions of one input row
    const cuuint64_t dims[4] = {8, cuuint64_t(r.gp_positions), cuuint64_t(d.in_h), cuuint64_t(d.batch)};
    const cuuint64_t strides[3] = {16, cuuint64_t(r.gp_positions) * 16, cuuint64_t(d.in_h) * r.gp_positions * 16};
    const cuuint32_t box[4] = {8, cuuint32_t(128 + r.gp_t - 1), 1, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult res = g_encode_tiled(tm_act, dt, 4, const_cast<void*>(xn), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                        CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(GIEB_CUDA_ERROR, "cuTensorMapEncodeTiled (position strips) failed with CUresult %d", int(res));
    small_tensor_fixup(tm_act, size_t(d.batch) * d.in_h * r.gp_positions * 16);
  } else if (mode == 1) {  // 1x1 / stride 1 / pad 0: the NHWC copy is the GEMM operand [pixels][Cp] itself
    const cuuint64_t plane = r.subsampled ? cuuint64_t(pl->g.out_h) * pl->g.out_w : cuuint64_t(d.in_h) * d.in_w;
    const cuuint64_t dims[2] = {cuuint64_t(el(r.c_padded)), cuuint64_t(d.batch) * plane};
    const cuuint64_t strides[1] = {cuuint64_t(r.c_padded) * 2};
    const cuuint32_t box[2] = {cuuint32_t(el(r.tile_k)), cuuint32_t(kTileM)};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult res = g_encode_tiled(tm_act, dt, 2, const_cast<void*>(xn), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(GIEB_CUDA_ERROR, "cuTensorMapEncodeTiled (activations) failed with CUresult %d", int(res));
    small_tensor_fixup(tm_act, size_t(d.batch) * plane * r.c_padded * 2);
  } else {
    const cuuint64_t dims[4] = {cuuint64_t(el(r.c_padded)), cuuint64_t(r.eff_in_w), cuuint64_t(d.in_h), cuuint64_t(d.batch)};
    cuuint64_t strides[3] = {cuuint64_t(r.c_padded) * 2, cuuint64_t(r.eff_in_w) * r.c_padded * 2,
                             cuuint64_t(d.in_h) * r.eff_in_w * r.c_padded * 2};
    if (r.gather_pairs) {  // overlapping pixels: one position (16 bytes) apart, each gp_t positions long
      strides[0] = 16;
      strides[1] = cuuint64_t(r.gp_positions) * 16;
      strides[2] = cuuint64_t(d.in_h) * r.gp_positions * 16;
    }
    const int lower[2] = {-r.eff_pad_w, -d.pad_h};
    const int upper[2] = {r.eff_pad_w - (r.eff_kernel_w - 1), d.pad_h - (d.kernel_h - 1)};
    const cuuint32_t trav[4] = {1, cuuint32_t(r.eff_stride_w), cuuint32_t(d.stride_h), 1};
    const CUresult res = g_encode_im2col(tm_act, dt, 4, const_cast<void*>(xn), dims, strides, lower, upper, cuuint32_t(el(r.tile_k)),
                                         cuuint32_t(kTileM), trav, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(GIEB_CUDA_ERROR, "cuTensorMapEncodeIm2col failed with CUresult %d", int(res));
    small_tensor_fixup(tm_act, r.gather_pairs ? size_t(d.batch) * d.in_h * r.gp_positions * 16 : size_t(d.batch) * d.in_h * r.eff_in_w * r.c_padded * 2);
  }
  {
    const cuuint64_t kp = cuuint64_t(d.kernel_h) * r.eff_kernel_w * r.c_padded;  // in 2-byte units
    const cuuint64_t dims[2] = {el(kp), cuuint64_t(d.out_channels)};
    const cuuint64_t strides[1] = {kp * 2};
    const cuuint32_t box[2] = {cuuint32_t(el(r.tile_k)), cuuint32_t(r.pair ? r.tile_n / 2 : r.tile_n)};  // a CTA of a pair loads half of the rows
    const cuuint32_t estr[2] = {1, 1};
    const CUresult res = g_encode_tiled(tm_wgt, dt, 2, const_cast<void*>(wk), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS) return fail(GIEB_CUDA_ERROR, "cuTensorMapEncodeTiled failed with CUresult %d", int(res));
    small_tensor_fixup(tm_wgt, size_t(kp) * d.out_channels * 2);
  }
  return GIEB_OK;
}

// The output (or the residual) of a channel-contiguous plan as the 2-D tensor {O channels, B*P*Q pixels}: boxes of
// 32 channels x 32 pixels with 64-byte swizzle, the unit one epilogue warp stages per TMA store / load.
int encode_epilogue_map(const gieb_conv_plan* pl, const void* ptr, CUtensorMap* tm) {
  const gieb_conv_desc& d = pl->desc;
  const CUtensorMapDataType dt = d.precision == GIEB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const cuuint64_t dims[2] = {cuuint64_t(d.out_channels), cuuint64_t(pl->g.pixels)};
  const cuuint64_t strides[1] = {cuuint64_t(d.out_channels) * 2};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult res = g_encode_tiled(tm, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                      CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) return fail(GIEB_CUDA_ERROR, "cuTensorMapEncodeTiled (epilogue tensor) failed with CUresult %d", int(res));
  small_tensor_fixup(tm, size_t(pl->g.pixels) * d.out_channels * 2);
  return GIEB_OK;
}

// `ev`, when given, receives four stage marks: before the repack, before the convolution kernel, after it, and
// after the split-K reduction (LaunchArgs::stage_events analogue, include/gpu_inference/kernel_registry.h:38-40).
int launch_impl(const gieb_conv_plan* pl, const void* x, const void* w, const void* bias, void* y, void* ws, size_t ws_bytes,
                cudaStream_t st, cudaEvent_t* ev = nullptr, const void* residual = nullptr, unsigned stage_mask = 7u) {
  // stage_mask (measurement only): bit 0 = layout repack + weight prepack, bit 1 = convolution kernel, bit 2 = split-K reduction
  if (pl == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null plan");
  const gieb_conv_desc& d = pl->desc;
  const Resolved& r = pl->r;
  if (x == nullptr || w == nullptr || y == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null device pointer");
  if (d.has_bias && bias == nullptr) return fail(GIEB_INVALID_ARGUMENT, "problem has a bias but no bias pointer was given");
  if (!d.has_bias) bias = nullptr;
  if ((d.flags & GIEB_FLAG_RESIDUAL) && residual == nullptr)
    return fail(GIEB_INVALID_ARGUMENT, "plan has a fused residual: launch it with gieb_conv_launch_fused and a residual pointer");
  if (!(d.flags & GIEB_FLAG_RESIDUAL) && residual != nullptr)
    return fail(GIEB_INVALID_ARGUMENT, "a residual was given but the plan was created without GIEB_FLAG_RESIDUAL");
  if (r.ws_total > 0) {
    if (reinterpret_cast<uintptr_t>(ws) % 256 != 0) return fail(GIEB_INVALID_ARGUMENT, "workspace must be 256-byte aligned");
    if (ws == nullptr || ws_bytes < r.ws_total)
      return fail(GIEB_WORKSPACE_TOO_SMALL, "needs %zu bytes of workspace, got %zu", r.ws_total, ws_bytes);
  }
  int cur = 0;
  GIEB_CUDA(cudaGetDevice(&cur));
  if (cur != pl->device) return fail(GIEB_INVALID_ARGUMENT, "plan was created for device %d but device %d is current", pl->device, cur);

  if (r.variant == 3) {
    if (ev) { GIEB_CUDA(cudaEventRecord(ev[0], st)); GIEB_CUDA(cudaEventRecord(ev[1], st)); }
    GIEB_CUDA(conv_fp32_launch(x, w, bias, y, d.batch, d.in_channels, d.in_h, d.in_w, d.out_channels, d.kernel_h, d.kernel_w,
                               d.stride_h, d.stride_w, d.pad_h, d.pad_w, pl->g.out_h, pl->g.out_w, d.relu, st));
    if (ev) { GIEB_CUDA(cudaEventRecord(ev[2], st)); GIEB_CUDA(cudaEventRecord(ev[3], st)); }
    return GIEB_OK;
  }

  std::call_once(g_driver_once, load_driver_entry_points);
  if (g_driver_err != cudaSuccess) return fail_cuda(g_driver_err, "resolving cuTensorMapEncode* driver entry points");

  uint8_t* wsb = static_cast<uint8_t*>(ws);
  void* xn = wsb;
  const void* wk = w;
  if (!(d.flags & GIEB_FLAG_WEIGHTS_PREPACKED)) wk = wsb + r.ws_x;
  else if (reinterpret_cast<uintptr_t>(w) % 16 != 0) return fail(GIEB_INVALID_ARGUMENT, "prepacked weights must be 16-byte aligned");
  float* part = r.reduce == 1 ? reinterpret_cast<float*>(wsb + r.ws_x + r.ws_w) : nullptr;

  // A direct-NCHW plan needs a 16-byte aligned x (TMA base address rule); otherwise this call takes the repack route.
  int mode = r.strip ? 3 : ((r.variant == 1 || r.variant == 5) ? 0 : (r.variant == 4 ? 1 : 2));
  if (mode == 2 && reinterpret_cast<uintptr_t>(x) % 16 != 0) mode = 1;
  const bool in_nhwc = (d.flags & GIEB_FLAG_INPUT_NHWC) != 0;
  if (in_nhwc) {  // read in place
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0) return fail(GIEB_INVALID_ARGUMENT, "a channel-contiguous input must be 16-byte aligned");
    xn = const_cast<void*>(x);
  }
  const int64_t rows = mode == 3 ? int64_t(d.batch) * pl->g.out_h * 128 : (mode == 2 ? int64_t(d.batch) * r.boxes_per_image * 64 : pl->g.pixels);
  // 1x1 filters over unpadded channels: OIHW *is* the [O][RS][C] layout, so when no activation repack would share the
  // launch the weights are read where they lie and the step is the convolution kernel alone (measured on 512 -> 128
  // channels at 28x28: 16.4 instead of 17.5 us per step).
  const bool w_direct = (mode == 2 || in_nhwc) && !(d.flags & GIEB_FLAG_WEIGHTS_PREPACKED) && d.precision != GIEB_TF32 &&
                        d.kernel_h * d.kernel_w == 1 && r.c_padded == d.in_channels && reinterpret_cast<uintptr_t>(w) % 16 == 0;
  if (w_direct) wk = w;

  CUtensorMap tm_act, tm_wgt;
  const int st_maps = encode_maps(pl, mode, mode == 2 ? x : xn, wk, &tm_act, &tm_wgt);
  if (st_maps != GIEB_OK) return st_maps;

  if (ev) GIEB_CUDA(cudaEventRecord(ev[0], st));
  if (!(stage_mask & 1u)) {
    // the workspace already holds the repacked tensors of an earlier full launch
  } else if (d.precision == GIEB_FP8_E4M3) {  // 1-byte tensors: their own transposing repack (one launch); c_padded is in 2-byte units
    GIEB_CUDA(repack_bytes_pair_launch(x, xn, d.batch, d.in_channels, d.in_h * d.in_w, r.c_padded * 2, w, const_cast<void*>(wk), d.out_channels,
                                       d.in_channels, d.kernel_h * d.kernel_w, r.c_padded * 2, st));
  } else if (d.precision == GIEB_TF32) {  // FP32 tensors rounded to TF32 while they are repacked (two launches)
    GIEB_CUDA(repack_tf32_launch(x, xn, d.batch, d.in_channels, d.in_h * d.in_w, r.c_padded / 2, st));
    GIEB_CUDA(repack_tf32_launch(w, const_cast<void*>(wk), d.out_channels, d.in_channels, d.kernel_h * d.kernel_w, r.c_padded / 2, st));
  } else if (r.variant == 5 && r.gather_pairs) {
    const bool with_w = !(d.flags & GIEB_FLAG_WEIGHTS_PREPACKED);
    GIEB_CUDA(gather_pairs_launch(x, xn, d.batch, d.in_channels, d.in_h, d.in_w, r.gp_positions, r.gp_left, r.gp_t, r.gp_shift,
                                  with_w ? w : nullptr, with_w ? const_cast<void*>(wk) : nullptr, d.out_channels, d.kernel_h, d.kernel_w, st));
  } else if (r.variant == 5) {  // row gather of the activations (and of the weights unless they come gathered)
    GIEB_CUDA(gather_rows_launch(x, xn, d.batch, d.in_channels, d.in_h, d.in_w, pl->g.out_w, d.kernel_w, d.stride_w, d.pad_w, r.c_padded,
                                 (d.flags & GIEB_FLAG_WEIGHTS_PREPACKED) ? nullptr : w, const_cast<void*>(wk), d.out_channels, d.kernel_h, st));
  } else if (mode == 2 || in_nhwc) {
    if (!(d.flags & GIEB_FLAG_WEIGHTS_PREPACKED) && !w_direct)
      GIEB_CUDA(repack_launch(w, const_cast<void*>(wk), d.out_channels, d.in_channels, d.kernel_h * d.kernel_w, r.c_padded, st));
  } else if (r.subsampled) {
    const bool with_w = !(d.flags & GIEB_FLAG_WEIGHTS_PREPACKED);
    GIEB_CUDA(repack_subsampled_launch(x, xn, d.batch, d.in_channels, d.in_h, d.in_w, pl->g.out_h, pl->g.out_w, d.stride_h, d.stride_w, r.c_padded,
                                       with_w ? w : nullptr, with_w ? const_cast<void*>(wk) : nullptr, d.out_channels, st));
  } else if (d.flags & GIEB_FLAG_WEIGHTS_PREPACKED)
    GIEB_CUDA(repack_launch(x, xn, d.batch, d.in_channels, d.in_h * d.in_w, r.c_padded, st));
  else
    GIEB_CUDA(repack_pair_launch(x, xn, d.batch, d.in_channels, d.in_h * d.in_w, r.c_padded, w, const_cast<void*>(wk),
                                 d.out_channels, d.in_channels, d.kernel_h * d.kernel_w, r.c_padded, st));

  ConvTcParams p;
  memset(&p, 0, sizeof(p));
  p.m_total = int(rows);
  p.y_elems = pl->g.y_elems;
  p.boxes_per_image = r.boxes_per_image;
  p.out_channels = d.out_channels;
  p.out_h = pl->g.out_h;
  p.out_w = pl->g.out_w;
  p.pq = pl->g.pq;
  p.kernel_w = r.eff_kernel_w;
  p.c_padded = r.c_padded;
  p.kb_per_tap = r.kb_per_tap;
  p.total_kb = r.total_kb;
  p.kb_per_split = r.kb_per_split;
  p.stride_h = d.stride_h; p.stride_w = r.eff_stride_w; p.pad_h = d.pad_h; p.pad_w = r.eff_pad_w;
  p.stages = r.stages;
  p.relu = d.relu; p.has_bias = d.has_bias;
  p.is_bf16 = d.precision == GIEB_BF16;
  p.is_tf32 = d.precision == GIEB_TF32;
  p.is_fp8 = d.precision == GIEB_FP8_E4M3;
  p.bias_fp32 = (p.is_tf32 || p.is_fp8 || (d.flags & GIEB_FLAG_BIAS_FP32)) ? 1 : 0;
  p.a_mode = mode;
  p.idesc = p.is_tf32 ? ptx::make_idesc_tf32(kTileM, r.tile_n, false, false)
            : r.swap  ? ptx::make_idesc_f16(kTileM, r.tile_m, p.is_bf16, false, mode == 2)  // A = 128 weight rows, B = the tile's pixels
                      : ptx::make_idesc_f16(r.pair ? 2 * kTileM : kTileM, r.tile_n, p.is_bf16, mode == 2, false);  // a pair's instruction spans 256 rows
  p.bias = bias;
  p.residual = residual;
  p.out_nhwc = (d.flags & GIEB_FLAG_OUTPUT_NHWC) ? 1 : 0;
  p.y = y;
  p.partial = part;
  p.status = pl->d_status;
  p.wait_limit = pl->wait_limit;
  p.debug_skip = pl->debug_skip;
  p.tiles_m = ceil_div(rows, r.tile_m);
  p.tiles_n = r.tiles_n;
  p.num_tiles = p.tiles_m * p.tiles_n * r.split_k;
  p.cluster_split = r.reduce == 2 ? r.split_k : 1;
  p.fd_cluster = FastDiv::make(p.cluster_split);
  p.fd_tiles_mn = FastDiv::make(p.tiles_m * p.tiles_n);
  p.fd_tiles_n = FastDiv::make(p.tiles_n);
  p.fd_pq = FastDiv::make(p.pq);
  p.fd_out_w = FastDiv::make(p.out_w);
  p.fd_kb_per_tap = FastDiv::make(p.kb_per_tap);
  p.fd_kernel_w = FastDiv::make(p.kernel_w);
  p.fd_boxes = FastDiv::make(p.boxes_per_image > 0 ? p.boxes_per_image : 1);
  p.fd_out_h = FastDiv::make(p.out_h > 0 ? p.out_h : 1);
  p.strip_bytes = r.strip ? (128 + r.gp_t - 1) * 16 : 0;
  // persistent CTAs: as many as can be resident at once, each walking the tile list
  const int64_t resident = r.pair ? kNumSmPairs : int64_t(kNumSms) * resident_ctas(r.tile_m, r.tile_n, r.smem);
  // cluster mode: one tile per CTA, blockIdx.x = tile * split + slice (the grid is a multiple of the cluster size);
  // pair mode: blockIdx.x = 2 * pair + rank, every pair walks the tile list
  dim3 grid(unsigned(p.cluster_split > 1 || p.num_tiles < resident ? p.num_tiles : resident) * (r.pair ? 2u : 1u));
  if (ev) GIEB_CUDA(cudaEventRecord(ev[1], st));
  // TMA epilogue: needs 16-byte aligned tensors; a call that is not takes the direct stores (the staging stays unused)
  CUtensorMap tm_out, tm_res;
  memset(&tm_out, 0, sizeof(tm_out));
  memset(&tm_res, 0, sizeof(tm_res));
  if (r.tma_epilogue && mode != 2 && reinterpret_cast<uintptr_t>(y) % 16 == 0 && reinterpret_cast<uintptr_t>(residual) % 16 == 0) {
    const int so = encode_epilogue_map(pl, y, &tm_out);
    if (so != GIEB_OK) return so;
    p.out_tma = 1;
    if (residual != nullptr) {
      const int sr = encode_epilogue_map(pl, residual, &tm_res);
      if (sr != GIEB_OK) return sr;
      p.res_tma = 1;
    }
  }
  if (r.swap) {
    const uintptr_t ya = reinterpret_cast<uintptr_t>(y);
    p.out_vec = (pl->g.pq % 4 == 0 && ya % 8 == 0) ? 4 : ((pl->g.pq % 2 == 0 && ya % 4 == 0) ? 2 : 1);
    p.res_vec = reinterpret_cast<uintptr_t>(residual) % 16 == 0 ? 1 : 0;
    if (ya % 16 == 0) {  // y as {P*Q, O, N}: boxes of 32 pixels x 32 channels, 64-byte swizzle
      const CUtensorMapDataType dt = d.precision == GIEB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
      const cuuint64_t pq = cuuint64_t(pl->g.pq);
      const cuuint64_t dims[3] = {pq, cuuint64_t(d.out_channels), cuuint64_t(d.batch)};
      const cuuint64_t strides[2] = {pq * 2, pq * d.out_channels * 2};
      const cuuint32_t box[3] = {32, 32, 1};
      const cuuint32_t estr[3] = {1, 1, 1};
      const CUresult res = g_encode_tiled(&tm_out, dt, 3, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (res != CUDA_SUCCESS) return fail(GIEB_CUDA_ERROR, "cuTensorMapEncodeTiled (NCHW output) failed with CUresult %d", int(res));
      small_tensor_fixup(&tm_out, size_t(pl->g.y_elems) * 2);
      p.swap_tma = 1;
    }
  }
  if (!(stage_mask & 2u)) {
  } else if (r.swap) GIEB_CUDA(conv_tc_swap_launch(r.tile_m, r.tile_n, r.tile_k, r.epi_warps, tm_act, tm_wgt, tm_out, p, grid, r.smem, st));
  else if (r.pair) GIEB_CUDA(conv_tc_pair_launch(r.tile_n, r.tile_k, tm_act, tm_wgt, tm_out, tm_res, p, grid, r.smem, st));
  else GIEB_CUDA(conv_tc_launch(r.tile_m, r.tile_n, r.tile_k, r.epi_warps, tm_act, tm_wgt, tm_out, tm_res, p, grid, r.smem, st));
  if (ev) GIEB_CUDA(cudaEventRecord(ev[2], st));
  if (r.reduce == 1 && (stage_mask & 4u))
    GIEB_CUDA(splitk_reduce_launch(part, r.split_k, pl->g.y_elems, d.out_channels, pl->g.pq, bias, p.bias_fp32, d.relu, p.is_tf32 ? 2 : p.is_bf16, residual,
                                   p.out_nhwc, y, st));
  if (ev) GIEB_CUDA(cudaEventRecord(ev[3], st));
  return GIEB_OK;
}

}  // namespace

extern "C" {

const char* gieb_last_error(void) { return g_err; }
int gieb_version(void) { return 1; }

int gieb_conv_validate(const gieb_conv_desc* desc) { return validate(desc); }

int gieb_conv_query(const gieb_conv_desc* desc, const gieb_conv_cfg* cfg, int device, gieb_conv_info* out) {
  (void)device;
  if (out == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null output");
  memset(out, 0, sizeof(*out));
  const int st = validate(desc);
  if (st != GIEB_OK) { snprintf(out->reason, sizeof(out->reason), "%s", g_err); return st; }
  Resolved r;
  const int rs = resolve(*desc, cfg, &r, out->reason, sizeof(out->reason));
  if (rs != GIEB_OK) return GIEB_OK;  // a well-formed question with the answer "not supported"
  fill_info(*desc, r, out);
  return GIEB_OK;
}

int gieb_padded_channels(const gieb_conv_desc* desc, const gieb_conv_cfg* cfg) {
  gieb_conv_info info;
  if (gieb_conv_query(desc, cfg, -1, &info) != GIEB_OK || !info.supported) return -1;
  return info.padded_channels;
}

int gieb_conv_plan_create(const gieb_conv_desc* desc, const gieb_conv_cfg* cfg, int device, gieb_conv_plan** out) {
  if (out == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null output");
  *out = nullptr;
  const int st = validate(desc);
  if (st != GIEB_OK) return st;
  Resolved r;
  char why[256] = "";
  if (resolve(*desc, cfg, &r, why, sizeof(why)) != GIEB_OK) return fail(GIEB_UNSUPPORTED, "%.255s", why);

  int prev = 0;
  GIEB_CUDA(cudaGetDevice(&prev));
  if (device < 0) device = prev;
  if (device != prev) GIEB_CUDA(cudaSetDevice(device));
  struct Restore { int prev, dev; ~Restore() { if (prev != dev) cudaSetDevice(prev); } } restore{prev, device};

  cudaDeviceProp prop;
  GIEB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) return fail(GIEB_UNSUPPORTED, "this library contains sm_100a code only; device %d is sm_%d%d", device, prop.major, prop.minor);

  gieb_conv_plan* pl = new (std::nothrow) gieb_conv_plan;
  if (pl == nullptr) return fail(GIEB_INTERNAL, "out of host memory");
  pl->desc = *desc;
  pl->r = r;
  pl->g = geometry(*desc);
  pl->device = device;
  pl->d_status = nullptr;

  // Plan-owned status word, zeroed through a private stream so no other stream is waited for or delayed
  // (the behaviour tests/test_runtime_concurrency.cu:53-73 pins for plan creation).
  cudaError_t e = cudaMalloc(&pl->d_status, sizeof(uint32_t));
  if (e == cudaSuccess) {
    cudaStream_t s = nullptr;
    e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
    if (e == cudaSuccess) {
      e = cudaMemsetAsync(pl->d_status, 0, sizeof(uint32_t), s);
      if (e == cudaSuccess) e = cudaStreamSynchronize(s);
      cudaStreamDestroy(s);
    }
  }
  if (e == cudaSuccess && r.variant != 3)
    e = r.swap ? conv_tc_swap_prepare(r.tile_m, r.tile_n, r.tile_k, r.epi_warps, kMaxDynamicSmem)
        : r.pair ? conv_tc_pair_prepare(r.tile_n, r.tile_k, kMaxDynamicSmem)
                 : conv_tc_prepare(r.tile_m, r.tile_n, r.tile_k, r.epi_warps, kMaxDynamicSmem);
  if (e != cudaSuccess) {
    if (pl->d_status) cudaFree(pl->d_status);
    delete pl;
    return fail_cuda(e, "plan creation");
  }
  *out = pl;
  return GIEB_OK;
}

void gieb_conv_plan_destroy(gieb_conv_plan* plan) {
  if (plan == nullptr) return;
  if (plan->d_status) cudaFree(plan->d_status);
  delete plan;
}

int gieb_conv_plan_info(const gieb_conv_plan* plan, gieb_conv_info* out) {
  if (plan == nullptr || out == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null argument");
  memset(out, 0, sizeof(*out));
  fill_info(plan->desc, plan->r, out);
  return GIEB_OK;
}

int gieb_conv_launch(const gieb_conv_plan* plan, const void* x, const void* w, const void* bias, void* y, void* workspace,
                     size_t workspace_bytes, void* stream) {
  return launch_impl(plan, x, w, bias, y, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int gieb_conv_plan_prepacked_weight_bytes(const gieb_conv_plan* plan, uint64_t* bytes) {
  if (plan == nullptr || bytes == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null argument");
  if (plan->r.variant == 3) return fail(GIEB_UNSUPPORTED, "the FP32 path reads OIHW weights directly");
  *bytes = uint64_t(plan->desc.out_channels) * plan->desc.kernel_h * plan->r.eff_kernel_w * plan->r.c_padded * 2;
  return GIEB_OK;
}

int gieb_conv_plan_prepack_weights(const gieb_conv_plan* plan, const void* w, void* dst, void* stream) {
  if (plan == nullptr || w == nullptr || dst == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null argument");
  const gieb_conv_desc& d = plan->desc;
  const Resolved& r = plan->r;
  if (r.variant == 3) return fail(GIEB_UNSUPPORTED, "the FP32 path reads OIHW weights directly");
  if (reinterpret_cast<uintptr_t>(dst) % 16 != 0) return fail(GIEB_INVALID_ARGUMENT, "prepacked weights must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (r.variant == 5 && r.gather_pairs)
    GIEB_CUDA(gather_pairs_launch(nullptr, nullptr, d.batch, d.in_channels, d.in_h, d.in_w, r.gp_positions, r.gp_left, r.gp_t, r.gp_shift, w, dst,
                                  d.out_channels, d.kernel_h, d.kernel_w, st));
  else if (r.variant == 5)
    GIEB_CUDA(gather_rows_launch(nullptr, nullptr, d.batch, d.in_channels, d.in_h, d.in_w, plan->g.out_w, d.kernel_w, d.stride_w, d.pad_w,
                                 r.c_padded, w, dst, d.out_channels, d.kernel_h, st));
  else
    GIEB_CUDA(repack_launch(w, dst, d.out_channels, d.in_channels, d.kernel_h * d.kernel_w, r.c_padded, st));
  return GIEB_OK;
}

int gieb_conv_launch_fused(const gieb_conv_plan* plan, const void* x, const void* w, const void* bias, const void* residual, void* y,
                           void* workspace, size_t workspace_bytes, void* stream) {
  return launch_impl(plan, x, w, bias, y, workspace, workspace_bytes, static_cast<cudaStream_t>(stream), nullptr, residual);
}

int gieb_conv_launch_stages(const gieb_conv_plan* plan, unsigned stage_mask, const void* x, const void* w, const void* bias, void* y,
                            void* workspace, size_t workspace_bytes, void* stream) {
  if (stage_mask == 0 || stage_mask > 7u) return fail(GIEB_INVALID_ARGUMENT, "stage_mask is a non-empty mask of bits 0 (repack), 1 (convolution), 2 (reduction)");
  if (plan != nullptr && plan->r.variant == 3 && !(stage_mask & 2u)) return GIEB_OK;  // the FP32 path is one kernel
  return launch_impl(plan, x, w, bias, y, workspace, workspace_bytes, static_cast<cudaStream_t>(stream), nullptr, nullptr,
                     plan != nullptr && plan->r.variant == 3 ? 7u : stage_mask);
}

int gieb_conv_time_stages(const gieb_conv_plan* plan, const void* x, const void* w, const void* bias, void* y, void* workspace,
                          size_t workspace_bytes, void* stream, int iters, float* stage_ms) {
  if (stage_ms == nullptr || iters <= 0 || iters > 4096) return fail(GIEB_INVALID_ARGUMENT, "iters must be in [1, 4096] and stage_ms non-null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaEvent_t* ev = new (std::nothrow) cudaEvent_t[size_t(iters) * 4];
  if (ev == nullptr) return fail(GIEB_INTERNAL, "out of host memory");
  int made = 0, rc = GIEB_OK;
  for (; made < iters * 4; ++made)
    if (cudaEventCreate(&ev[made]) != cudaSuccess) { rc = fail(GIEB_CUDA_ERROR, "cudaEventCreate failed"); break; }
  for (int i = 0; rc == GIEB_OK && i < iters; ++i) rc = launch_impl(plan, x, w, bias, y, workspace, workspace_bytes, st, ev + size_t(i) * 4);
  if (rc == GIEB_OK && cudaStreamSynchronize(st) != cudaSuccess) rc = fail(GIEB_CUDA_ERROR, "stream synchronisation failed");
  if (rc == GIEB_OK) {
    double acc[3] = {0, 0, 0};
    for (int i = 0; i < iters; ++i)
      for (int k = 0; k < 3; ++k) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, ev[size_t(i) * 4 + k], ev[size_t(i) * 4 + k + 1]);
        acc[k] += ms;
      }
    for (int k = 0; k < 3; ++k) stage_ms[k] = float(acc[k] / iters);
  }
  for (int i = 0; i < made; ++i) cudaEventDestroy(ev[i]);
  delete[] ev;
  return rc;
}

// ---- forward call for callers that cannot allocate device memory ------------------------------------------------
// Scratch of gieb_conv_forward_static: the first 256 bytes hold the status word the kernels report bounded-wait
// expiries to, the rest is the workspace (channel-padded NHWC copy, prepacked weights, split-K partials).
// Every GPU that loads the library holds these 8 MiB + 256 B until the process exits.
constexpr size_t kStaticScratchHeader = 256;
constexpr size_t kStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchHeader + kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
unsigned char* g_static_ptr[kMaxDevices] = {};  // device address of g_static_scratch, per device

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the address a kernel can use
// comes from cudaGetSymbolAddress, asked once per device while that device is current.
int static_scratch_for_current_device(unsigned char** out) {
  int dev = 0;
  GIEB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(GIEB_UNSUPPORTED, "device ordinal %d is outside the supported range", dev);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    unsigned char* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_scratch);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(static scratch)");
    if (p == nullptr) return fail(GIEB_INTERNAL, "the runtime returned a null address for the static scratch");
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return GIEB_OK;
}
}  // namespace

int gieb_conv_forward_static(const gieb_conv_desc* desc, const gieb_conv_cfg* cfg, const void* x, const void* w,
                             const void* bias, void* y, void* stream) {
  const int st = validate(desc);
  if (st != GIEB_OK) return st;
  if (desc->flags & GIEB_FLAG_RESIDUAL)
    return fail(GIEB_UNSUPPORTED, "the allocation-free call has no residual operand; problems with GIEB_FLAG_RESIDUAL go through a plan");
  gieb_conv_plan pl;  // lives on the host stack for the duration of this call only
  char why[256] = "";
  if (resolve(*desc, cfg, &pl.r, why, sizeof(why)) != GIEB_OK) return fail(GIEB_UNSUPPORTED, "%.255s", why);
  if (pl.r.ws_total > kStaticScratchBytes)
    return fail(GIEB_WORKSPACE_TOO_SMALL,
                "this problem needs %zu bytes of scratch but the built-in scratch holds %zu bytes; "
                "use gieb_conv_plan_create + gieb_conv_launch with a caller-provided workspace",
                pl.r.ws_total, kStaticScratchBytes);
  unsigned char* base = nullptr;
  const int ss = static_scratch_for_current_device(&base);
  if (ss != GIEB_OK) return ss;
  pl.desc = *desc;
  pl.g = geometry(*desc);
  GIEB_CUDA(cudaGetDevice(&pl.device));
  int cc_major = 0;
  GIEB_CUDA(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, pl.device));
  if (cc_major != 10) return fail(GIEB_UNSUPPORTED, "this library contains sm_100a code only; device %d has compute capability %d.x", pl.device, cc_major);
  pl.d_status = reinterpret_cast<uint32_t*>(base);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (pl.r.variant != 3)
    GIEB_CUDA(pl.r.swap ? conv_tc_swap_prepare(pl.r.tile_m, pl.r.tile_n, pl.r.tile_k, pl.r.epi_warps, kMaxDynamicSmem)
              : pl.r.pair ? conv_tc_pair_prepare(pl.r.tile_n, pl.r.tile_k, kMaxDynamicSmem)
                          : conv_tc_prepare(pl.r.tile_m, pl.r.tile_n, pl.r.tile_k, pl.r.epi_warps, kMaxDynamicSmem));
  // The array keeps whatever the previous call left: the status word must start at zero.  Everything else in the
  // scratch is fully rewritten by the repack kernels (padding channels included) and the split-K slices before use.
  GIEB_CUDA(cudaMemsetAsync(base, 0, kStaticScratchHeader, s));
  return launch_impl(&pl, x, w, bias, y, base + kStaticScratchHeader, kStaticScratchBytes, s);
}

int gieb_conv_plan_inject_stall(gieb_conv_plan* plan, uint32_t roles, uint64_t wait_limit_cycles) {
  if (plan == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null plan");
  if (roles > 3u) return fail(GIEB_INVALID_ARGUMENT, "roles is a mask of bit 0 (producers) and bit 1 (MMA issuer)");
  if (roles != 0 && (wait_limit_cycles == 0 || wait_limit_cycles > 2000000000ull))
    return fail(GIEB_INVALID_ARGUMENT, "an injected stall needs a wait limit between 1 and 2e9 SM cycles (about a second)");
  plan->debug_skip = roles;
  plan->wait_limit = roles != 0 ? static_cast<long long>(wait_limit_cycles) : ptx::kWaitLimitCycles;
  return GIEB_OK;
}

int gieb_conv_static_status(uint32_t* status_out, void* stream) {
  if (status_out == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null argument");
  unsigned char* base = nullptr;
  const int ss = static_scratch_for_current_device(&base);
  if (ss != GIEB_OK) return ss;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  GIEB_CUDA(cudaMemcpyAsync(status_out, base, sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
  GIEB_CUDA(cudaStreamSynchronize(s));
  return GIEB_OK;
}

int gieb_conv_plan_device_status(const gieb_conv_plan* plan, uint32_t* status_out) {
  if (plan == nullptr || status_out == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null argument");
  cudaStream_t s = nullptr;
  GIEB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  cudaError_t e = cudaMemcpyAsync(status_out, plan->d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  cudaStreamDestroy(s);
  if (e != cudaSuccess) return fail_cuda(e, "reading the plan status word");
  return GIEB_OK;
}

int gieb_repack_nchw_to_nhwc(const void* src, void* dst, int batch, int channels, int hw, int c_padded, void* stream) {
  if (src == nullptr || dst == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null device pointer");
  if (batch <= 0 || channels <= 0 || hw <= 0) return fail(GIEB_INVALID_ARGUMENT, "extents must be positive");
  if (c_padded < channels || c_padded % 8 != 0) return fail(GIEB_INVALID_ARGUMENT, "c_padded must be a multiple of 8 and >= channels");
  if (reinterpret_cast<uintptr_t>(dst) % 16 != 0) return fail(GIEB_INVALID_ARGUMENT, "destination must be 16-byte aligned");
  if (reinterpret_cast<uintptr_t>(src) % 2 != 0) return fail(GIEB_INVALID_ARGUMENT, "source must be 2-byte aligned");
  GIEB_CUDA(repack_launch(src, dst, batch, channels, hw, c_padded, static_cast<cudaStream_t>(stream)));
  return GIEB_OK;
}

int gieb_prepack_weights(const void* src, void* dst, int out_channels, int channels, int rs, int c_padded, void* stream) {
  return gieb_repack_nchw_to_nhwc(src, dst, out_channels, channels, rs, c_padded, stream);
}

int gieb_rmsnorm_launch(const gieb_rmsnorm_desc* d, const void* x, const void* gamma, void* y, const void* rin, void* rout,
                        void* stream) {
  // argument rules of rmsnorm_forward (src/transformer/rmsnorm.cu:155-160)
  if (d == nullptr) return fail(GIEB_INVALID_ARGUMENT, "rmsnorm: null descriptor");
  if (d->rows <= 0 || d->hidden <= 0) return fail(GIEB_INVALID_ARGUMENT, "rmsnorm: rows and hidden must be positive");
  if (!x || !gamma || !y) return fail(GIEB_INVALID_ARGUMENT, "rmsnorm: null pointer");
  if ((rin == nullptr) != (rout == nullptr)) return fail(GIEB_INVALID_ARGUMENT, "rmsnorm: residual_in and residual_out must be given together");
  if (y == x || y == gamma || y == rin || y == rout) return fail(GIEB_INVALID_ARGUMENT, "rmsnorm: y must not alias x, gamma or the residual buffers");
  if (d->dtype < 0 || d->dtype > 2) return fail(GIEB_INVALID_ARGUMENT, "rmsnorm: unknown dtype id %d", d->dtype);
  GIEB_CUDA(rmsnorm_launch(d->rows, d->hidden, d->eps, d->dtype, int(d->flags & 1u), x, gamma, y, rin, rout, static_cast<cudaStream_t>(stream)));
  return GIEB_OK;
}

int gieb_bias_act_launch(int precision, int batch, int channels, int hw, const void* bias, int relu, void* y, void* stream) {
  if (y == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null device pointer");
  if (batch <= 0 || channels <= 0 || hw <= 0) return fail(GIEB_INVALID_ARGUMENT, "extents must be positive");
  if (precision < 0 || precision > 2) return fail(GIEB_INVALID_ARGUMENT, "precision must be fp32, fp16 or bf16");
  GIEB_CUDA(bias_act_launch(precision, int64_t(batch) * channels * hw, channels, hw, bias, relu, y, static_cast<cudaStream_t>(stream)));
  return GIEB_OK;
}

int gieb_maxpool2d_launch(int precision, int batch, int channels, int h, int w, int kernel, int stride, int pad, const void* x,
                          void* y, void* stream) {
  if (x == nullptr || y == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null device pointer");
  if (batch <= 0 || channels <= 0 || h <= 0 || w <= 0 || kernel <= 0 || stride <= 0 || pad < 0 || pad >= kernel)
    return fail(GIEB_INVALID_ARGUMENT, "bad pooling geometry");
  if (h + 2 * pad < kernel || w + 2 * pad < kernel) return fail(GIEB_INVALID_ARGUMENT, "window larger than padded input");
  if (precision < 0 || precision > 2) return fail(GIEB_INVALID_ARGUMENT, "precision must be fp32, fp16 or bf16");
  GIEB_CUDA(maxpool2d_launch(precision, batch, channels, h, w, kernel, stride, pad, x, y, static_cast<cudaStream_t>(stream)));
  return GIEB_OK;
}

int gieb_maxpool2d_nhwc_launch(int precision, int batch, int channels, int h, int w, int kernel, int stride, int pad, const void* x,
                               void* y, void* stream) {
  if (x == nullptr || y == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null device pointer");
  if (batch <= 0 || channels <= 0 || h <= 0 || w <= 0 || kernel <= 0 || stride <= 0 || pad < 0 || pad >= kernel)
    return fail(GIEB_INVALID_ARGUMENT, "bad pooling geometry");
  if (h + 2 * pad < kernel || w + 2 * pad < kernel) return fail(GIEB_INVALID_ARGUMENT, "window larger than padded input");
  if (precision != GIEB_FP16 && precision != GIEB_BF16) return fail(GIEB_INVALID_ARGUMENT, "channel-contiguous pooling handles fp16 and bf16");
  if (channels % 8 != 0) return fail(GIEB_INVALID_ARGUMENT, "channel-contiguous pooling needs a channel count that is a multiple of 8");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) % 16 != 0) return fail(GIEB_INVALID_ARGUMENT, "tensors must be 16-byte aligned");
  GIEB_CUDA(maxpool2d_nhwc_launch(precision, batch, channels, h, w, kernel, stride, pad, x, y, static_cast<cudaStream_t>(stream)));
  return GIEB_OK;
}

int gieb_conv_estimate_us(const gieb_conv_desc* desc, const gieb_conv_cfg* cfg, double* microseconds) {
  if (desc == nullptr || microseconds == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null argument");
  const int st = gieb_conv_validate(desc);
  if (st != GIEB_OK) return st;
  Resolved r;
  char why[256];
  const int rs = resolve(*desc, cfg, &r, why, sizeof(why));
  if (rs != GIEB_OK) return fail(rs, "%s", why);
  // SM cycles at the 1.9 GHz these parts sustain; the FP32 path has no model: FLOPs at 20 TFLOP/s plus a launch
  if (r.variant == 3) *microseconds = 3.0 + 2.0 * double(geometry(*desc).y_elems) * desc->in_channels * desc->kernel_h * desc->kernel_w / 20e6;
  else *microseconds = r.est_cycles / 1900.0 + 3.0;
  return GIEB_OK;
}

int gieb_add_relu_launch(int precision, int relu, const void* a, const void* b, void* y, int64_t n, void* stream) {
  if (a == nullptr || b == nullptr || y == nullptr) return fail(GIEB_INVALID_ARGUMENT, "null device pointer");
  if (n <= 0) return fail(GIEB_INVALID_ARGUMENT, "element count must be positive");
  if (precision < 0 || precision > 2) return fail(GIEB_INVALID_ARGUMENT, "precision must be fp32, fp16 or bf16");
  GIEB_CUDA(add_relu_launch(precision, relu, a, b, y, n, static_cast<cudaStream_t>(stream)));
  return GIEB_OK;
}

}  // extern "C"
