// Layout repack for 16-bit tensors: [B][C][HW] -> [B][HW][Cp] with Cp >= C (extra channels written as zero).
// Used for the activations (NCHW -> channel-padded NHWC) and, with B = O and HW = R*S, for the weights
// (OIHW -> [O][R*S][Cp]).  Stands in for transpose_c_hw (src/kernels/tensor_core_mma.cu:61-82).  A pure
// permutation of 16-bit words: results are bit-exact whatever the bit patterns (NaN payloads included).
//
// The source may have any 2-byte alignment (tests/test_tensor_core.cpp:38-57 offsets X and W by one element);
// a 128-bit load path is taken when the source is 16-byte aligned and HW is a multiple of 8.  The destination is
// always written with 128-bit stores (Cp % 8 == 0, 16-byte aligned base).
#include <stdint.h>

#include "internal.h"
#include "ptx.cuh"

namespace gieb {
namespace {

constexpr int kTile = 64;          // channels and pixels per CTA tile
constexpr int kLdWords = 33;       // 32-bit words per shared-memory row (64 px + 1 word of padding)

// Tiled transpose of one 64-channel x 64-pixel tile by 256 threads; `tile` is kTile * kLdWords words of shared memory.
// LOAD: 0 = 2-byte loads (any alignment), 1 = 16-byte loads (HW % 8 == 0, 16-byte aligned source), 2 = 4-byte loads
// (HW even, 4-byte aligned source).
template <int LOAD>
__device__ __forceinline__ void repack_tile(uint32_t* tile, const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, int C,
                                            int HW, int Cp, int hw_tile, int c_tile, int b) {
  const int px0 = hw_tile * kTile;
  const int c0 = c_tile * kTile;
  const uint16_t* s = src + (size_t(b) * C + c0) * HW + px0;
  const int t = threadIdx.x;

  if (LOAD == 1) {
    // 64 channels x 8 vectors of 8 pixels; a vector never straddles HW because HW % 8 == 0.
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int v = t + i * 256;
      const int ch = v >> 3, pv = v & 7;
      uint4 q = make_uint4(0, 0, 0, 0);
      if (c0 + ch < C && px0 + pv * 8 < HW) q = *reinterpret_cast<const uint4*>(s + size_t(ch) * HW + pv * 8);
      uint32_t* d = &tile[ch * kLdWords + pv * 4];
      d[0] = q.x; d[1] = q.y; d[2] = q.z; d[3] = q.w;
    }
  } else if (LOAD == 2) {
    // 64 channels x 32 pixel pairs; a pair never straddles HW because HW is even, and every row starts 4-byte aligned
    const int pp = t & 31;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int ch = (t >> 5) + i * 8;
      uint32_t v = 0;
      if (c0 + ch < C && px0 + 2 * pp < HW) v = *reinterpret_cast<const uint32_t*>(s + size_t(ch) * HW + 2 * pp);
      tile[ch * kLdWords + pp] = v;
    }
  } else {
    uint16_t* tile16 = reinterpret_cast<uint16_t*>(tile);
    const int px = t & 63;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int ch = (t >> 6) + i * 4;
      uint16_t v = 0;
      if (c0 + ch < C && px0 + px < HW) v = s[size_t(ch) * HW + px];
      tile16[ch * (kLdWords * 2) + px] = v;
    }
  }
  __syncthreads();

  // Each thread emits one 16-byte vector = 8 consecutive channels of one pixel.  A warp covers 8 pixels x 4
  // channel groups (64 contiguous bytes per pixel) which is bank-conflict free with the 33-word row pitch.
  const uint16_t* tile16 = reinterpret_cast<const uint16_t*>(tile);
  const int lane = t & 31, warp = t >> 5;
  const int cg = (warp & 1) * 4 + (lane & 3);
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int px = ((warp >> 1) + it * 4) * 8 + (lane >> 2);
    if (px0 + px < HW && c0 + cg * 8 < Cp) {
      uint16_t o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = tile16[(cg * 8 + j) * (kLdWords * 2) + px];
      uint4 q;
      q.x = uint32_t(o[0]) | (uint32_t(o[1]) << 16);
      q.y = uint32_t(o[2]) | (uint32_t(o[3]) << 16);
      q.z = uint32_t(o[4]) | (uint32_t(o[5]) << 16);
      q.w = uint32_t(o[6]) | (uint32_t(o[7]) << 16);
      *reinterpret_cast<uint4*>(dst + (size_t(b) * HW + px0 + px) * Cp + c0 + cg * 8) = q;
    }
  }
}

// Small-HW variant (filter taps: HW = R*S <= 64).  One CTA handles `span` channels of one batch entry (a multiple of
// 64, as many as fit the shared memory: 448 for a 3x3 filter, 4096 for 1x1): the source slab [span][HW] is
// contiguous, so it is read linearly (128-bit loads when aligned), then written as [HW][span].  `slab` holds
// kTile * kSmallHwMax 16-bit words (the same shared memory as the tiled variant's tile).
constexpr int kSmallHwMax = 64;
__device__ __forceinline__ void repack_small_hw(uint16_t* slab, const uint16_t* __restrict__ src, uint16_t* __restrict__ dst,
                                                int C, int HW, int Cp, int span, int c_tile, int b) {
  const int c0 = c_tile * span;
  const int nch = min(span, C - c0);  // may be <= 0 for pure padding tiles
  const int n = nch > 0 ? nch * HW : 0;
  const uint16_t* s = src + (size_t(b) * C + c0) * HW;
  if ((reinterpret_cast<uintptr_t>(s) & 15u) == 0 && (n & 7) == 0) {
    for (int i = threadIdx.x; i < (n >> 3); i += 256) reinterpret_cast<uint4*>(slab)[i] = reinterpret_cast<const uint4*>(s)[i];
  } else {
    for (int i = threadIdx.x; i < n; i += 256) slab[i] = s[i];
  }
  __syncthreads();
  const int groups = min(span, Cp - c0) >> 3;  // 8-channel vectors in this tile
  for (int v = threadIdx.x; v < HW * groups; v += 256) {
    const int px = v / groups, cg = v - px * groups;
    uint16_t o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int ch = cg * 8 + j;
      o[j] = ch < nch ? slab[ch * HW + px] : uint16_t(0);
    }
    uint4 q;
    q.x = uint32_t(o[0]) | (uint32_t(o[1]) << 16);
    q.y = uint32_t(o[2]) | (uint32_t(o[3]) << 16);
    q.z = uint32_t(o[4]) | (uint32_t(o[5]) << 16);
    q.w = uint32_t(o[6]) | (uint32_t(o[7]) << 16);
    *reinterpret_cast<uint4*>(dst + (size_t(b) * HW + px) * Cp + c0 + cg * 8) = q;
  }
}

// One repack job: a whole tensor.  mode 0 = tiled with 2-byte loads, 1 = tiled with 128-bit loads, 2 = small-HW slab,
// 3 = tiled with 32-bit loads.
struct RepackJob {
  const uint16_t* src;
  uint16_t* dst;
  int C, HW, Cp, batch;
  int mode;
  int hw_tiles, c_tiles;
  int span;  // mode 2: channels per CTA
  unsigned blocks;  // hw_tiles * c_tiles * batch
  int prefetch;     // (read from the first job) L2 prefetch of the source lines before the dependency wait
  // mode 4 (pixel subsampling for strided 1x1 convolutions): HW = out_h * out_w pixels are taken from a source plane of
  // src_hw = h * w elements, destination pixel (p, q) from source pixel (p * sub_sh, q * sub_sw)
  int src_hw, src_w, sub_ow, sub_sh, sub_sw;
};

// The 128-byte lines one CTA is about to read, one prefetch per line, never outside the source tensor.
__device__ __forceinline__ void prefetch_source(const RepackJob& j, int hw_tile, int c_tile, int bi) {
  const int t = threadIdx.x;
  if (j.mode == 4) return;  // (a strided selection of the source: its lines are not one run per channel)
  if (j.mode == 2) {
    const int c0 = c_tile * j.span;
    const int nch = min(j.span, j.C - c0);
    if (nch <= 0) return;
    const uint8_t* s = reinterpret_cast<const uint8_t*>(j.src + (size_t(bi) * j.C + c0) * j.HW);
    const int bytes = nch * j.HW * 2;
    for (int o = t * 128; o < bytes + 127; o += 256 * 128) ptx::prefetch_l2(s + min(o, bytes - 1));
  } else if (t < 2 * kTile) {
    const int ch = c_tile * kTile + (t >> 1), px0 = hw_tile * kTile;
    if (ch < j.C && px0 < j.HW) {
      const uint8_t* row = reinterpret_cast<const uint8_t*>(j.src + (size_t(bi) * j.C + ch) * j.HW + px0);
      const int bytes = min(kTile, j.HW - px0) * 2;
      ptx::prefetch_l2(row + ((t & 1) ? bytes - 1 : 0));  // a 128-byte run touches at most two lines
    }
  }
}

// The tiled transpose over a strided selection of the source pixels: what a 1x1 convolution with stride > 1 and no padding
// reads.  Only those pixels are repacked ([B][out_h * out_w][Cp]); the convolution then runs as a stride-1 1x1 over the copy
// and the copy is stride_h * stride_w times smaller than the tensor.  2-byte loads (the selected pixels are not adjacent).
__device__ __forceinline__ void repack_tile_sub(uint32_t* tile, const RepackJob& j, int hw_tile, int c_tile, int b) {
  const int px0 = hw_tile * kTile, c0 = c_tile * kTile, t = threadIdx.x;
  uint16_t* tile16 = reinterpret_cast<uint16_t*>(tile);
  const int px = t & 63;
  const int dp = px0 + px;                       // destination pixel
  const int p = dp / j.sub_ow, q = dp - p * j.sub_ow;
  const uint16_t* s = j.src + (size_t(b) * j.C + c0) * j.src_hw + size_t(p * j.sub_sh) * j.src_w + q * j.sub_sw;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int ch = (t >> 6) + i * 4;
    uint16_t v = 0;
    if (c0 + ch < j.C && dp < j.HW) v = s[size_t(ch) * j.src_hw];
    tile16[ch * (kLdWords * 2) + px] = v;
  }
  __syncthreads();
  const int lane = t & 31, warp = t >> 5;
  const int cg = (warp & 1) * 4 + (lane & 3);
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int opx = ((warp >> 1) + it * 4) * 8 + (lane >> 2);
    if (px0 + opx < j.HW && c0 + cg * 8 < j.Cp) {
      uint16_t o[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = tile16[(cg * 8 + e) * (kLdWords * 2) + opx];
      uint4 v;
      v.x = uint32_t(o[0]) | (uint32_t(o[1]) << 16);
      v.y = uint32_t(o[2]) | (uint32_t(o[3]) << 16);
      v.z = uint32_t(o[4]) | (uint32_t(o[5]) << 16);
      v.w = uint32_t(o[6]) | (uint32_t(o[7]) << 16);
      *reinterpret_cast<uint4*>(j.dst + (size_t(b) * j.HW + px0 + opx) * j.Cp + c0 + cg * 8) = v;
    }
  }
}

// Up to two jobs in one launch (activations + weights): block indices [0, a.blocks) belong to job a, the rest to job b.
__global__ void __launch_bounds__(256) repack_jobs_kernel(const RepackJob a, const RepackJob b) {
  __shared__ __align__(16) uint32_t smem[kTile * kLdWords];  // 8448 B >= kTile * kSmallHwMax * 2 = 8192 B
  const bool first = blockIdx.x < a.blocks;
  const RepackJob& j = first ? a : b;
  unsigned id = first ? blockIdx.x : blockIdx.x - a.blocks;
  const int hw_tile = int(id % unsigned(j.hw_tiles));
  id /= unsigned(j.hw_tiles);
  const int c_tile = int(id % unsigned(j.c_tiles));
  const int bi = int(id / unsigned(j.c_tiles));
  // Launched with programmatic stream serialization, so this CTA may be resident well before the previous kernel of the
  // stream has finished.  Meanwhile it starts its source lines on their way from HBM into L2 (a cache fill at the
  // coherence point: harmless even if that kernel still writes them), so that the loads below hit L2.
  if (a.prefetch) prefetch_source(j, hw_tile, c_tile, bi);
  // Wait for the previous kernel (it may still read the destination or write the source), then let the convolution
  // kernel behind this one begin its set-up.
  ptx::grid_dep_wait();
  ptx::grid_dep_launch();
  if (j.mode == 4) repack_tile_sub(smem, j, hw_tile, c_tile, bi);
  else if (j.mode == 2) repack_small_hw(reinterpret_cast<uint16_t*>(smem), j.src, j.dst, j.C, j.HW, j.Cp, j.span, c_tile, bi);
  else if (j.mode == 1) repack_tile<1>(smem, j.src, j.dst, j.C, j.HW, j.Cp, hw_tile, c_tile, bi);
  else if (j.mode == 3) repack_tile<2>(smem, j.src, j.dst, j.C, j.HW, j.Cp, hw_tile, c_tile, bi);
  else repack_tile<0>(smem, j.src, j.dst, j.C, j.HW, j.Cp, hw_tile, c_tile, bi);
}

// ---- row gather for convolutions with very few input channels ------------------------------------------------------
// X2[n][h][q][s * C + c] = x[n][c][h][q * stride_w - pad_w + s]  (zero outside the image, zero-filled up to c2), and
// W2[o][r][s * C + c] = w[o][c][r][s].  A convolution with an R x S kernel over C channels becomes one with an R x 1
// kernel over c2 = round_up(S * C, 16) channels on a tensor of width Q: a 7x7 stem over 3 channels reduces over
// 7 slabs of 32 instead of 49 taps of 16 padded channels.  Pure data movement: bit-exact.
struct GatherJob {
  const uint16_t* x;
  uint16_t* x2;
  const uint16_t* w;  // null: activations only
  uint16_t* w2;
  int B, C, H, W, Q, S, R, O, stride_w, pad_w, c2;
  unsigned x_blocks;
  int64_t rows;       // B * H * Q
};

constexpr int kGatherRows = 128;  // output positions (consecutive q of one image row) per block

// Block = one (image, input row, chunk of kGatherRows output columns).  The C input-row segments the chunk touches are
// staged in shared memory with coalesced loads; each thread then assembles 16-byte output vectors from them through
// a small table (element e of a gathered row -> offset of its (channel, tap) in the staged strip).
__global__ void __launch_bounds__(256) gather_rows_kernel(const GatherJob j) {
  extern __shared__ __align__(16) uint8_t gsm[];
  ptx::grid_dep_wait();
  ptx::grid_dep_launch();
  if (blockIdx.x >= j.x_blocks) {  // weights: one thread per (o, r, e)
    const int64_t total = int64_t(j.O) * j.R * j.c2;
    for (int64_t i = int64_t(blockIdx.x - j.x_blocks) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x - j.x_blocks) * 256) {
      const int e = int(i % j.c2);
      const int64_t orr = i / j.c2;
      const int r = int(orr % j.R), o = int(orr / j.R);
      uint16_t v = 0;
      if (e < j.S * j.C) {
        const int s = e / j.C, c = e - s * j.C;
        v = j.w[((int64_t(o) * j.C + c) * j.R + r) * j.S + s];
      }
      j.w2[i] = v;
    }
    return;
  }
  const int chunks = (j.Q + kGatherRows - 1) / kGatherRows;
  const int chunk = int(blockIdx.x % unsigned(chunks));
  const unsigned nh = blockIdx.x / unsigned(chunks);
  const int h = int(nh % unsigned(j.H)), n = int(nh / unsigned(j.H));
  const int q0 = chunk * kGatherRows;
  const int nq = min(kGatherRows, j.Q - q0);
  const int strip_w = (kGatherRows - 1) * j.stride_w + j.S;  // input columns one chunk can touch
  const int w0 = q0 * j.stride_w - j.pad_w;                  // first of them (may be negative: zero padding)
  uint16_t* strip = reinterpret_cast<uint16_t*>(gsm);        // [C][strip_w]
  int* table = reinterpret_cast<int*>(gsm + ((size_t(j.C) * strip_w * 2 + 15) & ~size_t(15)));  // [c2], -1 = padding
  const uint16_t* xrow = j.x + (int64_t(n) * j.C * j.H + h) * j.W;
  const int64_t plane = int64_t(j.H) * j.W;
  for (int i = threadIdx.x; i < j.C * strip_w; i += 256) {
    const int c = i / strip_w, col = i - c * strip_w;
    const int wc = w0 + col;
    strip[i] = (wc >= 0 && wc < j.W) ? __ldg(xrow + c * plane + wc) : uint16_t(0);
  }
  for (int e = threadIdx.x; e < j.c2; e += 256) {
    const int s = e / j.C, c = e - s * j.C;
    table[e] = e < j.S * j.C ? c * strip_w + s : -1;
  }
  __syncthreads();
  const int vpr = j.c2 >> 3;  // 16-byte vectors per output position
  uint4* dst = reinterpret_cast<uint4*>(j.x2 + ((int64_t(n) * j.H + h) * j.Q + q0) * j.c2);
  for (int i = threadIdx.x; i < nq * vpr; i += 256) {
    const int rl = i / vpr, k = i - rl * vpr;
    const int base = rl * j.stride_w;
    uint16_t o[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
      const int off = table[k * 8 + t];
      o[t] = off >= 0 ? strip[off + base] : uint16_t(0);
    }
    uint4 v;
    v.x = uint32_t(o[0]) | (uint32_t(o[1]) << 16);
    v.y = uint32_t(o[2]) | (uint32_t(o[3]) << 16);
    v.z = uint32_t(o[4]) | (uint32_t(o[5]) << 16);
    v.w = uint32_t(o[6]) | (uint32_t(o[7]) << 16);
    dst[i] = v;
  }
}

// Whole-row variant for the common case (Q <= kGatherRows, W % 8 == 0, 16-byte aligned x, pad_w <= 8, c2 = 32 so that
// a thread keeps one 8-channel group): a block takes kFastRows consecutive input rows of one image.  The rows are read
// with 16-byte loads into shared memory at column offset 8 (zero margins stand in for the padding), every thread
// keeps the eight strip offsets of its channel group in registers, and the block's output
// X2[n][h0 .. h0+kFastRows)[0 .. Q)[c2] is one contiguous run written with 16-byte stores.
constexpr int kFastRows = 4;
__global__ void __launch_bounds__(256) gather_rows_fast_kernel(const GatherJob j, int sw) {
  extern __shared__ __align__(16) uint8_t gsm[];
  ptx::grid_dep_wait();
  ptx::grid_dep_launch();
  if (blockIdx.x >= j.x_blocks) {  // weights: one thread per (o, r, e)
    const int64_t total = int64_t(j.O) * j.R * j.c2;
    for (int64_t i = int64_t(blockIdx.x - j.x_blocks) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x - j.x_blocks) * 256) {
      const int e = int(i % j.c2);
      const int64_t orr = i / j.c2;
      const int r = int(orr % j.R), o = int(orr / j.R);
      uint16_t v = 0;
      if (e < j.S * j.C) {
        const int s = e / j.C, c = e - s * j.C;
        v = j.w[((int64_t(o) * j.C + c) * j.R + r) * j.S + s];
      }
      j.w2[i] = v;
    }
    return;
  }
  const int groups = (j.H + kFastRows - 1) / kFastRows;
  const int n = int(blockIdx.x / unsigned(groups));
  const int h0 = int(blockIdx.x % unsigned(groups)) * kFastRows;
  const int rows = min(kFastRows, j.H - h0);
  uint16_t* strip = reinterpret_cast<uint16_t*>(gsm);  // [rows][C][sw]; input column w sits at index 8 + w
  const int vec_w = j.W >> 3;
  const int64_t plane = int64_t(j.H) * j.W;
  const uint16_t* x0 = j.x + (int64_t(n) * j.C * j.H + h0) * j.W;
  for (int i = threadIdx.x; i < rows * j.C * vec_w; i += 256) {
    const int v = i % vec_w, rc = i / vec_w;
    const int c = rc % j.C, r = rc / j.C;
    const uint4 val = __ldg(reinterpret_cast<const uint4*>(x0 + c * plane + int64_t(r) * j.W) + v);
    *reinterpret_cast<uint4*>(strip + (r * j.C + c) * sw + 8 + v * 8) = val;
  }
  const int margin = sw - j.W;  // 8 leading zeros, the rest trailing
  for (int i = threadIdx.x; i < rows * j.C * margin; i += 256) {
    const int m = i % margin, rc = i / margin;
    strip[rc * sw + (m < 8 ? m : j.W + m)] = 0;
  }
  // this thread's channel group k = threadIdx.x % 4 never changes (256 % 4 == 0)
  const int k = threadIdx.x & 3;
  int off[8];
#pragma unroll
  for (int t = 0; t < 8; ++t) {
    const int e = k * 8 + t;
    const int s = e / j.C, c = e - s * j.C;
    off[t] = e < j.S * j.C ? c * sw + s + 8 - j.pad_w : -1;
  }
  __syncthreads();
  uint4* dst = reinterpret_cast<uint4*>(j.x2 + ((int64_t(n) * j.H + h0) * j.Q) * j.c2);
  const int per_row = j.Q * 4;
  for (int i = threadIdx.x; i < rows * per_row; i += 256) {
    const int r = i / per_row;
    const int rl = (i - r * per_row) >> 2;
    const uint16_t* sp = strip + r * j.C * sw + rl * j.stride_w;
    uint16_t o[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) o[t] = off[t] >= 0 ? sp[off[t]] : uint16_t(0);
    uint4 v;
    v.x = uint32_t(o[0]) | (uint32_t(o[1]) << 16);
    v.y = uint32_t(o[2]) | (uint32_t(o[3]) << 16);
    v.z = uint32_t(o[4]) | (uint32_t(o[5]) << 16);
    v.w = uint32_t(o[6]) | (uint32_t(o[7]) << 16);
    dst[i] = v;
  }
}

RepackJob make_job(const void* src, void* dst, int batch, int channels, int hw, int c_padded) {
  RepackJob j;
  j.src = static_cast<const uint16_t*>(src);
  j.dst = static_cast<uint16_t*>(dst);
  j.C = channels; j.HW = hw; j.Cp = c_padded; j.batch = batch;
  j.c_tiles = (c_padded + kTile - 1) / kTile;
  j.span = kTile;
  if (hw < 32 && hw <= kSmallHwMax) {
    j.mode = 2;
    j.hw_tiles = 1;
    j.span = (kTile * kSmallHwMax / hw) / kTile * kTile;  // as many 64-channel groups as the slab holds
    if (j.span > ((c_padded + kTile - 1) / kTile) * kTile) j.span = ((c_padded + kTile - 1) / kTile) * kTile;
    j.c_tiles = (c_padded + j.span - 1) / j.span;
  } else {
    j.mode = ((reinterpret_cast<uintptr_t>(src) & 15u) == 0 && (hw & 7) == 0) ? 1
             : (((reinterpret_cast<uintptr_t>(src) & 3u) == 0 && (hw & 1) == 0) ? 3 : 0);
    j.hw_tiles = (hw + kTile - 1) / kTile;
  }
  j.blocks = 0;
  j.prefetch = prefetch_enabled() ? 1 : 0;
  j.src_hw = hw; j.src_w = 0; j.sub_ow = 1; j.sub_sh = j.sub_sw = 0;
  return j;
}

}  // namespace

cudaError_t repack_pair_launch(const void* src_a, void* dst_a, int batch_a, int ch_a, int hw_a, int cp_a, const void* src_b,
                               void* dst_b, int batch_b, int ch_b, int hw_b, int cp_b, cudaStream_t stream) {
  RepackJob a = make_job(src_a, dst_a, batch_a, ch_a, hw_a, cp_a);
  RepackJob b = a;
  const int64_t na = int64_t(a.hw_tiles) * a.c_tiles * batch_a;
  int64_t nb = 0;
  if (src_b != nullptr) {
    b = make_job(src_b, dst_b, batch_b, ch_b, hw_b, cp_b);
    nb = int64_t(b.hw_tiles) * b.c_tiles * batch_b;
  }
  if (na + nb > 2147483647LL) return cudaErrorInvalidValue;
  a.blocks = unsigned(na);
  b.blocks = unsigned(nb);
  const cudaError_t e = launch_pdl(repack_jobs_kernel, dim3(unsigned(na + nb)), dim3(256), 0, stream, a, b);
  if (e != cudaSuccess) return e;
  return cudaGetLastError();
}

cudaError_t repack_subsampled_launch(const void* x, void* xn, int batch, int channels, int h, int w, int out_h, int out_w, int stride_h,
                                     int stride_w, int c_padded, const void* wsrc, void* wdst, int out_channels, cudaStream_t stream) {
  RepackJob a = make_job(x, xn, batch, channels, out_h * out_w, c_padded);
  a.mode = 4;
  a.hw_tiles = (out_h * out_w + kTile - 1) / kTile;
  a.c_tiles = (c_padded + kTile - 1) / kTile;
  a.span = kTile;
  a.src_hw = h * w; a.src_w = w; a.sub_ow = out_w; a.sub_sh = stride_h; a.sub_sw = stride_w;
  RepackJob b = a;
  const int64_t na = int64_t(a.hw_tiles) * a.c_tiles * batch;
  int64_t nb = 0;
  if (wsrc != nullptr) {  // the 1x1 filters: [O][C] -> [O][Cp]
    b = make_job(wsrc, wdst, out_channels, channels, 1, c_padded);
    nb = int64_t(b.hw_tiles) * b.c_tiles * out_channels;
  }
  if (na + nb > 2147483647LL) return cudaErrorInvalidValue;
  a.blocks = unsigned(na);
  b.blocks = unsigned(nb);
  const cudaError_t e = launch_pdl(repack_jobs_kernel, dim3(unsigned(na + nb)), dim3(256), 0, stream, a, b);
  if (e != cudaSuccess) return e;
  return cudaGetLastError();
}

// ---- column-pair gather: the row gather for stride_w = 2 and at most 4 channels, four times smaller --------------------
// X3[n][h][i][j * C + c] = x[n][c][h][2 * (i - left) + j], j = 0, 1 (8 values = 16 bytes per position i, zero where the
// column lies outside the image or C * 2 < 8).  The window of output column q (input columns 2q - pad .. 2q - pad + S - 1)
// is the T adjacent positions q .. q + T - 1, i.e. the T * 16 contiguous bytes at position q: the convolution's tensor
// map reads X3 with a pixel stride of ONE position (16 bytes) and T * 8 "channels" per pixel, so consecutive pixels overlap
// and nothing is stored twice.  W3[o][r][t * 8 + j * C + c] = w[o][c][r][2t + j - shift] (zero outside the kernel).
struct PairGatherJob {
  const uint16_t* x;   // null: weights only
  uint16_t* x3;
  const uint16_t* w;   // null: activations only
  uint16_t* w3;
  int B, C, H, W, R, S, O, positions, left, T, shift, words;  // words: x may be read as aligned 32-bit column pairs
  unsigned x_blocks;
};

namespace {
__global__ void __launch_bounds__(256) gather_pairs_kernel(const PairGatherJob j) {
  ptx::grid_dep_wait();
  ptx::grid_dep_launch();
  if (blockIdx.x >= j.x_blocks) {  // weights: one thread per (o, r, e)
    const int c2 = j.T * 8;
    const int64_t total = int64_t(j.O) * j.R * c2;
    for (int64_t i = int64_t(blockIdx.x - j.x_blocks) * 256 + threadIdx.x; i < total; i += int64_t(gridDim.x - j.x_blocks) * 256) {
      const int e = int(i % c2);
      const int64_t orr = i / c2;
      const int r = int(orr % j.R), o = int(orr / j.R);
      const int t = e >> 3, k = e & 7;
      uint16_t v = 0;
      if (k < 2 * j.C) {
        const int jj = k / j.C, c = k - jj * j.C;
        const int s = 2 * t + jj - j.shift;
        if (s >= 0 && s < j.S) v = j.w[((int64_t(o) * j.C + c) * j.R + r) * j.S + s];
      }
      j.w3[i] = v;
    }
    return;
  }
  const int64_t total = int64_t(j.B) * j.H * j.positions;
  const int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= total) return;
  const int pos = int(i % j.positions);
  const int64_t nh = i / j.positions;
  const int h = int(nh % j.H), n = int(nh / j.H);
  const int pp = pos - j.left;
  uint16_t v[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (pp >= 0 && 2 * pp < j.W) {
    const uint16_t* src = j.x + ((int64_t(n) * j.C) * j.H + h) * j.W + 2 * pp;
    for (int c = 0; c < j.C; ++c) {
      const uint16_t* p = src + int64_t(c) * j.H * j.W;
      if (j.words) {
        const uint32_t two = *reinterpret_cast<const uint32_t*>(p);
        v[c] = uint16_t(two & 0xffffu);
        v[j.C + c] = uint16_t(two >> 16);
      } else {
        v[c] = p[0];
        v[j.C + c] = p[1];
      }
    }
  }
  uint4 o;
  o.x = uint32_t(v[0]) | (uint32_t(v[1]) << 16);
  o.y = uint32_t(v[2]) | (uint32_t(v[3]) << 16);
  o.z = uint32_t(v[4]) | (uint32_t(v[5]) << 16);
  o.w = uint32_t(v[6]) | (uint32_t(v[7]) << 16);
  reinterpret_cast<uint4*>(j.x3)[i] = o;
}
}  // namespace

cudaError_t gather_pairs_launch(const void* x, void* x3, int batch, int channels, int h, int w, int positions, int left, int t_positions,
                                int shift, const void* wsrc, void* w3, int out_channels, int kernel_h, int kernel_w, cudaStream_t stream) {
  PairGatherJob j;
  j.x = static_cast<const uint16_t*>(x);
  j.x3 = static_cast<uint16_t*>(x3);
  j.w = static_cast<const uint16_t*>(wsrc);
  j.w3 = static_cast<uint16_t*>(w3);
  j.B = batch; j.C = channels; j.H = h; j.W = w; j.R = kernel_h; j.S = kernel_w; j.O = out_channels;
  j.positions = positions; j.left = left; j.T = t_positions; j.shift = shift;
  j.words = (reinterpret_cast<uintptr_t>(x) & 3u) == 0 ? 1 : 0;   // (w is even on this route)
  const int64_t xb = x != nullptr ? (int64_t(batch) * h * positions + 255) / 256 : 0;
  int64_t wb = 0;
  if (wsrc != nullptr) {
    wb = (int64_t(out_channels) * kernel_h * t_positions * 8 + 255) / 256;
    if (wb > 1024) wb = 1024;
  }
  if (xb + wb > 2147483647LL || xb + wb == 0) return cudaErrorInvalidValue;
  j.x_blocks = unsigned(xb);
  const cudaError_t e = launch_pdl(gather_pairs_kernel, dim3(unsigned(xb + wb)), dim3(256), 0, stream, j);
  if (e != cudaSuccess) return e;
  return cudaGetLastError();
}

cudaError_t gather_rows_launch(const void* x, void* x2, int batch, int channels, int h, int w, int q, int kernel_w, int stride_w,
                               int pad_w, int c2, const void* wsrc, void* w2, int out_channels, int kernel_h, cudaStream_t stream) {
  GatherJob j;
  j.x = static_cast<const uint16_t*>(x);
  j.x2 = static_cast<uint16_t*>(x2);
  j.w = static_cast<const uint16_t*>(wsrc);
  j.w2 = static_cast<uint16_t*>(w2);
  j.B = batch; j.C = channels; j.H = h; j.W = w; j.Q = q; j.S = kernel_w; j.R = kernel_h; j.O = out_channels;
  j.stride_w = stride_w; j.pad_w = pad_w; j.c2 = c2;
  j.rows = int64_t(batch) * h * q;
  const int chunks = (q + kGatherRows - 1) / kGatherRows;
  const int64_t xb = x != nullptr ? int64_t(batch) * h * chunks : 0;
  int64_t wb = 0;
  if (wsrc != nullptr) {
    wb = (int64_t(out_channels) * kernel_h * c2 + 255) / 256;
    if (wb > 1024) wb = 1024;
  }
  if (x != nullptr && q <= kGatherRows && (w & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && pad_w <= 8 && c2 == 32) {
    int need = (q - 1) * stride_w + kernel_w + 8 - pad_w;
    if (need < w + 16) need = w + 16;
    const int sw = (need + 7) & ~7;
    const size_t fast_smem = size_t(kFastRows) * channels * sw * 2;
    const int64_t fb = int64_t(batch) * ((h + kFastRows - 1) / kFastRows);
    if (fast_smem <= 48 * 1024 && fb + wb <= 2147483647LL) {
      j.x_blocks = unsigned(fb);
      const cudaError_t e = launch_pdl(gather_rows_fast_kernel, dim3(unsigned(fb + wb)), dim3(256), fast_smem, stream, j, sw);
      if (e != cudaSuccess) return e;
      return cudaGetLastError();
    }
  }
  if (xb + wb > 2147483647LL || xb + wb == 0) return cudaErrorInvalidValue;
  j.x_blocks = unsigned(xb);
  const int strip_w = (kGatherRows - 1) * stride_w + kernel_w;
  const size_t smem = ((size_t(channels) * strip_w * 2 + 15) & ~size_t(15)) + size_t(c2) * 4;
  if (smem > 48 * 1024) return cudaErrorInvalidValue;  // channels * (127 * stride + S) * 2 bytes: far below for S*C <= 64, stride <= 8
  const cudaError_t e = launch_pdl(gather_rows_kernel, dim3(unsigned(xb + wb)), dim3(256), smem, stream, j);
  if (e != cudaSuccess) return e;
  return cudaGetLastError();
}

namespace {

// FP32 [B][C][HW] -> [B][HW][Cp] with every value rounded to TF32 (round to nearest, ties away: cvt.rna, the rounding
// of round_to_tf32 in the reference, src/runtime/reference.cu:95-104), channels zero-padded to Cp.  32 x 32 tiles.
__global__ void __launch_bounds__(256) repack_tf32_kernel(const float* __restrict__ src, float* __restrict__ dst, int C, int HW, int Cp) {
  __shared__ float tile[32][33];
  ptx::grid_dep_wait();
  ptx::grid_dep_launch();
  const int b = blockIdx.z, c0 = blockIdx.y * 32, p0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 8 rows of 32 threads
  for (int r = ty; r < 32; r += 8) {
    const int c = c0 + r, px = p0 + tx;
    float v = 0.f;
    if (c < C && px < HW) {
      uint32_t u;
      asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(src[(size_t(b) * C + c) * HW + px]));
      v = __uint_as_float(u);
    }
    tile[r][tx] = v;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int px = p0 + r, c = c0 + tx;
    if (px < HW && c < Cp) dst[(size_t(b) * HW + px) * Cp + c] = tile[tx][r];
  }
}

// 1-byte elements (FP8 bit patterns): [B][C][HW] -> [B][HW][Cp], channels zero-padded to Cp (a multiple of 32).  Pure data
// movement, bit-exact.  Up to two tensors per launch (activations and weights), like repack_jobs_kernel, and the same
// two shapes of work:
//   tile mode: one CTA transposes a 64-channel x 64-pixel tile: 4-byte loads along the pixels where the plane size and the
//     source address allow it, 16-byte stores of 16 consecutive channels (a warp writes 8 pixels x 64 bytes);
//   slab mode (planes of at most 16 elements: filter taps): one CTA takes `span` channels of one batch entry; the source
//     slab [span][HW] is contiguous and is read linearly, then written as [HW][span].
// Both prefetch their source lines into L2 before the dependency wait (see repack_jobs_kernel).
struct ByteJob {
  const uint8_t* src;
  uint8_t* dst;
  int C, HW, Cp, hw_tiles, c_tiles, span;  // span > 0: slab mode
  unsigned blocks;
};
constexpr int kBytePitch = 68;
constexpr int kByteSlab = 8192;  // bytes of shared memory a slab may take

__global__ void __launch_bounds__(256) repack_bytes_kernel(const ByteJob a, const ByteJob b, int prefetch) {
  __shared__ __align__(16) uint8_t tile[kByteSlab];
  static_assert(64 * kBytePitch <= kByteSlab, "the tile mode's 64 x 64 tile must fit the slab buffer");
  const bool first = blockIdx.x < a.blocks;
  const ByteJob& j = first ? a : b;
  unsigned id = first ? blockIdx.x : blockIdx.x - a.blocks;
  const int hw_tile = int(id % unsigned(j.hw_tiles));
  id /= unsigned(j.hw_tiles);
  const int c_tile = int(id % unsigned(j.c_tiles));
  const int bi = int(id / unsigned(j.c_tiles));
  const int t = threadIdx.x;
  if (j.span > 0) {
    const int c0 = c_tile * j.span;
    const int nch = min(j.span, j.C - c0);           // may be <= 0 for pure padding tiles
    const int n = nch > 0 ? nch * j.HW : 0;
    const uint8_t* s = j.src + (size_t(bi) * j.C + c0) * j.HW;
    if (prefetch)
      for (int o = t * 128; o < n + 127 && n > 0; o += 256 * 128) ptx::prefetch_l2(s + min(o, n - 1));
    ptx::grid_dep_wait();
    ptx::grid_dep_launch();
    if ((reinterpret_cast<uintptr_t>(s) & 15u) == 0 && (n & 15) == 0) {
      for (int i = t; i < (n >> 4); i += 256) reinterpret_cast<uint4*>(tile)[i] = reinterpret_cast<const uint4*>(s)[i];
    } else {
      for (int i = t; i < n; i += 256) tile[i] = s[i];
    }
    __syncthreads();
    const int groups = min(j.span, j.Cp - c0) >> 4;  // 16-channel vectors in this tile
    for (int v = t; v < j.HW * groups; v += 256) {
      const int px = v / groups, cg = v - px * groups;
      uint32_t o[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int e = 0; e < 16; ++e) {
        const int ch = cg * 16 + e;
        if (ch < nch) o[e >> 2] |= uint32_t(tile[ch * j.HW + px]) << (8 * (e & 3));
      }
      *reinterpret_cast<uint4*>(j.dst + (size_t(bi) * j.HW + px) * j.Cp + c0 + cg * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    return;
  }
  const int c0 = c_tile * 64, px0 = hw_tile * 64;
  const uint8_t* s = j.src + (size_t(bi) * j.C + c0) * j.HW + px0;
  if (prefetch && t < 64 && c0 + t < j.C && px0 < j.HW) ptx::prefetch_l2(s + size_t(t) * j.HW);  // 64 bytes: one line, or the first of two
  ptx::grid_dep_wait();
  ptx::grid_dep_launch();
  const bool words = (j.HW & 3) == 0 && (reinterpret_cast<uintptr_t>(j.src) & 3u) == 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int idx = t + i * 256, ch = idx >> 4, q = (idx & 15) * 4;
    uint32_t v = 0;
    if (c0 + ch < j.C && px0 + q < j.HW) {
      const uint8_t* p = s + size_t(ch) * j.HW + q;
      if (words) v = *reinterpret_cast<const uint32_t*>(p);   // a group of four never straddles the plane (HW % 4 == 0)
      else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (px0 + q + e < j.HW) v |= uint32_t(p[e]) << (8 * e);
      }
    }
    *reinterpret_cast<uint32_t*>(tile + ch * kBytePitch + q) = v;
  }
  __syncthreads();
  const int cg = t & 3, px = t >> 2;
  if (px0 + px < j.HW && c0 + cg * 16 < j.Cp) {
    uint32_t o[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      uint32_t v = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) v |= uint32_t(tile[(cg * 16 + w * 4 + e) * kBytePitch + px]) << (8 * e);
      o[w] = v;
    }
    *reinterpret_cast<uint4*>(j.dst + (size_t(bi) * j.HW + px0 + px) * j.Cp + c0 + cg * 16) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

ByteJob make_byte_job(const void* src, void* dst, int batch, int channels, int hw, int c_padded) {
  ByteJob j;
  j.src = static_cast<const uint8_t*>(src);
  j.dst = static_cast<uint8_t*>(dst);
  j.C = channels; j.HW = hw; j.Cp = c_padded;
  if (hw <= 16) {   // filter taps: as many 64-channel groups per CTA as the slab holds
    j.span = (kByteSlab / hw) / 64 * 64;
    if (j.span > (c_padded + 63) / 64 * 64) j.span = (c_padded + 63) / 64 * 64;
    j.hw_tiles = 1;
    j.c_tiles = (c_padded + j.span - 1) / j.span;
  } else {
    j.span = 0;
    j.hw_tiles = (hw + 63) / 64;
    j.c_tiles = (c_padded + 63) / 64;
  }
  j.blocks = unsigned(int64_t(j.hw_tiles) * j.c_tiles * batch);
  return j;
}

}  // namespace

cudaError_t repack_bytes_pair_launch(const void* src_a, void* dst_a, int batch_a, int ch_a, int hw_a, int cp_a, const void* src_b,
                                     void* dst_b, int batch_b, int ch_b, int hw_b, int cp_b, cudaStream_t stream) {
  if (int64_t((hw_a + 63) / 64) * ((cp_a + 63) / 64) * batch_a + int64_t((hw_b + 63) / 64) * ((cp_b + 63) / 64) * batch_b > 2147483647LL)
    return cudaErrorInvalidValue;
  const ByteJob a = make_byte_job(src_a, dst_a, batch_a, ch_a, hw_a, cp_a);
  const ByteJob b = make_byte_job(src_b, dst_b, batch_b, ch_b, hw_b, cp_b);
  const cudaError_t e = launch_pdl(repack_bytes_kernel, dim3(a.blocks + b.blocks), dim3(256), 0, stream, a, b, prefetch_enabled() ? 1 : 0);
  if (e != cudaSuccess) return e;
  return cudaGetLastError();
}

cudaError_t repack_tf32_launch(const void* src, void* dst, int batch, int channels, int hw, int c_padded, cudaStream_t stream) {
  const dim3 grid(unsigned((hw + 31) / 32), unsigned((c_padded + 31) / 32), unsigned(batch));
  if (grid.y > 65535 || grid.z > 65535) return cudaErrorInvalidValue;
  const cudaError_t e = launch_pdl(repack_tf32_kernel, grid, dim3(256), 0, stream, static_cast<const float*>(src), static_cast<float*>(dst),
                                   channels, hw, c_padded);
  if (e != cudaSuccess) return e;
  return cudaGetLastError();
}

cudaError_t repack_launch(const void* src, void* dst, int batch, int channels, int hw, int c_padded, cudaStream_t stream) {
  return repack_pair_launch(src, dst, batch, channels, hw, c_padded, nullptr, nullptr, 0, 0, 0, 0, stream);
}

}  // namespace gieb
