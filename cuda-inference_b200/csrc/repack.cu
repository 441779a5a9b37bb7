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

namespace gieb {
namespace {

constexpr int kTile = 64;          // channels and pixels per CTA tile
constexpr int kLdWords = 33;       // 32-bit words per shared-memory row (64 px + 1 word of padding)

// Tiled transpose, 256 threads. grid = (ceil(HW/64), ceil(Cp/64), B).
template <bool VEC_LOAD>
__global__ void __launch_bounds__(256)
repack_tiled_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, int C, int HW, int Cp) {
  __shared__ uint32_t tile[kTile * kLdWords];  // [channel][pixel pair]
  const int px0 = blockIdx.x * kTile;
  const int c0 = blockIdx.y * kTile;
  const int b = blockIdx.z;
  const uint16_t* s = src + (size_t(b) * C + c0) * HW + px0;
  const int t = threadIdx.x;

  if (VEC_LOAD) {
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

// Small-HW variant (filter taps: HW = R*S <= 256).  One CTA handles 64 channels of one batch entry: the source
// slab [64][HW] is contiguous, so it is read linearly, then written as [HW][64].
constexpr int kSmallHwMax = 256;
__global__ void __launch_bounds__(256)
repack_small_hw_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, int C, int HW, int Cp) {
  __shared__ uint16_t slab[kTile * kSmallHwMax];
  const int c0 = blockIdx.x * kTile;
  const int b = blockIdx.y;
  const int nch = min(kTile, C - c0);  // may be <= 0 for pure padding tiles
  const int n = nch > 0 ? nch * HW : 0;
  const uint16_t* s = src + (size_t(b) * C + c0) * HW;
  for (int i = threadIdx.x; i < n; i += 256) slab[i] = s[i];
  __syncthreads();
  const int groups = min(kTile, Cp - c0) >> 3;  // 8-channel vectors in this tile
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

}  // namespace

cudaError_t repack_launch(const void* src, void* dst, int batch, int channels, int hw, int c_padded, cudaStream_t stream) {
  const auto* s = static_cast<const uint16_t*>(src);
  auto* d = static_cast<uint16_t*>(dst);
  const int ctiles = (c_padded + kTile - 1) / kTile;
  if (hw < 32 && hw <= kSmallHwMax && batch <= 65535) {
    repack_small_hw_kernel<<<dim3(unsigned(ctiles), unsigned(batch)), 256, 0, stream>>>(s, d, channels, hw, c_padded);
    return cudaGetLastError();
  }
  // grid.z carries the batch: chunk it to stay inside the 65535 limit.
  const bool vec = (reinterpret_cast<uintptr_t>(src) & 15u) == 0 && (hw & 7) == 0;
  for (int b0 = 0; b0 < batch; b0 += 65535) {
    const int nb = batch - b0 < 65535 ? batch - b0 : 65535;
    dim3 grid(unsigned((hw + kTile - 1) / kTile), unsigned(ctiles), unsigned(nb));
    const uint16_t* sb = s + size_t(b0) * channels * hw;
    uint16_t* db = d + size_t(b0) * hw * c_padded;
    if (vec) repack_tiled_kernel<true><<<grid, 256, 0, stream>>>(sb, db, channels, hw, c_padded);
    else repack_tiled_kernel<false><<<grid, 256, 0, stream>>>(sb, db, channels, hw, c_padded);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  return cudaSuccess;
}

}  // namespace gieb
