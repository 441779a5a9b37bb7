// Elementwise operators around the convolution:
//  * bias_act: in-place y = act(y + bias[channel]) on NCHW -- stands in for bias_act_kernel
//    (src/kernels/elementwise.cu:13-23); the unfused comparator of the fusion tests.
//  * maxpool2d and add(+ReLU): glue of the ResNet-50-shaped chain.  The reference library has no such operators;
//    they follow the operator definitions (window maximum ignoring padding; float add, one rounding, optional ReLU).
// 16-bit tensors use 128-bit accesses when pointers and sizes allow, scalar accesses otherwise.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "internal.h"

namespace gieb {
namespace {

__device__ __forceinline__ float cvt(float v) { return v; }
__device__ __forceinline__ float cvt(__half v) { return __half2float(v); }
__device__ __forceinline__ float cvt(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T rnd(float v);
template <> __device__ __forceinline__ float rnd<float>(float v) { return v; }
template <> __device__ __forceinline__ __half rnd<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 rnd<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256)
bias_act_kernel(T* __restrict__ y, const T* __restrict__ bias, int64_t total, int channels, int hw, int relu) {
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
    float v = cvt(y[i]);
    if (bias != nullptr) v += cvt(bias[(i / hw) % channels]);
    if (relu) v = fmaxf(v, 0.f);
    y[i] = rnd<T>(v);
  }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
add_relu_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, int64_t n, int relu) {
  constexpr int W = 16 / sizeof(T);
  const int64_t step = int64_t(gridDim.x) * blockDim.x;
  const int64_t first = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  int64_t done = 0;
  if (VEC) {
    const int64_t nvec = n / W;
    for (int64_t v = first; v < nvec; v += step) {
      const uint4 ra = reinterpret_cast<const uint4*>(a)[v], rb = reinterpret_cast<const uint4*>(b)[v];
      T ta[W], tb[W];
      memcpy(ta, &ra, 16);
      memcpy(tb, &rb, 16);
#pragma unroll
      for (int j = 0; j < W; ++j) {
        T s = rnd<T>(cvt(ta[j]) + cvt(tb[j]));
        if (relu && cvt(s) < 0.f) s = rnd<T>(0.f);
        ta[j] = s;
      }
      uint4 o;
      memcpy(&o, ta, 16);
      reinterpret_cast<uint4*>(y)[v] = o;
    }
    done = nvec * W;
  }
  for (int64_t i = done + first; i < n; i += step) {
    T s = rnd<T>(cvt(a[i]) + cvt(b[i]));
    if (relu && cvt(s) < 0.f) s = rnd<T>(0.f);
    y[i] = s;
  }
}

// One thread per output position of a plane (32-bit index arithmetic only), grid.y strides over the B*C planes;
// consecutive threads walk ow, so window reads are coalesced along w and served from L1 across the 3 taps.
template <typename T>
__global__ void __launch_bounds__(256)
maxpool2d_kernel(const T* __restrict__ x, T* __restrict__ y, int planes, int h, int w, int oh, int ow, int k, int stride, int pad) {
  const int pos = blockIdx.x * blockDim.x + threadIdx.x;
  if (pos >= oh * ow) return;
  const int oy = pos / ow, ox = pos - oy * ow;
  const int iy0 = oy * stride - pad, ix0 = ox * stride - pad;
  const int r0 = iy0 < 0 ? -iy0 : 0, r1 = min(k, h - iy0);
  const int s0 = ix0 < 0 ? -ix0 : 0, s1 = min(k, w - ix0);
  for (int plane = blockIdx.y; plane < planes; plane += gridDim.y) {
    const T* xp = x + size_t(plane) * h * w + iy0 * w + ix0;
    float best = -INFINITY;
    for (int r = r0; r < r1; ++r)
      for (int s = s0; s < s1; ++s) best = fmaxf(best, cvt(xp[r * w + s]));
    y[size_t(plane) * oh * ow + pos] = rnd<T>(best);
  }
}

// 3x3 / stride 2 / pad 1 on 16-bit planes with an even width (the ResNet stem pool): output column ox needs input
// columns 2ox-1, 2ox, 2ox+1.  One aligned 32-bit load fetches (2ox, 2ox+1); column 2ox-1 is the upper half of the left
// neighbour's word, taken with a warp shuffle (lane 0 of a warp loads it itself).  Three loads per output instead of nine.
template <typename T2>
__global__ void __launch_bounds__(256)
maxpool_3x3s2p1_kernel(const uint32_t* __restrict__ x, uint16_t* __restrict__ y, int planes, int h, int w2, int oh, int ow) {
  const int ox = blockIdx.x * blockDim.x + threadIdx.x;  // one thread per output column, consecutive in a warp
  const int oy = blockIdx.y;
  const int lane = threadIdx.x & 31;
  const bool live = ox < ow;
  const int cx = live ? ox : ow - 1;  // dead lanes shadow the last column so that shuffles stay defined
  for (int plane = blockIdx.z; plane < planes; plane += gridDim.z) {
    const uint32_t* xp = x + size_t(plane) * h * w2;
    T2 best = T2();
    bool first = true;
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      const int iy = 2 * oy - 1 + r;
      if (iy < 0 || iy >= h) continue;  // block-uniform (oy is per block)
      const uint32_t word = xp[size_t(iy) * w2 + cx];  // columns 2cx, 2cx+1 (2cx+1 < w: w is even, cx < ow = w/2)
      uint32_t left = __shfl_up_sync(0xffffffffu, word, 1);
      if (lane == 0) left = cx > 0 ? xp[size_t(iy) * w2 + cx - 1] : 0u;
      const T2 cur = *reinterpret_cast<const T2*>(&word);
      T2 m = __hmax2(cur, T2(cur.y, cur.y));            // max(col 2cx, col 2cx+1) in .x
      if (cx > 0) {
        const T2 lf = *reinterpret_cast<const T2*>(&left);
        m = __hmax2(m, T2(lf.y, lf.y));                  // col 2cx-1
      }
      best = first ? m : __hmax2(best, m);
      first = false;
    }
    if (live) y[(size_t(plane) * oh + oy) * ow + ox] = *reinterpret_cast<const uint16_t*>(&best.x);
  }
}

// The same pool for widths that are multiples of 4 (8-byte aligned rows): one WARP walks down one plane (or one 128-column
// strip of it).  A lane owns output columns 2l, 2l+1 = input columns 4l-1 .. 4l+3: one 8-byte load per input row plus the
// left neighbour's last column by shuffle; the horizontal maxima of a row are computed once and serve the two output rows
// that contain it, so every input element is read once.  Rows are fetched eight at a time (eight loads in flight per lane).
template <typename T2>
__global__ void __launch_bounds__(256)
maxpool_3x3s2p1_rows_kernel(const uint2* __restrict__ x, uint32_t* __restrict__ y, int planes, int h, int w4, int oh, int ow2, int strips,
                            int bands, int band_rows) {
  const int lane = threadIdx.x & 31;
  const int64_t job = int64_t(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);  // (plane, strip)
  if (job >= int64_t(planes) * strips * bands) return;  // whole warps leave together
  // few planes: a plane is cut into `bands` bands of band_rows output rows (a multiple of 4), one warp each
  const int band = int(job % bands);
  const int64_t ps = job / bands;
  const int plane = int(ps / strips), strip = int(ps - int64_t(plane) * strips);
  const int oy_begin = band * band_rows, oy_end = min(oh, oy_begin + band_rows);
  const int c = strip * 32 + lane;               // this lane's 4-column group
  const bool live = c < w4;
  const int cc = live ? c : w4 - 1;              // dead lanes shadow the last group so that shuffles stay defined
  const uint2* xp = x + size_t(plane) * h * w4 + cc;
  uint32_t* yp = y + size_t(plane) * oh * ow2 + cc;
  T2 carry = T2();     // horizontal maxima of input row 2*oy - 1 (the row above the window's middle); unused while have_carry is false
  bool have_carry = false;
  if (oy_begin > 0) {  // the row above this band's first window row
    const size_t ro = size_t(2 * oy_begin - 1) * w4;
    const uint2 v0 = xp[ro];
    uint32_t l0 = __shfl_up_sync(0xffffffffu, v0.y, 1);
    if (lane == 0 && cc > 0) l0 = xp[ro - 1].y;
    const T2 a = *reinterpret_cast<const T2*>(&v0.x), b = *reinterpret_cast<const T2*>(&v0.y);
    const T2 l = *reinterpret_cast<const T2*>(&l0);
    carry = __hmax2(__hmax2(a, T2(a.y, b.x)), T2(cc > 0 ? l.y : a.x, b.y));
    have_carry = true;
  }
  for (int oy0 = oy_begin; oy0 < oy_end; oy0 += 4) {
    // rows 2*oy0 .. 2*oy0 + 7 (eight rows = four output rows), all loads first
    uint2 v[8];
    uint32_t lf[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int iy = 2 * oy0 + r;
      v[r] = iy < h ? xp[size_t(iy) * w4] : make_uint2(0u, 0u);
    }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      lf[r] = __shfl_up_sync(0xffffffffu, v[r].y, 1);
      const int iy = 2 * oy0 + r;
      if (lane == 0 && cc > 0 && iy < h) lf[r] = xp[size_t(iy) * w4 - 1].y;
    }
    T2 hm[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const T2 a = *reinterpret_cast<const T2*>(&v[r].x), b = *reinterpret_cast<const T2*>(&v[r].y);
      const T2 l = *reinterpret_cast<const T2*>(&lf[r]);
      T2 m = __hmax2(a, T2(a.y, b.x));
      hm[r] = __hmax2(m, T2(cc > 0 ? l.y : a.x, b.y));
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int oy = oy0 + k;
      if (oy >= oy_end) break;
      T2 m = hm[2 * k];                                   // row 2*oy (always inside: oy < oh = h / 2)
      if (2 * oy + 1 < h) m = __hmax2(m, hm[2 * k + 1]);  // row 2*oy + 1
      if (have_carry) m = __hmax2(m, carry);              // row 2*oy - 1
      carry = hm[2 * k + 1];
      have_carry = true;
      if (live) yp[size_t(oy) * ow2] = *reinterpret_cast<const uint32_t*>(&m);
    }
  }
}

// Channel-contiguous variant ([B][H][W][C], C % 8 == 0, 16-bit types): one thread per (output pixel, group of 8
// channels); consecutive threads take consecutive groups, so every window tap is a coalesced 16-byte load.
template <typename T2>
__global__ void __launch_bounds__(256)
maxpool2d_nhwc_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int64_t total, int c8, int h, int w, int oh, int ow, int k,
                      int stride, int pad) {
  const int64_t step = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += step) {
    const int g = int(i % c8);
    int64_t px = i / c8;
    const int ox = int(px % ow);
    px /= ow;
    const int oy = int(px % oh);
    const int b = int(px / oh);
    const int iy0 = oy * stride - pad, ix0 = ox * stride - pad;
    const int r0 = iy0 < 0 ? -iy0 : 0, r1 = min(k, h - iy0);
    const int s0 = ix0 < 0 ? -ix0 : 0, s1 = min(k, w - ix0);
    bool first = true;
    uint4 best = make_uint4(0, 0, 0, 0);
    for (int r = r0; r < r1; ++r)
      for (int s = s0; s < s1; ++s) {
        const uint4 v = x[((int64_t(b) * h + iy0 + r) * w + ix0 + s) * c8 + g];
        if (first) {
          best = v;
          first = false;
        } else {
          T2* bp = reinterpret_cast<T2*>(&best);
          const T2* vp = reinterpret_cast<const T2*>(&v);
#pragma unroll
          for (int q = 0; q < 4; ++q) bp[q] = __hmax2(bp[q], vp[q]);
        }
      }
    y[i] = best;
  }
}

unsigned grid_for(int64_t work) {
  int64_t b = (work + 255) / 256;
  if (b > kNumSms * 32) b = kNumSms * 32;
  return unsigned(b < 1 ? 1 : b);
}

}  // namespace

cudaError_t bias_act_launch(int precision, int64_t total, int channels, int hw, const void* bias, int relu, void* y,
                            cudaStream_t st) {
  const unsigned g = grid_for(total);
  switch (precision) {
    case 0: bias_act_kernel<float><<<g, 256, 0, st>>>(static_cast<float*>(y), static_cast<const float*>(bias), total, channels, hw, relu); break;
    case 1: bias_act_kernel<__half><<<g, 256, 0, st>>>(static_cast<__half*>(y), static_cast<const __half*>(bias), total, channels, hw, relu); break;
    case 2: bias_act_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<__nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(bias), total, channels, hw, relu); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

template <typename T>
static cudaError_t add_relu_t(int relu, const void* a, const void* b, void* y, int64_t n, cudaStream_t st) {
  const bool vec = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0;
  const unsigned g = grid_for(vec ? n / (16 / sizeof(T)) + 1 : n);
  if (vec) add_relu_kernel<T, true><<<g, 256, 0, st>>>(static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(y), n, relu);
  else add_relu_kernel<T, false><<<g, 256, 0, st>>>(static_cast<const T*>(a), static_cast<const T*>(b), static_cast<T*>(y), n, relu);
  return cudaGetLastError();
}

cudaError_t add_relu_launch(int precision, int relu, const void* a, const void* b, void* y, int64_t n, cudaStream_t st) {
  switch (precision) {
    case 0: return add_relu_t<float>(relu, a, b, y, n, st);
    case 1: return add_relu_t<__half>(relu, a, b, y, n, st);
    case 2: return add_relu_t<__nv_bfloat16>(relu, a, b, y, n, st);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t maxpool2d_launch(int precision, int batch, int channels, int h, int w, int k, int stride, int pad, const void* x,
                             void* y, cudaStream_t st) {
  const int oh = (h + 2 * pad - k) / stride + 1, ow = (w + 2 * pad - k) / stride + 1;
  const int64_t planes64 = int64_t(batch) * channels;
  if (planes64 > 2147483647LL || int64_t(oh) * ow > 2147483647LL) return cudaErrorInvalidValue;
  const int planes = int(planes64);
  if ((precision == 1 || precision == 2) && k == 3 && stride == 2 && pad == 1 && (w & 3) == 0 && (h & 1) == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 7u) == 0 && (reinterpret_cast<uintptr_t>(y) & 3u) == 0) {
    const int w4 = w / 4, strips = (w4 + 31) / 32;
    // enough warps for every SM (about 32 each): planes x column strips, and bands of output rows when that is too few
    int bands = int((int64_t(kNumSms) * 32 + int64_t(planes) * strips - 1) / (int64_t(planes) * strips));
    const int max_bands = (oh + 3) / 4;
    if (bands > max_bands) bands = max_bands;
    if (bands < 1) bands = 1;
    const int band_rows = ((oh + bands - 1) / bands + 3) / 4 * 4;
    bands = (oh + band_rows - 1) / band_rows;
    const int64_t jobs = int64_t(planes) * strips * bands;
    const unsigned blocks = unsigned((jobs + 7) / 8);
    if (precision == 1)
      maxpool_3x3s2p1_rows_kernel<__half2><<<blocks, 256, 0, st>>>(static_cast<const uint2*>(x), static_cast<uint32_t*>(y), planes, h, w4, oh, ow / 2, strips, bands, band_rows);
    else
      maxpool_3x3s2p1_rows_kernel<__nv_bfloat162><<<blocks, 256, 0, st>>>(static_cast<const uint2*>(x), static_cast<uint32_t*>(y), planes, h, w4, oh, ow / 2, strips, bands, band_rows);
    return cudaGetLastError();
  }
  if ((precision == 1 || precision == 2) && k == 3 && stride == 2 && pad == 1 && (w & 1) == 0 && (h & 1) == 0 &&
      (reinterpret_cast<uintptr_t>(x) & 3u) == 0 && oh <= 65535) {
    const dim3 g3(unsigned((ow + 255) / 256), unsigned(oh), unsigned(planes < 4096 ? planes : 4096));
    const dim3 b3(unsigned(ow < 256 ? ((ow + 31) / 32) * 32 : 256));
    if (precision == 1)
      maxpool_3x3s2p1_kernel<__half2><<<g3, b3, 0, st>>>(static_cast<const uint32_t*>(x), static_cast<uint16_t*>(y), planes, h, w / 2, oh, ow);
    else
      maxpool_3x3s2p1_kernel<__nv_bfloat162><<<g3, b3, 0, st>>>(static_cast<const uint32_t*>(x), static_cast<uint16_t*>(y), planes, h, w / 2, oh, ow);
    return cudaGetLastError();
  }
  const dim3 g(unsigned((oh * ow + 255) / 256), unsigned(planes < 32768 ? planes : 32768));
  switch (precision) {
    case 0: maxpool2d_kernel<float><<<g, 256, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(y), planes, h, w, oh, ow, k, stride, pad); break;
    case 1: maxpool2d_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half*>(x), static_cast<__half*>(y), planes, h, w, oh, ow, k, stride, pad); break;
    case 2: maxpool2d_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), planes, h, w, oh, ow, k, stride, pad); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t maxpool2d_nhwc_launch(int precision, int batch, int channels, int h, int w, int k, int stride, int pad, const void* x,
                                  void* y, cudaStream_t st) {
  const int oh = (h + 2 * pad - k) / stride + 1, ow = (w + 2 * pad - k) / stride + 1;
  if (channels % 8 != 0 || (precision != 1 && precision != 2)) return cudaErrorInvalidValue;
  const int c8 = channels / 8;
  const int64_t total = int64_t(batch) * oh * ow * c8;
  const unsigned g = grid_for(total);
  if (precision == 1)
    maxpool2d_nhwc_kernel<__half2><<<g, 256, 0, st>>>(static_cast<const uint4*>(x), static_cast<uint4*>(y), total, c8, h, w, oh, ow, k, stride, pad);
  else
    maxpool2d_nhwc_kernel<__nv_bfloat162><<<g, 256, 0, st>>>(static_cast<const uint4*>(x), static_cast<uint4*>(y), total, c8, h, w, oh, ow, k, stride, pad);
  return cudaGetLastError();
}

}  // namespace gieb
