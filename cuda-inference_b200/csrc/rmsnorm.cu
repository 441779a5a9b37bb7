// Fused RMSNorm and residual-add + RMSNorm.  Stands in for rmsnorm_kernel (src/transformer/rmsnorm.cu:39-98):
//   s = x                       (plain)      or   s = round_T(x + residual_in), residual_out = s   (fused)
//   y = round_T( s * rsqrt(mean(s^2) + eps) * gamma )
// FP32 arithmetic, one rounding per stored value; the residual stream is rounded to T BEFORE the square sum, as in
// the reference (rmsnorm.cu:57-66).
//
// Fast path (hidden % VEC == 0, all pointers 16-byte aligned, row fits 8 vectors x 1024 threads): one CTA per row,
// 128-bit loads issued up front, the row stays in registers across the block reduction, so every byte crosses
// HBM exactly once (x, residual in; residual, y out).  Anything else takes the scalar two-pass path.
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

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nw = (blockDim.x + 31) >> 5;
  if (nw == 1) return v;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float r = lane < nw ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  return r;
}

template <typename T> struct Vec { static constexpr int N = 16 / sizeof(T); };

// gamma vector i (VEC elements) as floats, from either T or float storage.
template <typename T, bool GAMMA_F32>
__device__ __forceinline__ void load_gamma(const void* gamma, int i, float (&g)[Vec<T>::N]) {
  constexpr int VEC = Vec<T>::N;
  if (GAMMA_F32) {
    const float4* gp = reinterpret_cast<const float4*>(gamma) + size_t(i) * (VEC / 4);
#pragma unroll
    for (int q = 0; q < VEC / 4; ++q) {
      const float4 f = __ldg(gp + q);
      g[q * 4 + 0] = f.x; g[q * 4 + 1] = f.y; g[q * 4 + 2] = f.z; g[q * 4 + 3] = f.w;
    }
  } else {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(gamma) + i);
    T tv[VEC];
    memcpy(tv, &raw, 16);
#pragma unroll
    for (int j = 0; j < VEC; ++j) g[j] = cvt(tv[j]);
  }
}

template <typename T, bool FUSED, bool GAMMA_F32, int NV>
__global__ void __launch_bounds__(NV == 8 ? 1024 : 256)
rmsnorm_row_kernel(const T* x, const void* __restrict__ gamma, T* __restrict__ y, const T* res_in,
                   T* res_out, int hidden, float eps) {
  constexpr int VEC = Vec<T>::N;
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const int nvec = hidden / VEC;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * hidden);
  const uint4* rr = FUSED ? reinterpret_cast<const uint4*>(res_in + row * hidden) : nullptr;

  uint4 xv[NV], rv[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      xv[k] = xr[i];  // plain loads: res_out may alias x
      if (FUSED) rv[k] = rr[i];
    }
  }
  float s[NV][VEC];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      T a[VEC];
      memcpy(a, &xv[k], 16);
      if (FUSED) {
        T b[VEC];
        memcpy(b, &rv[k], 16);
#pragma unroll
        for (int j = 0; j < VEC; ++j) a[j] = rnd<T>(cvt(a[j]) + cvt(b[j]));
        uint4 o;
        memcpy(&o, a, 16);
        reinterpret_cast<uint4*>(res_out + row * hidden)[i] = o;
      }
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        s[k][j] = cvt(a[j]);
        ss = fmaf(s[k][j], s[k][j], ss);
      }
    }
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / float(hidden) + eps);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      float g[VEC];
      load_gamma<T, GAMMA_F32>(gamma, i, g);
      T o[VEC];
#pragma unroll
      for (int j = 0; j < VEC; ++j) o[j] = rnd<T>(s[k][j] * inv * g[j]);
      uint4 ov;
      memcpy(&ov, o, 16);
      reinterpret_cast<uint4*>(y + row * hidden)[i] = ov;
    }
  }
}

// Scalar two-pass path for odd hidden sizes, misaligned pointers and very long rows.
template <typename T, bool FUSED, bool GAMMA_F32>
__global__ void __launch_bounds__(1024)
rmsnorm_generic_kernel(const T* x, const void* __restrict__ gamma, T* __restrict__ y, const T* res_in,
                       T* res_out, int hidden, float eps) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const T* xr = x + row * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float f = cvt(xr[i]);
    if (FUSED) {
      const T sv = rnd<T>(f + cvt(res_in[row * hidden + i]));
      res_out[row * hidden + i] = sv;
      f = cvt(sv);
    }
    ss = fmaf(f, f, ss);
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / float(hidden) + eps);
  const T* src = FUSED ? res_out + row * hidden : xr;  // each thread re-reads only what it wrote itself
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float g = GAMMA_F32 ? static_cast<const float*>(gamma)[i] : cvt(static_cast<const T*>(gamma)[i]);
    y[row * hidden + i] = rnd<T>(cvt(src[i]) * inv * g);
  }
}

bool aligned16(const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T, bool FUSED, bool GAMMA_F32>
cudaError_t run(int rows, int hidden, float eps, const void* x, const void* gamma, void* y, const void* rin, void* rout,
                cudaStream_t st) {
  constexpr int VEC = Vec<T>::N;
  const T* xp = static_cast<const T*>(x);
  T* yp = static_cast<T*>(y);
  const T* ri = static_cast<const T*>(rin);
  T* ro = static_cast<T*>(rout);
  const bool fast = hidden % VEC == 0 && hidden / VEC <= 8 * 1024 && aligned16(x) && aligned16(gamma) && aligned16(y) &&
                    aligned16(rin) && aligned16(rout);
  if (fast) {
    const int nvec = hidden / VEC;
    int nv = 1;
    while (nv < 8 && (nvec + nv - 1) / nv > 256) nv <<= 1;   // prefer <= 256 threads, up to 8 vectors each
    int threads = (nvec + nv - 1) / nv;
    threads = (threads + 31) & ~31;
    if (threads > 1024) threads = 1024;
    switch (nv) {
      case 1: rmsnorm_row_kernel<T, FUSED, GAMMA_F32, 1><<<rows, threads, 0, st>>>(xp, gamma, yp, ri, ro, hidden, eps); break;
      case 2: rmsnorm_row_kernel<T, FUSED, GAMMA_F32, 2><<<rows, threads, 0, st>>>(xp, gamma, yp, ri, ro, hidden, eps); break;
      case 4: rmsnorm_row_kernel<T, FUSED, GAMMA_F32, 4><<<rows, threads, 0, st>>>(xp, gamma, yp, ri, ro, hidden, eps); break;
      default: rmsnorm_row_kernel<T, FUSED, GAMMA_F32, 8><<<rows, threads, 0, st>>>(xp, gamma, yp, ri, ro, hidden, eps); break;
    }
  } else {
    int threads = 32;
    while (threads < hidden && threads < 1024) threads <<= 1;
    rmsnorm_generic_kernel<T, FUSED, GAMMA_F32><<<rows, threads, 0, st>>>(xp, gamma, yp, ri, ro, hidden, eps);
  }
  return cudaGetLastError();
}

template <typename T>
cudaError_t run_t(int rows, int hidden, float eps, int gamma_fp32, const void* x, const void* gamma, void* y, const void* rin,
                  void* rout, cudaStream_t st) {
  const bool fused = rin != nullptr && rout != nullptr;
  if (fused) return gamma_fp32 ? run<T, true, true>(rows, hidden, eps, x, gamma, y, rin, rout, st)
                               : run<T, true, false>(rows, hidden, eps, x, gamma, y, rin, rout, st);
  return gamma_fp32 ? run<T, false, true>(rows, hidden, eps, x, gamma, y, rin, rout, st)
                    : run<T, false, false>(rows, hidden, eps, x, gamma, y, rin, rout, st);
}

}  // namespace

cudaError_t rmsnorm_launch(int rows, int hidden, float eps, int dtype, int gamma_fp32, const void* x, const void* gamma,
                           void* y, const void* res_in, void* res_out, cudaStream_t stream) {
  switch (dtype) {
    case 0: return run_t<float>(rows, hidden, eps, 1, x, gamma, y, res_in, res_out, stream);
    case 1: return run_t<__half>(rows, hidden, eps, gamma_fp32, x, gamma, y, res_in, res_out, stream);
    case 2: return run_t<__nv_bfloat16>(rows, hidden, eps, gamma_fp32, x, gamma, y, res_in, res_out, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace gieb
