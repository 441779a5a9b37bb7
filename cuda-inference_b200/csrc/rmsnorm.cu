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

#include <cooperative_groups.h>
#include <cooperative_groups/reduce.h>

#include "internal.h"

namespace cg = cooperative_groups;

namespace gieb {
namespace {

// Storage type <-> FP32 (one rounding on the way back).
template <typename T> struct Num;
template <> struct Num<float> {
  static __device__ __forceinline__ float up(float v) { return v; }
  static __device__ __forceinline__ float down(float v) { return v; }
};
template <> struct Num<__half> {
  static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half down(float v) { return __float2half_rn(v); }
};
template <> struct Num<__nv_bfloat16> {
  static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 down(float v) { return __float2bfloat16_rn(v); }
};

// Sum over the CTA, the same bits in every thread: each warp reduces its own values, warp leaders publish one partial
// each, and after ONE barrier every thread folds the (at most 32) partials itself in warp order.
__device__ __forceinline__ float cta_sum(float v, float* partial) {
  const cg::thread_block_tile<32> warp = cg::tiled_partition<32>(cg::this_thread_block());
  v = cg::reduce(warp, v, cg::plus<float>());
  if (warp.meta_group_size() == 1) return v;
  if (warp.thread_rank() == 0) partial[warp.meta_group_rank()] = v;
  __syncthreads();
  float total = 0.f;
  for (unsigned w = 0; w < warp.meta_group_size(); ++w) total += partial[w];
  return total;
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
    for (int j = 0; j < VEC; ++j) g[j] = Num<T>::up(tv[j]);
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
        for (int j = 0; j < VEC; ++j) a[j] = Num<T>::down(Num<T>::up(a[j]) + Num<T>::up(b[j]));
        uint4 o;
        memcpy(&o, a, 16);
        reinterpret_cast<uint4*>(res_out + row * hidden)[i] = o;
      }
#pragma unroll
      for (int j = 0; j < VEC; ++j) {
        s[k][j] = Num<T>::up(a[j]);
        ss = fmaf(s[k][j], s[k][j], ss);
      }
    }
  }
  ss = cta_sum(ss, red);
  const float inv = rsqrtf(ss / float(hidden) + eps);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int i = threadIdx.x + k * blockDim.x;
    if (i < nvec) {
      float g[VEC];
      load_gamma<T, GAMMA_F32>(gamma, i, g);
      T o[VEC];
#pragma unroll
      for (int j = 0; j < VEC; ++j) o[j] = Num<T>::down(s[k][j] * inv * g[j]);
      uint4 ov;
      memcpy(&ov, o, 16);
      reinterpret_cast<uint4*>(y + row * hidden)[i] = ov;
    }
  }
}

// Element-wise path for odd hidden sizes, misaligned pointers and very long rows.  The normalised stream (x, or the rounded
// x + residual) is kept as FP32 in shared memory between the square sum and the scaling when the row fits (`staged` floats
// of dynamic shared memory, 0 = it does not): global memory is then read once here as well; longer rows are read again.
template <typename T, bool FUSED, bool GAMMA_F32>
__global__ void __launch_bounds__(1024)
rmsnorm_generic_kernel(const T* x, const void* __restrict__ gamma, T* __restrict__ y, const T* res_in,
                       T* res_out, int hidden, float eps, int staged) {
  extern __shared__ float row_f32[];
  __shared__ float red[32];
  const size_t base = size_t(blockIdx.x) * hidden;
  auto stream_value = [&](int i) {   // element i of the stream that is normalised (stores the residual stream when fused)
    float f = Num<T>::up(x[base + i]);
    if (FUSED) {
      const T sv = Num<T>::down(f + Num<T>::up(res_in[base + i]));
      res_out[base + i] = sv;
      f = Num<T>::up(sv);
    }
    return f;
  };
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float f = stream_value(i);
    if (i < staged) row_f32[i] = f;
    ss = fmaf(f, f, ss);
  }
  ss = cta_sum(ss, red);
  const float inv = rsqrtf(ss / float(hidden) + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    // beyond the staged part a thread reads back what it stored itself (res_out) or the input again
    const float f = i < staged ? row_f32[i] : Num<T>::up(FUSED ? res_out[base + i] : x[base + i]);
    const float g = GAMMA_F32 ? static_cast<const float*>(gamma)[i] : Num<T>::up(static_cast<const T*>(gamma)[i]);
    y[base + i] = Num<T>::down(f * inv * g);
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
    const int staged = hidden <= 12 * 1024 ? hidden : 0;  // <= 48 KiB of dynamic shared memory (no opt-in needed)
    rmsnorm_generic_kernel<T, FUSED, GAMMA_F32><<<rows, threads, size_t(staged) * sizeof(float), st>>>(xp, gamma, yp, ri, ro, hidden, eps, staged);
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
