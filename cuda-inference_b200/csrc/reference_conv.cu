// Support for validate-then-time tuning: a slow, obviously-correct GPU convolution with double accumulation, the
// comparison of a kernel's output against it under the scale-aware tolerance, and a reproducible fill of device
// buffers.  These stand in for gpu_conv2d_reference (src/runtime/reference.cu:83-93), TolerancePolicy /
// compare_outputs (src/runtime/reference.cu:139-205) and make_conv_data (src/runtime/testing.cu:83-86) of the
// reference library, which its autotuner links.  Nothing here runs on the forward path.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "internal.h"

namespace gieb {
namespace {

template <typename T> __device__ __forceinline__ double as_double(T v);
template <> __device__ __forceinline__ double as_double<float>(float v) { return double(v); }
template <> __device__ __forceinline__ double as_double<__half>(__half v) { return double(__half2float(v)); }
template <> __device__ __forceinline__ double as_double<__nv_bfloat16>(__nv_bfloat16 v) { return double(__bfloat162float(v)); }

// One thread per output element, NCHW; ref = act(sum + bias) rounded once to float, scale = sum |x*w| + |bias|.
template <typename T>
__global__ void __launch_bounds__(256)
reference_conv_kernel(const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias, float* __restrict__ ref,
                      float* __restrict__ scale, int B, int C, int H, int W, int O, int R, int S, int sh, int sw, int ph, int pw,
                      int P, int Q, int relu) {
  const int64_t total = int64_t(B) * O * P * Q;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
    const int q = int(i % Q);
    int64_t t = i / Q;
    const int p = int(t % P);
    t /= P;
    const int o = int(t % O);
    const int n = int(t / O);
    double acc = 0.0, mag = 0.0;
    for (int c = 0; c < C; ++c)
      for (int r = 0; r < R; ++r) {
        const int ih = p * sh - ph + r;
        if (ih < 0 || ih >= H) continue;
        for (int s = 0; s < S; ++s) {
          const int iw = q * sw - pw + s;
          if (iw < 0 || iw >= W) continue;
          const double a = as_double(x[((int64_t(n) * C + c) * H + ih) * W + iw]);
          const double b = as_double(w[((int64_t(o) * C + c) * R + r) * S + s]);
          acc += a * b;
          mag += fabs(a * b);
        }
      }
    if (bias != nullptr) {
      const double b = as_double(bias[o]);
      acc += b;
      mag += fabs(b);
    }
    if (relu && acc < 0.0) acc = 0.0;
    ref[i] = float(acc);
    scale[i] = float(mag);
  }
}

struct Tolerance {
  double c_acc, c_out, u_acc, u_out, abs_floor, sqrt_k;
};

// out[0] = elements over tolerance, out[1] = non-finite elements, out[2] = bits of max |err| (as a non-negative float)
template <typename T>
__global__ void __launch_bounds__(256)
check_output_kernel(const T* __restrict__ y, const float* __restrict__ ref, const float* __restrict__ scale, int64_t n, Tolerance t,
                    unsigned long long* out) {
  unsigned long long over = 0, bad = 0;
  float worst = 0.f;
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    const double v = as_double(y[i]);
    if (isnan(v) || isinf(v)) { ++bad; continue; }
    const double err = fabs(v - double(ref[i]));
    const double tol = t.c_acc * t.u_acc * t.sqrt_k * double(scale[i]) + t.c_out * t.u_out * fabs(double(ref[i])) + t.abs_floor;
    if (err > tol) ++over;
    worst = fmaxf(worst, float(err));
  }
  if (over) atomicAdd(&out[0], over);
  if (bad) atomicAdd(&out[1], bad);
  atomicMax(reinterpret_cast<unsigned int*>(&out[2]), __float_as_uint(worst));  // non-negative floats order like their bits
}

__device__ __forceinline__ uint64_t splitmix(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void __launch_bounds__(256) fill_uniform_kernel(T* p, int64_t n, uint64_t seed, float lo, float hi) {
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    const uint64_t r = splitmix(seed * 0x100000001B3ull + uint64_t(i));
    const float u = float(r >> 40) * (1.0f / 16777216.0f);  // 24 random bits -> [0, 1)
    p[i] = from_float<T>(lo + (hi - lo) * u);
  }
}

unsigned blocks_for(int64_t n) {
  int64_t b = (n + 255) / 256;
  if (b > 148 * 64) b = 148 * 64;
  return unsigned(b < 1 ? 1 : b);
}

}  // namespace

cudaError_t reference_conv_launch(int precision, const void* x, const void* w, const void* bias, float* ref, float* scale, int B, int C,
                                  int H, int W, int O, int R, int S, int sh, int sw, int ph, int pw, int P, int Q, int relu,
                                  cudaStream_t st) {
  const unsigned g = blocks_for(int64_t(B) * O * P * Q);
  switch (precision) {
    case 0: reference_conv_kernel<float><<<g, 256, 0, st>>>(static_cast<const float*>(x), static_cast<const float*>(w), static_cast<const float*>(bias), ref, scale, B, C, H, W, O, R, S, sh, sw, ph, pw, P, Q, relu); break;
    case 1: reference_conv_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half*>(x), static_cast<const __half*>(w), static_cast<const __half*>(bias), ref, scale, B, C, H, W, O, R, S, sh, sw, ph, pw, P, Q, relu); break;
    case 2: reference_conv_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(bias), ref, scale, B, C, H, W, O, R, S, sh, sw, ph, pw, P, Q, relu); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t check_output_launch(int precision, const void* y, const float* ref, const float* scale, int64_t n, int64_t k,
                                unsigned long long* out3, cudaStream_t st) {
  // constants of TolerancePolicy::for_problem (src/runtime/reference.cu:139-167) for a single final rounding
  Tolerance t;
  t.c_acc = 8.0; t.c_out = 1.0; t.u_acc = 5.9604644775390625e-08; t.u_out = 5.9604644775390625e-08; t.abs_floor = 1e-30;
  if (precision == 1) { t.u_out = 4.8828125e-04; t.abs_floor = 3.0e-8; }
  if (precision == 2) t.u_out = 3.90625e-03;
  t.sqrt_k = sqrt(double(k));
  const unsigned g = blocks_for(n);
  switch (precision) {
    case 0: check_output_kernel<float><<<g, 256, 0, st>>>(static_cast<const float*>(y), ref, scale, n, t, out3); break;
    case 1: check_output_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half*>(y), ref, scale, n, t, out3); break;
    case 2: check_output_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(y), ref, scale, n, t, out3); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t fill_uniform_launch(int precision, void* p, int64_t n, uint64_t seed, float lo, float hi, cudaStream_t st) {
  const unsigned g = blocks_for(n);
  switch (precision) {
    case 0: fill_uniform_kernel<float><<<g, 256, 0, st>>>(static_cast<float*>(p), n, seed, lo, hi); break;
    case 1: fill_uniform_kernel<__half><<<g, 256, 0, st>>>(static_cast<__half*>(p), n, seed, lo, hi); break;
    case 2: fill_uniform_kernel<__nv_bfloat16><<<g, 256, 0, st>>>(static_cast<__nv_bfloat16*>(p), n, seed, lo, hi); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace gieb
