// Instantiations and host-side dispatch of the single-CTA points of the tensor-core convolution kernel
// (conv_tc_kernel.cuh), and the split-K reduction kernel.
#include "conv_tc_kernel.cuh"

namespace gieb {
namespace {

template <int BN, int BK, int MH, int EW>
cudaError_t prepare_one(size_t smem_bytes) {
  return cudaFuncSetAttribute(conv_tc_kernel<BN, BK, MH, EW, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes));
}

template <int BN, int BK, int MH, int EW>
cudaError_t launch_one(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& to, const CUtensorMap& tr, const ConvTcParams& p,
                       dim3 grid, size_t smem, cudaStream_t st) {
  cudaError_t e = launch_pdl_cluster(conv_tc_kernel<BN, BK, MH, EW, false>, grid, dim3(32 * (kProducerWarps + 1 + EW)), smem, st,
                                     unsigned(p.cluster_split > 1 ? p.cluster_split : 1), ta, tw, to, tr, p);
  if (e != cudaSuccess) return e;
  return cudaGetLastError();
}

#define GIEB_TC_DISPATCH(FN, ...) \
  switch ((epi_warps == 16 ? 1000000 : 0) + tile_m / 128 * 100000 + tile_n * 100 + tile_k) { \
    case 0 + 1 * 100000 + 32 * 100 + 16: return FN<32, 16, 1, 8>(__VA_ARGS__); \
    case 0 + 2 * 100000 + 32 * 100 + 16: return FN<32, 16, 2, 8>(__VA_ARGS__); \
    case 0 + 1 * 100000 + 32 * 100 + 32: return FN<32, 32, 1, 8>(__VA_ARGS__); \
    case 0 + 2 * 100000 + 32 * 100 + 32: return FN<32, 32, 2, 8>(__VA_ARGS__); \
    case 0 + 1 * 100000 + 32 * 100 + 64: return FN<32, 64, 1, 8>(__VA_ARGS__); \
    case 0 + 2 * 100000 + 32 * 100 + 64: return FN<32, 64, 2, 8>(__VA_ARGS__); \
    case 0 + 1 * 100000 + 64 * 100 + 16: return FN<64, 16, 1, 8>(__VA_ARGS__); \
    case 0 + 2 * 100000 + 64 * 100 + 16: return FN<64, 16, 2, 8>(__VA_ARGS__); \
    case 0 + 1 * 100000 + 64 * 100 + 32: return FN<64, 32, 1, 8>(__VA_ARGS__); \
    case 0 + 2 * 100000 + 64 * 100 + 32: return FN<64, 32, 2, 8>(__VA_ARGS__); \
    case 0 + 1 * 100000 + 64 * 100 + 64: return FN<64, 64, 1, 8>(__VA_ARGS__); \
    case 0 + 2 * 100000 + 64 * 100 + 64: return FN<64, 64, 2, 8>(__VA_ARGS__); \
    case 0 + 1 * 100000 + 128 * 100 + 16: return FN<128, 16, 1, 8>(__VA_ARGS__); \
    case 0 + 2 * 100000 + 128 * 100 + 16: return FN<128, 16, 2, 8>(__VA_ARGS__); \
    case 0 + 1 * 100000 + 128 * 100 + 32: return FN<128, 32, 1, 8>(__VA_ARGS__); \
    case 0 + 2 * 100000 + 128 * 100 + 32: return FN<128, 32, 2, 8>(__VA_ARGS__); \
    case 0 + 1 * 100000 + 128 * 100 + 64: return FN<128, 64, 1, 8>(__VA_ARGS__); \
    case 0 + 2 * 100000 + 128 * 100 + 64: return FN<128, 64, 2, 8>(__VA_ARGS__); \
    case 0 + 1 * 100000 + 256 * 100 + 16: return FN<256, 16, 1, 8>(__VA_ARGS__); \
    case 0 + 2 * 100000 + 256 * 100 + 16: return FN<256, 16, 2, 8>(__VA_ARGS__); \
    case 0 + 1 * 100000 + 256 * 100 + 32: return FN<256, 32, 1, 8>(__VA_ARGS__); \
    case 0 + 2 * 100000 + 256 * 100 + 32: return FN<256, 32, 2, 8>(__VA_ARGS__); \
    case 0 + 1 * 100000 + 256 * 100 + 64: return FN<256, 64, 1, 8>(__VA_ARGS__); \
    case 0 + 2 * 100000 + 256 * 100 + 64: return FN<256, 64, 2, 8>(__VA_ARGS__); \
    case 1000000 + 1 * 100000 + 128 * 100 + 16: return FN<128, 16, 1, 16>(__VA_ARGS__); \
    case 1000000 + 2 * 100000 + 128 * 100 + 16: return FN<128, 16, 2, 16>(__VA_ARGS__); \
    case 1000000 + 1 * 100000 + 128 * 100 + 32: return FN<128, 32, 1, 16>(__VA_ARGS__); \
    case 1000000 + 2 * 100000 + 128 * 100 + 32: return FN<128, 32, 2, 16>(__VA_ARGS__); \
    case 1000000 + 1 * 100000 + 128 * 100 + 64: return FN<128, 64, 1, 16>(__VA_ARGS__); \
    case 1000000 + 2 * 100000 + 128 * 100 + 64: return FN<128, 64, 2, 16>(__VA_ARGS__); \
    case 1000000 + 1 * 100000 + 256 * 100 + 16: return FN<256, 16, 1, 16>(__VA_ARGS__); \
    case 1000000 + 2 * 100000 + 256 * 100 + 16: return FN<256, 16, 2, 16>(__VA_ARGS__); \
    case 1000000 + 1 * 100000 + 256 * 100 + 32: return FN<256, 32, 1, 16>(__VA_ARGS__); \
    case 1000000 + 2 * 100000 + 256 * 100 + 32: return FN<256, 32, 2, 16>(__VA_ARGS__); \
    case 1000000 + 1 * 100000 + 256 * 100 + 64: return FN<256, 64, 1, 16>(__VA_ARGS__); \
    case 1000000 + 2 * 100000 + 256 * 100 + 64: return FN<256, 64, 2, 16>(__VA_ARGS__); \
    default: return cudaErrorInvalidValue;                                            \
  }

// ---- split-K reduction: y = round(act(sum_z partial[z] + bias)) -------------------------------------------------
// Follows the arithmetic of splitk_reduce (src/kernels/tensor_core_mma.cu:254-262): partials summed in slice order
// in FP32, then bias, ReLU and one rounding.
template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ partial, int splits, int64_t total, int64_t slice_stride, int out_channels,
                     int pq, FastDiv fd_pq, FastDiv fd_oc, const void* __restrict__ bias, int bias_fp32, int relu,
                     const T* residual, int out_nhwc, T* y) {
  ptx::grid_dep_wait();  // launched with programmatic stream serialization right behind the convolution kernel
  const int64_t step = int64_t(gridDim.x) * blockDim.x;
  const int64_t first = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  // bias of the channel of element i plus, when given, the residual element (same layout as the output)
  auto bias_of = [&](int64_t i) -> float {
    float extra = residual != nullptr ? to_f32(residual[i]) : 0.f;
    if (bias == nullptr) return extra;
    int oc;
    if (total < (int64_t(1) << 31)) {  // the usual case: multiply-high divisions
      if (out_nhwc) {
        oc = int(i) - fd_oc.div(int(i)) * out_channels;
      } else {
        const int plane = fd_pq.div(int(i));
        oc = plane - fd_oc.div(plane) * out_channels;
      }
    } else {
      oc = out_nhwc ? int(i % out_channels) : int((i / pq) % out_channels);
    }
    return extra + (bias_fp32 ? static_cast<const float*>(bias)[oc] : to_f32(static_cast<const T*>(bias)[oc]));
  };
  if (VEC) {
    const int64_t nvec = total >> 2;
    for (int64_t v = first; v < nvec; v += step) {
      float4 acc = reinterpret_cast<const float4*>(partial)[v];
      for (int z = 1; z < splits; ++z) {
        const float4 q = reinterpret_cast<const float4*>(partial + z * slice_stride)[v];
        acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
      }
      const int64_t i = v << 2;
      float r[4] = {acc.x + bias_of(i), acc.y + bias_of(i + 1), acc.z + bias_of(i + 2), acc.w + bias_of(i + 3)};
      if (relu) {
#pragma unroll
        for (int j = 0; j < 4; ++j) r[j] = fmaxf(r[j], 0.f);
      }
      T o[4] = {from_f32<T>(r[0]), from_f32<T>(r[1]), from_f32<T>(r[2]), from_f32<T>(r[3])};
      reinterpret_cast<uint2*>(y)[v] = *reinterpret_cast<const uint2*>(o);
    }
    for (int64_t i = (nvec << 2) + first; i < total; i += step) {
      float acc = 0.f;
      for (int z = 0; z < splits; ++z) acc += partial[z * slice_stride + i];
      acc += bias_of(i);
      if (relu) acc = fmaxf(acc, 0.f);
      y[i] = from_f32<T>(acc);
    }
  } else {
    for (int64_t i = first; i < total; i += step) {
      float acc = 0.f;
      for (int z = 0; z < splits; ++z) acc += partial[z * slice_stride + i];
      acc += bias_of(i);
      if (relu) acc = fmaxf(acc, 0.f);
      y[i] = from_f32<T>(acc);
    }
  }
}

}  // namespace

// 8 epilogue warps x ceil(chunks / 2) boxes = 16 warps x ceil(chunks / 4) boxes for the tile widths that may run 16 warps
size_t conv_tc_epilogue_staging_bytes(int tile_n) { return size_t(8) * (tile_n >= 64 ? tile_n / 64 : 1) * 2048; }

int conv_tc_threads(int epi_warps) { return 32 * (kProducerWarps + 1 + epi_warps); }

size_t conv_tc_smem_bytes(int tile_m, int tile_n, int tile_k, int stages, size_t epilogue_bytes, bool pair) {
  const size_t rows = pair ? size_t(kTileM) + tile_n / 2 : size_t(tile_m) + tile_n;  // operand rows one CTA stages per slab
  return 1024 + kCtrlBytes + size_t(stages) * rows * tile_k * 2 + epilogue_bytes;
}

cudaError_t conv_tc_prepare(int tile_m, int tile_n, int tile_k, int epi_warps, size_t smem_bytes) {
  GIEB_TC_DISPATCH(prepare_one, smem_bytes)
}

cudaError_t conv_tc_launch(int tile_m, int tile_n, int tile_k, int epi_warps, const CUtensorMap& tm_act, const CUtensorMap& tm_wgt,
                           const CUtensorMap& tm_out, const CUtensorMap& tm_res, const ConvTcParams& p, dim3 grid, size_t smem_bytes,
                           cudaStream_t stream) {
  GIEB_TC_DISPATCH(launch_one, tm_act, tm_wgt, tm_out, tm_res, p, grid, smem_bytes, stream)
}

cudaError_t splitk_reduce_launch(const float* partial, int splits, int64_t total, int out_channels, int pq, const void* bias,
                                 int bias_fp32, int relu, int out_type, const void* residual, int out_nhwc, void* y,
                                 cudaStream_t stream) {
  const int64_t slice_stride = (total + 3) & ~int64_t(3);
  const bool vec = out_type != 2 && (reinterpret_cast<uintptr_t>(y) & 7u) == 0;
  const int64_t work = vec ? (total + 3) / 4 : total;
  int64_t blocks = (work + 255) / 256;
  if (blocks > kNumSms * 16) blocks = kNumSms * 16;
  if (blocks < 1) blocks = 1;
  const FastDiv fd_pq = FastDiv::make(pq), fd_oc = FastDiv::make(out_channels);
  cudaError_t e;
  if (out_type == 2) {
    auto* yy = static_cast<float*>(y);
    auto* rr = static_cast<const float*>(residual);
    e = launch_pdl(splitk_reduce_kernel<float, false>, dim3(unsigned(blocks)), dim3(256), 0, stream, partial, splits, total, slice_stride, out_channels, pq, fd_pq, fd_oc, bias, bias_fp32, relu, rr, out_nhwc, yy);
  } else if (out_type == 1) {
    auto* yy = static_cast<__nv_bfloat16*>(y);
    auto* rr = static_cast<const __nv_bfloat16*>(residual);
    if (vec) e = launch_pdl(splitk_reduce_kernel<__nv_bfloat16, true>, dim3(unsigned(blocks)), dim3(256), 0, stream, partial, splits, total, slice_stride, out_channels, pq, fd_pq, fd_oc, bias, bias_fp32, relu, rr, out_nhwc, yy);
    else e = launch_pdl(splitk_reduce_kernel<__nv_bfloat16, false>, dim3(unsigned(blocks)), dim3(256), 0, stream, partial, splits, total, slice_stride, out_channels, pq, fd_pq, fd_oc, bias, bias_fp32, relu, rr, out_nhwc, yy);
  } else {
    auto* yy = static_cast<__half*>(y);
    auto* rr = static_cast<const __half*>(residual);
    if (vec) e = launch_pdl(splitk_reduce_kernel<__half, true>, dim3(unsigned(blocks)), dim3(256), 0, stream, partial, splits, total, slice_stride, out_channels, pq, fd_pq, fd_oc, bias, bias_fp32, relu, rr, out_nhwc, yy);
    else e = launch_pdl(splitk_reduce_kernel<__half, false>, dim3(unsigned(blocks)), dim3(256), 0, stream, partial, splits, total, slice_stride, out_channels, pq, fd_pq, fd_oc, bias, bias_fp32, relu, rr, out_nhwc, yy);
  }
  return e != cudaSuccess ? e : cudaGetLastError();
}

}  // namespace gieb
