// Instantiations and host-side dispatch of the transposed-accumulator points of the tensor-core convolution kernel
// (conv_tc_kernel.cuh with SWAP = true): NCHW output written by TMA stores.  A translation unit of its own so that it
// compiles beside the others.
#include "conv_tc_kernel.cuh"

namespace gieb {
namespace {

template <int BN, int BK, int MH, int EW>
cudaError_t prepare_swap(size_t smem_bytes) {
  return cudaFuncSetAttribute(conv_tc_kernel<BN, BK, MH, EW, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes));
}

template <int BN, int BK, int MH, int EW>
cudaError_t launch_swap(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& to, const CUtensorMap& tr, const ConvTcParams& p,
                        dim3 grid, size_t smem, cudaStream_t st) {
  cudaError_t e = launch_pdl_cluster(conv_tc_kernel<BN, BK, MH, EW, false, true>, grid, dim3(32 * (kProducerWarps + 1 + EW)), smem, st, 1u,
                                     ta, tw, to, tr, p);
  if (e != cudaSuccess) return e;
  return cudaGetLastError();
}

#define GIEB_TC_SWAP_DISPATCH(FN, ...)                                                        \
  switch ((epi_warps == 16 ? 1000000 : 0) + tile_m / 128 * 100000 + tile_n * 100 + tile_k) {  \
    case 0 + 1 * 100000 + 128 * 100 + 16: return FN<128, 16, 1, 8>(__VA_ARGS__);              \
    case 0 + 2 * 100000 + 128 * 100 + 16: return FN<128, 16, 2, 8>(__VA_ARGS__);              \
    case 0 + 1 * 100000 + 128 * 100 + 32: return FN<128, 32, 1, 8>(__VA_ARGS__);              \
    case 0 + 2 * 100000 + 128 * 100 + 32: return FN<128, 32, 2, 8>(__VA_ARGS__);              \
    case 0 + 1 * 100000 + 128 * 100 + 64: return FN<128, 64, 1, 8>(__VA_ARGS__);              \
    case 0 + 2 * 100000 + 128 * 100 + 64: return FN<128, 64, 2, 8>(__VA_ARGS__);              \
    case 0 + 1 * 100000 + 256 * 100 + 16: return FN<256, 16, 1, 8>(__VA_ARGS__);              \
    case 0 + 2 * 100000 + 256 * 100 + 16: return FN<256, 16, 2, 8>(__VA_ARGS__);              \
    case 0 + 1 * 100000 + 256 * 100 + 32: return FN<256, 32, 1, 8>(__VA_ARGS__);              \
    case 0 + 2 * 100000 + 256 * 100 + 32: return FN<256, 32, 2, 8>(__VA_ARGS__);              \
    case 0 + 1 * 100000 + 256 * 100 + 64: return FN<256, 64, 1, 8>(__VA_ARGS__);              \
    case 0 + 2 * 100000 + 256 * 100 + 64: return FN<256, 64, 2, 8>(__VA_ARGS__);              \
    case 1000000 + 1 * 100000 + 128 * 100 + 16: return FN<128, 16, 1, 16>(__VA_ARGS__);       \
    case 1000000 + 2 * 100000 + 128 * 100 + 16: return FN<128, 16, 2, 16>(__VA_ARGS__);       \
    case 1000000 + 1 * 100000 + 128 * 100 + 32: return FN<128, 32, 1, 16>(__VA_ARGS__);       \
    case 1000000 + 2 * 100000 + 128 * 100 + 32: return FN<128, 32, 2, 16>(__VA_ARGS__);       \
    case 1000000 + 1 * 100000 + 128 * 100 + 64: return FN<128, 64, 1, 16>(__VA_ARGS__);       \
    case 1000000 + 2 * 100000 + 128 * 100 + 64: return FN<128, 64, 2, 16>(__VA_ARGS__);       \
    case 1000000 + 1 * 100000 + 256 * 100 + 16: return FN<256, 16, 1, 16>(__VA_ARGS__);       \
    case 1000000 + 2 * 100000 + 256 * 100 + 16: return FN<256, 16, 2, 16>(__VA_ARGS__);       \
    case 1000000 + 1 * 100000 + 256 * 100 + 32: return FN<256, 32, 1, 16>(__VA_ARGS__);       \
    case 1000000 + 2 * 100000 + 256 * 100 + 32: return FN<256, 32, 2, 16>(__VA_ARGS__);       \
    case 1000000 + 1 * 100000 + 256 * 100 + 64: return FN<256, 64, 1, 16>(__VA_ARGS__);       \
    case 1000000 + 2 * 100000 + 256 * 100 + 64: return FN<256, 64, 2, 16>(__VA_ARGS__);       \
    default: return cudaErrorInvalidValue;                                                    \
  }

}  // namespace

cudaError_t conv_tc_swap_prepare(int tile_m, int tile_n, int tile_k, int epi_warps, size_t smem_bytes) {
  GIEB_TC_SWAP_DISPATCH(prepare_swap, smem_bytes)
}

cudaError_t conv_tc_swap_launch(int tile_m, int tile_n, int tile_k, int epi_warps, const CUtensorMap& tm_act, const CUtensorMap& tm_wgt,
                                const CUtensorMap& tm_out, const ConvTcParams& p, dim3 grid, size_t smem_bytes, cudaStream_t stream) {
  GIEB_TC_SWAP_DISPATCH(launch_swap, tm_act, tm_wgt, tm_out, tm_out, p, grid, smem_bytes, stream)
}

}  // namespace gieb
