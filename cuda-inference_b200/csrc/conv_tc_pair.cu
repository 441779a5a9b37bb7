// Instantiations and host-side dispatch of the CTA-pair points of the tensor-core convolution kernel
// (conv_tc_kernel.cuh with PAIR = true): 256-pixel x tile_n-channel tiles computed by clusters of two CTAs with
// tcgen05.mma.cta_group::2.  A translation unit of its own so that it compiles beside the single-CTA points.
#include "conv_tc_kernel.cuh"

namespace gieb {
namespace {

template <int BN, int BK, int EW>
cudaError_t prepare_pair(size_t smem_bytes) {
  return cudaFuncSetAttribute(conv_tc_kernel<BN, BK, 1, EW, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes));
}

template <int BN, int BK, int EW>
cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tw, const CUtensorMap& to, const CUtensorMap& tr, const ConvTcParams& p,
                        dim3 grid, size_t smem, cudaStream_t st) {
  // the cluster is the pair: blockIdx.x = 2 * pair + rank
  cudaError_t e = launch_pdl_cluster(conv_tc_kernel<BN, BK, 1, EW, true>, grid, dim3(32 * (kProducerWarps + 1 + EW)), smem, st, 2u, ta, tw, to,
                                     tr, p);
  if (e != cudaSuccess) return e;
  return cudaGetLastError();
}

// 64-column tiles drain with 8 epilogue warps, wider ones with 16 (a CTA of a pair always has its SM to itself).
#define GIEB_TC_PAIR_DISPATCH(FN, ...)                                  \
  switch (tile_n * 100 + tile_k) {                                      \
    case 64 * 100 + 16: return FN<64, 16, 8>(__VA_ARGS__);              \
    case 64 * 100 + 32: return FN<64, 32, 8>(__VA_ARGS__);              \
    case 64 * 100 + 64: return FN<64, 64, 8>(__VA_ARGS__);              \
    case 128 * 100 + 16: return FN<128, 16, 16>(__VA_ARGS__);           \
    case 128 * 100 + 32: return FN<128, 32, 16>(__VA_ARGS__);           \
    case 128 * 100 + 64: return FN<128, 64, 16>(__VA_ARGS__);           \
    case 256 * 100 + 16: return FN<256, 16, 16>(__VA_ARGS__);           \
    case 256 * 100 + 32: return FN<256, 32, 16>(__VA_ARGS__);           \
    case 256 * 100 + 64: return FN<256, 64, 16>(__VA_ARGS__);           \
    default: return cudaErrorInvalidValue;                              \
  }

}  // namespace

int conv_tc_pair_epi_warps(int tile_n) { return tile_n >= 128 ? 16 : 8; }

cudaError_t conv_tc_pair_prepare(int tile_n, int tile_k, size_t smem_bytes) { GIEB_TC_PAIR_DISPATCH(prepare_pair, smem_bytes) }

cudaError_t conv_tc_pair_launch(int tile_n, int tile_k, const CUtensorMap& tm_act, const CUtensorMap& tm_wgt, const CUtensorMap& tm_out,
                                const CUtensorMap& tm_res, const ConvTcParams& p, dim3 grid, size_t smem_bytes, cudaStream_t stream) {
  GIEB_TC_PAIR_DISPATCH(launch_pair, tm_act, tm_wgt, tm_out, tm_res, p, grid, smem_bytes, stream)
}

}  // namespace gieb
