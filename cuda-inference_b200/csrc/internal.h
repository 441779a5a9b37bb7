// Internal interfaces between the C ABI layer (api.cu) and the kernel translation units.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace gieb {

// Device-status codes ORed into a plan's status word by a kernel that gave up on a bounded wait.
enum : uint32_t {
  kStatusProducerTimeout = 1u << 0,
  kStatusMmaTimeout = 1u << 1,
  kStatusEpilogueTimeout = 1u << 2,
};

constexpr int kNumSms = 148;       // streaming multiprocessors of the one supported target (B200): grids are sized in multiples of it
constexpr int kTileM = 128;        // output pixels per CTA tile = TMEM lanes = UMMA M
constexpr int kMaxStages = 8;
constexpr int kProducerWarps = 3;  // warps 0..2 issue the TMA loads, slab by slab in turn
// warp 3: MMA issuer and TMEM owner; warps 4..11 (4..19 with 16 epilogue warps): epilogue
static_assert((kProducerWarps + 1) % 4 == 0, "epilogue warp w must sit on TMEM lane quarter w % 4");

// Division by a run-time constant as multiply-high + shift (round-up reciprocal method): exact for 0 <= n < 2^31 and
// 1 <= d < 2^31.  The host builds it once per launch; a device-side divide costs a few cycles instead of ~150.
struct FastDiv {
  uint32_t d, mul, shr;
#if defined(__CUDACC__)
  __host__ __device__
#endif
  static FastDiv make(int divisor) {
    FastDiv f;
    f.d = uint32_t(divisor);
    if (divisor <= 1) {
      f.mul = 0;
      f.shr = 0;
    } else {
      uint32_t lg = 0;  // ceil(log2(d))
      while ((1ull << lg) < uint64_t(f.d)) ++lg;
      const uint32_t p = 31 + lg;
      f.mul = uint32_t(((1ull << p) + f.d - 1) / f.d);
      f.shr = p - 32;
    }
    return f;
  }
#if defined(__CUDACC__)
  __device__ __forceinline__ int div(int n) const { return d == 1 ? n : int(__umulhi(uint32_t(n), mul) >> shr); }
  __device__ __forceinline__ void divmod(int n, int& q, int& r) const {
    q = div(n);
    r = n - q * int(d);
  }
#endif
  int div_host(int n) const { return d == 1 ? n : int((uint64_t(uint32_t(n)) * mul >> 32) >> shr); }
};

#if defined(__CUDACC__)
// Launch with programmatic stream serialization: the grid may be scheduled before the previous kernel of the stream
// has finished; the kernel orders itself with ptx::grid_dep_wait().  Works under stream capture (the edge becomes a
// programmatic dependency of the graph).
// GIEB_DISABLE_PDL=1 in the environment launches every kernel fully serialised (a debugging aid).
bool pdl_enabled();
bool prefetch_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                      unsigned cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  return launch_pdl_cluster(kernel, grid, block, smem, stream, 1u, static_cast<Args&&>(args)...);
}
#endif

// Everything the tensor-core kernel needs besides the two tensor maps.  Plain data, passed by value.
struct ConvTcParams {
  int m_total;        // GEMM rows: B * P * Q output pixels (modes 0, 1) or box-numbered rows (mode 2)
  int64_t y_elems;    // B * O * P * Q
  int out_channels;   // O (GEMM N)
  int out_h, out_w;   // P, Q
  int pq;             // P * Q
  int kernel_w;       // S (taps are enumerated r-major: tap = r * S + s)
  int c_padded;       // channels of the NHWC copy / prepacked weights
  int kb_per_tap;     // c_padded / BK
  int total_kb;       // R * S * kb_per_tap reduction slabs
  int kb_per_split;   // slabs per split-K slice
  int tiles_m, tiles_n;  // tile grid over (pixels, output channels)
  int num_tiles;      // tiles_m * tiles_n * split_k: the list every persistent CTA walks with stride gridDim.x
  int stride_h, stride_w, pad_h, pad_w;
  int stages;
  int relu, has_bias, is_bf16, bias_fp32;
  // 1: FP32 storage computed as TF32 (kind::tf32).  Tile and padding quantities (BK, c_padded, kb_per_tap) stay in
  // 2-byte units, i.e. twice the FP32 element counts; TMA coordinates along channels are halved; Y is float.
  int is_tf32;
  int is_fp8;            // FP8 E4M3 operands (kind::f8f6f4), FP16 output: channel coordinates are twice the 2-byte-unit counts
  // How the activation operand reaches shared memory:
  //   0  im2col-mode TMA over the channel-padded NHWC copy (any kernel / stride / padding)
  //   1  tiled TMA over the same copy seen as the matrix [pixels][c_padded] (1x1, stride 1, pad 0)
  //   2  tiled TMA straight from the caller's NCHW tensor, pixels contiguous (MN-major operand; 1x1, stride 1,
  //      pad 0, H*W % 8 == 0, 16-byte aligned x): no repack of the activations at all.  Rows of the GEMM are then
  //      numbered in 64-pixel boxes that never straddle an image: m_total = batch * boxes_per_image * 64.
  int a_mode;
  int boxes_per_image;  // mode 2: ceil(H*W / 64)
  int strip_bytes;      // mode 3: bytes of one position strip (one TMA box); rows are numbered in 128-row boxes per output row
  FastDiv fd_out_h;     // mode 3: reciprocal of out_h
  uint32_t idesc;
  // > 1: split-K slices of one tile form a thread-block cluster (cluster rank = slice) and are summed through
  // distributed shared memory; blockIdx.x = tile * cluster_split + slice, one tile per CTA, `partial` unused.
  int cluster_split;
  FastDiv fd_cluster;
  FastDiv fd_tiles_mn, fd_tiles_n, fd_pq, fd_out_w, fd_kb_per_tap, fd_kernel_w, fd_boxes;  // reciprocals of the fields above
  const void* bias;
  const void* residual;  // optional tensor of the output's shape, layout and type, added before the activation
  int out_nhwc;          // 0: y (and residual, partials) are NCHW; 1: channel-contiguous [B][P][Q][O]
  int out_tma, res_tma;  // channel-contiguous output leaves through TMA stores / the residual arrives through TMA loads
  // Transposed-accumulator kernels: swap_tma = y may be written by TMA stores over its {P*Q, O, N} view (16-byte aligned y,
  // P*Q % 8 == 0); out_vec = pixels per store (4, 2 or 1) of the path that handles everything else (a unit that crosses
  // into the next image, or an unaligned y): needs P*Q % out_vec == 0 and y aligned to 2 * out_vec bytes.
  int swap_tma, out_vec;
  void* y;            // output in the storage type (split_k == 1 or cluster reduction)
  float* partial;     // [splits][B*O*P*Q] FP32 partial sums in the output's element order (workspace reduction), else null
  uint32_t* status;
  long long wait_limit;  // SM cycles a device-side wait may last before its role gives up and reports to *status
  int res_vec;           // transposed-accumulator epilogue: the residual may be read as 16-byte vectors (pointer 16-byte aligned)
  uint32_t debug_skip;   // test hook, 0 in production: bit 0 = the producers load nothing, bit 1 = the MMA warp issues nothing
};

// tile_m is 128 or 256 output pixels per CTA (one or two TMEM accumulators sharing each weight tile).
// pair: the tile belongs to a CTA pair (tile_m = 256), each CTA stages 128 activation rows and tile_n / 2 weight rows.
// epilogue_bytes: staging of the epilogue behind the ring (TMA-store boxes, or the NCHW transposition tiles).
size_t conv_tc_smem_bytes(int tile_m, int tile_n, int tile_k, int stages, size_t epilogue_bytes, bool pair = false);
size_t conv_tc_epilogue_staging_bytes(int tile_n);
// epi_warps: 8, or 16 for CTAs that have an SM to themselves (tile_n >= 128 only)
int conv_tc_threads(int epi_warps);
cudaError_t conv_tc_prepare(int tile_m, int tile_n, int tile_k, int epi_warps, size_t smem_bytes);  // opt in to large dynamic shared memory
// tm_out / tm_res: the output and the residual as 2-D tensors {channels, pixels} with a 32 x 32 box and 64-byte swizzle;
// read only when p.out_tma / p.res_tma are set.
cudaError_t conv_tc_launch(int tile_m, int tile_n, int tile_k, int epi_warps, const CUtensorMap& tm_act, const CUtensorMap& tm_wgt,
                           const CUtensorMap& tm_out, const CUtensorMap& tm_res, const ConvTcParams& p, dim3 grid, size_t smem_bytes,
                           cudaStream_t stream);

// CTA-pair points (tcgen05.mma.cta_group::2): tile_m = 256, tile_n 64 / 128 / 256; `grid` = 2 x the number of pairs.
int conv_tc_pair_epi_warps(int tile_n);
cudaError_t conv_tc_pair_prepare(int tile_n, int tile_k, size_t smem_bytes);
cudaError_t conv_tc_pair_launch(int tile_n, int tile_k, const CUtensorMap& tm_act, const CUtensorMap& tm_wgt, const CUtensorMap& tm_out,
                                const CUtensorMap& tm_res, const ConvTcParams& p, dim3 grid, size_t smem_bytes, cudaStream_t stream);

// Transposed-accumulator points (lane = output channel): NCHW output through TMA stores; tile_n 128 or 256, 16-bit types.
// tm_out: y as the 3-D tensor {P*Q, O, N} with a 32-pixel x 32-channel box and 64-byte swizzle (read when p.swap_tma).
cudaError_t conv_tc_swap_prepare(int tile_m, int tile_n, int tile_k, int epi_warps, size_t smem_bytes);
cudaError_t conv_tc_swap_launch(int tile_m, int tile_n, int tile_k, int epi_warps, const CUtensorMap& tm_act, const CUtensorMap& tm_wgt,
                                const CUtensorMap& tm_out, const ConvTcParams& p, dim3 grid, size_t smem_bytes, cudaStream_t stream);

// Sum of split-K partials + bias (+ residual) + ReLU + one rounding; `total` = B*O*P*Q elements in the output's order.
cudaError_t splitk_reduce_launch(const float* partial, int splits, int64_t total, int out_channels, int pq,
                                 const void* bias, int bias_fp32, int relu, int out_type, const void* residual, int out_nhwc,
                                 void* y, cudaStream_t stream);  // out_type: 0 fp16, 1 bf16, 2 fp32

// 16-bit [B][C][HW] -> [B][HW][Cp] (zero-filled channel padding).
cudaError_t repack_launch(const void* src, void* dst, int batch, int channels, int hw, int c_padded, cudaStream_t stream);
// FP32 [B][C][HW] -> [B][HW][Cp] (Cp in FP32 elements) with every value rounded to TF32 (ties away).
cudaError_t repack_tf32_launch(const void* src, void* dst, int batch, int channels, int hw, int c_padded, cudaStream_t stream);
// 1-byte elements (FP8), two tensors in one launch: [batch][channels][hw] -> [batch][hw][c_padded], zero-padded channels;
// c_padded counts elements (a multiple of 32); destinations 16-byte aligned.
cudaError_t repack_bytes_pair_launch(const void* src_a, void* dst_a, int batch_a, int ch_a, int hw_a, int cp_a, const void* src_b,
                                     void* dst_b, int batch_b, int ch_b, int hw_b, int cp_b, cudaStream_t stream);
// Two repacks (activations + weights) in ONE launch; src_b == nullptr runs only the first.
// Column-pair gather (row gather for stride_w = 2 and <= 4 channels): X3[n][h][positions][8], W3[o][r][t_positions * 8].
cudaError_t gather_pairs_launch(const void* x, void* x3, int batch, int channels, int h, int w, int positions, int left, int t_positions,
                                int shift, const void* wsrc, void* w3, int out_channels, int kernel_h, int kernel_w, cudaStream_t stream);
// Activations of a strided 1x1 convolution: only the pixels it reads, [batch][out_h * out_w][c_padded]; optionally the
// 1x1 filters in the same launch.
cudaError_t repack_subsampled_launch(const void* x, void* xn, int batch, int channels, int h, int w, int out_h, int out_w, int stride_h,
                                     int stride_w, int c_padded, const void* wsrc, void* wdst, int out_channels, cudaStream_t stream);
cudaError_t repack_pair_launch(const void* src_a, void* dst_a, int batch_a, int ch_a, int hw_a, int cp_a, const void* src_b,
                               void* dst_b, int batch_b, int ch_b, int hw_b, int cp_b, cudaStream_t stream);

// Row gather for convolutions with few input channels (16-bit types, bit-exact):
//   x2[n][h][q][s*C + c] = x[n][c][h][q*stride_w - pad_w + s]   (c2 = padded S*C elements per position, zero-filled)
//   w2[o][r][s*C + c]    = w[o][c][r][s]
// x == nullptr gathers only the weights, wsrc == nullptr only the activations.  x2 needs 16-byte alignment.
cudaError_t gather_rows_launch(const void* x, void* x2, int batch, int channels, int h, int w, int q, int kernel_w, int stride_w,
                               int pad_w, int c2, const void* wsrc, void* w2, int out_channels, int kernel_h, cudaStream_t stream);

// FP32 SIMT implicit GEMM straight from NCHW.
cudaError_t conv_fp32_launch(const void* x, const void* w, const void* bias, void* y, int batch, int c, int h, int wd,
                             int o, int r, int s, int stride_h, int stride_w, int pad_h, int pad_w, int out_h, int out_w,
                             int relu, cudaStream_t stream);
int conv_fp32_tile(int64_t pixels, int o);          // 64 or 32: edge of the square output tile a CTA computes
int64_t conv_fp32_num_blocks(int64_t pixels, int o);

cudaError_t rmsnorm_launch(int rows, int hidden, float eps, int dtype, int gamma_fp32, const void* x, const void* gamma,
                           void* y, const void* res_in, void* res_out, cudaStream_t stream);

cudaError_t bias_act_launch(int precision, int64_t total, int channels, int hw, const void* bias, int relu, void* y,
                            cudaStream_t stream);
cudaError_t maxpool2d_launch(int precision, int batch, int channels, int h, int w, int k, int stride, int pad, const void* x,
                             void* y, cudaStream_t stream);
// [B][H][W][C] tensors, C % 8 == 0, 16-bit types.
cudaError_t maxpool2d_nhwc_launch(int precision, int batch, int channels, int h, int w, int k, int stride, int pad, const void* x,
                                  void* y, cudaStream_t stream);
cudaError_t add_relu_launch(int precision, int relu, const void* a, const void* b, void* y, int64_t n, cudaStream_t stream);

}  // namespace gieb
