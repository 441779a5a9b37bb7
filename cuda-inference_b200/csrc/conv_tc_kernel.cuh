// Implicit-GEMM convolution on the sm_100a tensor cores.
//
// GEMM view used here (transposed with respect to the reference's, src/kernels/tensor_core_mma.cu:99-251, which
// puts output channels on M): rows (M) are output PIXELS, columns (N) are output CHANNELS, the reduction runs over
// (r, s, c) with the channel fastest:
//      D[pixel, oc] = sum_{r,s,c} Xn[pixel @ (r,s), c] * Wk[oc, (r,s), c]
//   * Xn is the channel-contiguous (NHWC, channel-padded) copy of the activations.  One reduction slab of BK
//     channels at one filter tap is fetched by a single TMA im2col-mode load, which also produces the zero
//     padding, the stride and the wrap from one output row / image to the next.
//   * Wk is the prepacked weight matrix [O][R*S*Cp]; a slab is one tiled TMA box.
//   * Both land in shared memory in the 128/64/32-byte swizzled K-major layout tcgen05.mma reads, in a ring of
//     `stages` buffers guarded by full/empty mbarriers.
//   * One thread issues tcgen05.mma (128 x BN x 16 per instruction); the FP32 accumulator tile lives in tensor
//     memory: lane = pixel, column = output channel.  CTAs are persistent and the accumulator is double-buffered.
//   * Eight or sixteen epilogue warps read the accumulators with tcgen05.ld, add bias, apply ReLU, round once to the
//     storage type and store.  NCHW: for a fixed channel the 32 lanes of a warp hold 32 consecutive pixels, so every store
//     instruction writes one contiguous run, and any output pointer alignment is legal
//     (tests/test_runtime_concurrency.cu:190-216).  Channel-contiguous output: 32 x 32 boxes staged in shared memory and
//     written by TMA stores.  With split-K the FP32 partial tile is stored (or exchanged inside a cluster) instead.
// Two more forms of the same kernel, chosen per plan: CTA pairs (PAIR: 256-pixel tiles on tcgen05.mma.cta_group::2) and
// the transposed accumulator (SWAP: lane = output channel, NCHW output through TMA stores); see the template below.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "internal.h"
#include "ptx.cuh"

namespace gieb {
namespace {

constexpr uint32_t kCtrlBytes = 3072;  // [0,2048): two bias tiles as float; [2048,3072): mbarriers + TMEM address slot

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p) {
  if constexpr (std::is_same<T, __half>::value) return __half2float(*p);
  else if constexpr (std::is_same<T, float>::value) return *p;
  else return __bfloat162float(*p);
}

template <typename T>
__device__ __forceinline__ T round_to(float a) {
  if constexpr (std::is_same<T, __half>::value) return __float2half_rn(a);
  else if constexpr (std::is_same<T, float>::value) return a;
  else return __float2bfloat16_rn(a);
}

// Epilogue of one 32-column chunk for one accumulator row (= one output pixel): + bias, optional ReLU, one rounding,
// 32 stores that are `stride` elements apart (consecutive output channels of an NCHW tensor).  Branch-free body:
// the ReLU / storage-type / full-chunk decisions are made once per chunk by the caller.
template <typename T, bool RELU>
__device__ __forceinline__ void store_chunk_full(const uint32_t (&v)[32], const float* __restrict__ bias, T* __restrict__ dst,
                                                 int64_t stride) {
  const float4* b4 = reinterpret_cast<const float4*>(bias);
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const float4 b = b4[q];
    const float bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      float a = __uint_as_float(v[q * 4 + t]) + bb[t];
      if (RELU) a = fmaxf(a, 0.f);
      *dst = round_to<T>(a);
      dst += stride;
    }
  }
}

// General form: any element stride, partial chunks, optional residual (same layout as the output).
template <typename T, bool RELU>
__device__ __forceinline__ void store_chunk_tail(const uint32_t (&v)[32], const float* __restrict__ bias, T* dst, const T* res,
                                                 int64_t stride, int nvalid) {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    if (j < nvalid) {
      float a = __uint_as_float(v[j]) + bias[j];
      if (res != nullptr) a += load_as_float(res + int64_t(j) * stride);
      if (RELU) a = fmaxf(a, 0.f);
      dst[int64_t(j) * stride] = round_to<T>(a);
    }
  }
}

// A full chunk with a residual in the output's own layout.  Nothing proves to the compiler that the residual and the output
// do not overlap, so written as one loop every load would wait for the store before it: the loads of eight channels are
// issued as a group, then their eight stores.
template <typename T, bool RELU>
__device__ __forceinline__ void store_chunk_full_res(const uint32_t (&v)[32], const float* __restrict__ bias, T* dst, const T* res,
                                                     int64_t stride) {
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float r[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = load_as_float(res + int64_t(g * 8 + j) * stride);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float a = __uint_as_float(v[g * 8 + j]) + bias[g * 8 + j] + r[j];
      if (RELU) a = fmaxf(a, 0.f);
      dst[int64_t(g * 8 + j) * stride] = round_to<T>(a);
    }
  }
}

// Eight consecutive channels of one accumulator row: + bias (+ residual) -> ReLU -> one rounding, packed as 16 bytes.
template <typename T, bool RELU, bool RES>
__device__ __forceinline__ uint4 finish8(const uint32_t (&v)[32], int q, const float* __restrict__ bias, uint4 r) {
  const float4* b4 = reinterpret_cast<const float4*>(bias);
  const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
  uint32_t ow[4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float4 b = b4[q * 2 + h];
    const float bb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      float a0 = __uint_as_float(v[q * 8 + h * 4 + t * 2]) + bb[t * 2];
      float a1 = __uint_as_float(v[q * 8 + h * 4 + t * 2 + 1]) + bb[t * 2 + 1];
      if (RES) {
        const uint32_t w = rw[h * 2 + t];
        if constexpr (std::is_same<T, __half>::value) {
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
          a0 += f.x; a1 += f.y;
        } else {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w));
          a0 += f.x; a1 += f.y;
        }
      }
      if (RELU) { a0 = fmaxf(a0, 0.f); a1 = fmaxf(a1, 0.f); }
      if constexpr (std::is_same<T, __half>::value) {
        const __half2 o = __floats2half2_rn(a0, a1);
        ow[h * 2 + t] = *reinterpret_cast<const uint32_t*>(&o);
      } else {
        const __nv_bfloat162 o = __floats2bfloat162_rn(a0, a1);
        ow[h * 2 + t] = *reinterpret_cast<const uint32_t*>(&o);
      }
    }
  }
  return make_uint4(ow[0], ow[1], ow[2], ow[3]);
}

// Channel-contiguous output: the 32 channels of a chunk are 64 contiguous, 16-byte aligned bytes of one pixel.
// Four 16-byte stores per lane (and four 16-byte residual loads) instead of 32 two-byte ones.
template <typename T, bool RELU, bool RES>
__device__ __forceinline__ void store_chunk_contiguous(const uint32_t (&v)[32], const float* __restrict__ bias, T* dst, const T* res) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 r = make_uint4(0, 0, 0, 0);
    if (RES) r = reinterpret_cast<const uint4*>(res)[q];
    reinterpret_cast<uint4*>(dst)[q] = finish8<T, RELU, RES>(v, q, bias, r);
  }
}

// The same chunk into a staging box for a TMA store: 32 rows (lanes) of 64 bytes in the 64-byte-swizzled layout the
// tensor map describes (16-byte cell q of row r sits at cell q ^ ((r >> 1) & 3)); bank-conflict free.  With RES the
// box already holds the residual values (a TMA load put them there) and is overwritten in place.
template <typename T, bool RELU, bool RES>
__device__ __forceinline__ void chunk_to_staging(const uint32_t (&v)[32], const float* __restrict__ bias, uint8_t* box, int lane) {
  uint8_t* row = box + lane * 64;
  const int sw = (lane >> 1) & 3;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4* cell = reinterpret_cast<uint4*>(row + ((q ^ sw) << 4));
    uint4 r = make_uint4(0, 0, 0, 0);
    if (RES) r = *cell;
    *cell = finish8<T, RELU, RES>(v, q, bias, r);
  }
}

template <typename T>
__device__ __forceinline__ void chunk_to_staging(const uint32_t (&v)[32], const float* bias, uint8_t* box, int lane, int relu, bool res) {
  if (res) {
    if (relu) chunk_to_staging<T, true, true>(v, bias, box, lane);
    else chunk_to_staging<T, false, true>(v, bias, box, lane);
  } else {
    if (relu) chunk_to_staging<T, true, false>(v, bias, box, lane);
    else chunk_to_staging<T, false, false>(v, bias, box, lane);
  }
}

// Transposed accumulator: 32 consecutive pixels of ONE channel (this lane's) -> + bias (+ residual), ReLU on the rounded pair
// (rounding is monotonic and keeps zero), packed as 64 bytes and written as the lane's row of the warp's staging box (32 rows of 64
// bytes, 64-byte swizzled: 16-byte cell q of row r sits at cell q ^ ((r >> 1) & 3); conflict-free).
template <typename T, bool RES>
__device__ __forceinline__ void row_to_staging(const uint32_t (&v)[32], float bias, const uint4 (&res)[4], bool relu, uint8_t* box, int lane) {
  uint32_t w[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float a0 = __uint_as_float(v[2 * j]) + bias, a1 = __uint_as_float(v[2 * j + 1]) + bias;
    if constexpr (RES) {  // the residual's 32 pixels of this lane's channel, in storage type
      const uint4& r4 = res[j >> 2];
      const uint32_t rw = (j & 3) == 0 ? r4.x : ((j & 3) == 1 ? r4.y : ((j & 3) == 2 ? r4.z : r4.w));
      if constexpr (std::is_same<T, __half>::value) {
        const float2 rf = __half22float2(*reinterpret_cast<const __half2*>(&rw));
        a0 += rf.x; a1 += rf.y;
      } else {
        const float2 rf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rw));
        a0 += rf.x; a1 += rf.y;
      }
    }
    if constexpr (std::is_same<T, __half>::value) {
      __half2 o = __floats2half2_rn(a0, a1);
      const __half2 oz = __hmax2(o, __half2half2(__ushort_as_half(0)));
      w[j] = relu ? *reinterpret_cast<const uint32_t*>(&oz) : *reinterpret_cast<const uint32_t*>(&o);
    } else {
      __nv_bfloat162 o = __floats2bfloat162_rn(a0, a1);
      const __nv_bfloat162 oz = __hmax2(o, __bfloat162bfloat162(__ushort_as_bfloat16(0)));
      w[j] = relu ? *reinterpret_cast<const uint32_t*>(&oz) : *reinterpret_cast<const uint32_t*>(&o);
    }
  }
  const int sw = (lane >> 1) & 3;
#pragma unroll
  for (int q = 0; q < 4; ++q)
    *reinterpret_cast<uint4*>(box + lane * 64 + ((q ^ sw) << 4)) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
}

// dst / res point at the first element of the chunk for this row; consecutive channels are `stride` elements apart
// (P*Q for NCHW, 1 for channel-contiguous output).
template <typename T>
__device__ __forceinline__ void store_chunk(const uint32_t (&v)[32], const float* bias, T* dst, const T* res, int64_t stride,
                                            int nvalid, int relu) {
  if constexpr (sizeof(T) == 2) {
    if (nvalid == 32 && stride == 1 && ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(res)) & 15u) == 0) {
      if (res != nullptr) {
        if (relu) store_chunk_contiguous<T, true, true>(v, bias, dst, res);
        else store_chunk_contiguous<T, false, true>(v, bias, dst, res);
      } else {
        if (relu) store_chunk_contiguous<T, true, false>(v, bias, dst, res);
        else store_chunk_contiguous<T, false, false>(v, bias, dst, res);
      }
      return;
    }
  }
  if (nvalid == 32 && res == nullptr) {
    if (relu) store_chunk_full<T, true>(v, bias, dst, stride);
    else store_chunk_full<T, false>(v, bias, dst, stride);
  } else if (nvalid == 32) {
    if (relu) store_chunk_full_res<T, true>(v, bias, dst, res, stride);
    else store_chunk_full_res<T, false>(v, bias, dst, res, stride);
  } else {
    if (relu) store_chunk_tail<T, true>(v, bias, dst, res, stride, nvalid);
    else store_chunk_tail<T, false>(v, bias, dst, res, stride, nvalid);
  }
}

// Output element type by the problem's precision: float for TF32, else the 16-bit storage type.
template <typename F>
__device__ __forceinline__ void with_output_type(const ConvTcParams& p, F&& f) {
  if (p.is_tf32) f(static_cast<float*>(p.y), static_cast<const float*>(p.residual));
  else if (p.is_bf16) f(static_cast<__nv_bfloat16*>(p.y), static_cast<const __nv_bfloat16*>(p.residual));
  else f(static_cast<__half*>(p.y), static_cast<const __half*>(p.residual));
}

// Persistent CTAs: each CTA walks the tile list (tile = blockIdx.x, += gridDim.x; output-channel tiles fastest, then
// pixel tiles, then split-K slices).  The operand ring and its phases run on across tiles, and the accumulator is
// double-buffered in tensor memory whenever two tiles fit the 512 columns, so the epilogue of tile t overlaps the
// loads and MMAs of tile t+1.
// MH = number of 128-pixel halves per tile (1 or 2).  With MH = 2 the tile is 256 pixels: two activation loads and two
// accumulators share every weight tile, which halves the weight traffic per FLOP.
// EW = number of epilogue warps, 8 or 16.  The epilogue is a long dependent instruction stream per warp (TMEM load ->
// bias -> ReLU -> rounding -> store, ~1100 cycles per 32-column chunk even with a warp alone on its scheduler), so
// CTAs that own an SM anyway (ring too large for two) run 16 epilogue warps: four per TMEM lane quarter.
// PAIR: the tile is 256 pixels x BN channels computed by a pair of CTAs (a cluster of two) with tcgen05.mma.cta_group::2:
// CTA r of the pair loads its own 128 pixels of the activation slab and its own BN / 2 rows of the weight slab (plain
// per-CTA TMA loads whose bytes are counted on the leader's full barrier), the leader's MMA warp issues one 256 x BN x 16
// instruction for both SMs and signals the ring slots and the accumulator barriers of both CTAs with multicast commits,
// and each CTA's epilogue warps drain the 128 accumulator rows that sit in their own tensor memory.  Per slab and SM that is
// (128 + BN / 2) rows of operands instead of (128 + BN): the weight traffic from L2 is halved.  MH = 1, no cluster split-K,
// 16-bit types.
// SWAP: the accumulator is held TRANSPOSED -- tensor-memory lane = output channel, column = output pixel -- by handing the
// weight slab to the instruction as its A operand (M = 128 channels per instruction, BN / 128 of them per slab) and the
// activation slab as its B operand (N = 128 or 256 pixels).  Shared-memory layouts and producers are unchanged: both slabs
// are K-major row blocks either way.  An epilogue thread then owns one channel and 32 consecutive pixels, i.e. 64
// contiguous bytes of an NCHW tensor: the warp stages its 32 channels x 32 pixels as one box and a TMA store writes it
// (tensor {P*Q, O, N}); for NCHW output whose planes are 16-byte multiples.  BN 128 or 256, 16-bit types, no split-K,
// no pair.
template <int BN, int BK, int MH, int EW, bool PAIR, bool SWAP = false>
__global__ void __launch_bounds__(32 * (kProducerWarps + 1 + EW), (EW == 16 || PAIR) ? 1 : 2)  // EW = 8: at most 80 registers, two CTAs per SM
conv_tc_kernel(const __grid_constant__ CUtensorMap tm_act, const __grid_constant__ CUtensorMap tm_wgt,
               const __grid_constant__ CUtensorMap tm_out, const __grid_constant__ CUtensorMap tm_res, const ConvTcParams p) {
  constexpr int ROW_BYTES = BK * 2;
  constexpr uint32_t A_HALF_BYTES = kTileM * ROW_BYTES;
  constexpr uint32_t A_BYTES = MH * A_HALF_BYTES;
  static_assert(!PAIR || (MH == 1 && BN >= 32), "a CTA pair computes one 256-pixel tile");
  static_assert(!SWAP || (!PAIR && BN % 128 == 0), "the transposed accumulator takes 128 channels per instruction");
  constexpr int B_ROWS = PAIR ? BN / 2 : BN;                   // weight rows this CTA loads per slab
  constexpr uint32_t B_BYTES = B_ROWS * ROW_BYTES;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr int MMAS_PER_SLAB = BK / 16;
  constexpr bool PAIR_SLABS = BN <= 128;                       // narrow MMAs are issue-bound: see the MMA role
  constexpr uint32_t ACC_COLS = MH * BN;                       // columns of one accumulator set
  constexpr int ACC_BUFS = ACC_COLS <= 256 ? 2 : 1;            // double-buffer when it fits
  constexpr uint32_t TMEM_COLS = ACC_COLS * ACC_BUFS < 32 ? 32 : ACC_COLS * ACC_BUFS;
  static_assert(TMEM_COLS <= 512, "accumulators must fit the 512 TMEM columns");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
  float* bias_s = reinterpret_cast<float*>(smem);  // [2][256]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + 2048);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* acc_full = empty_bar + kMaxStages;     // [2] MMA -> epilogue: accumulator complete
  uint64_t* acc_empty = acc_full + 2;              // [2] epilogue -> MMA: accumulator drained
  constexpr int EG = EW / 4;                        // epilogue warps per TMEM lane quarter
  constexpr int kEpiBufs = (BN / 32 + EG - 1) / EG;  // 32-column chunks one epilogue warp owns per 128-pixel half
  uint64_t* res_bar = acc_empty + 2;               // [EW epilogue warps][kEpiBufs] residual tile landed (TMA epilogue only)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(res_bar + EW * kEpiBufs);
  uint8_t* stage_base = smem + kCtrlBytes;
  // TMA epilogue staging: per epilogue warp kEpiBufs boxes of 32 pixels x 32 channels (2 KiB, 64-byte swizzle)
  uint8_t* epi_base = stage_base + size_t(p.stages) * STAGE_BYTES;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = p.stages;
  const int tiles_mn = p.tiles_m * p.tiles_n;
  const bool cluster = !PAIR && p.cluster_split > 1;
  const uint32_t pair_rank = PAIR ? ptx::cluster_ctarank() : 0u;  // 0 = leader (issues the MMAs), 1 = peer
  const bool leader = pair_rank == 0;
  // persistent walk over the tile list: by CTA, or by CTA pair
  const int tile_first = PAIR ? int(blockIdx.x >> 1) : int(blockIdx.x);
  const int tile_step = PAIR ? int(gridDim.x >> 1) : int(gridDim.x);
  ptx::grid_dep_launch();  // the next kernel of the stream may begin its own set-up (it orders itself with grid_dep_wait)

  if (threadIdx.x == 0) {
    ptx::prefetch_tensormap(&tm_act);
    ptx::prefetch_tensormap(&tm_wgt);
    if (p.out_tma) ptx::prefetch_tensormap(&tm_out);
    if (p.res_tma) ptx::prefetch_tensormap(&tm_res);
  }
  // The barriers are initialised by a thread of the last epilogue warp, which has nothing else to do before the set-up
  // barrier: the producers decode their first tile meanwhile (~25 cycles per mbarrier.init, one after the other).
  if (threadIdx.x == 32 * (kProducerWarps + EW)) {
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&acc_full[b], 1);
      ptx::mbar_init(&acc_empty[b], PAIR ? 2 * EW : EW);  // one arrival per epilogue warp (of both CTAs of a pair: the leader's barrier collects them)
    }
    if (p.res_tma)
      for (int b = 0; b < EW * kEpiBufs; ++b) ptx::mbar_init(&res_bar[b], 1);
    ptx::fence_mbar_init();
  }
  if (warp == kProducerWarps) {
    if constexpr (PAIR) {
      ptx::tmem_alloc_pair(tmem_slot, TMEM_COLS);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(tmem_slot, TMEM_COLS);
      ptx::tmem_relinquish();
    }
  }
  // The set-up barrier (mbarriers initialised, TMEM allocated) is joined by every warp exactly once, from inside its
  // role and only after it has decoded its first tile, so the decode overlaps the set-up instead of following it.
  // The kernel is launched with programmatic stream serialization: up to this join it may run beside the previous
  // kernel of the stream (the repack), so the join also waits for that kernel's completion.
  bool joined = false;
  uint32_t tmem_base = 0;
  auto join_setup = [&]() {
    if (!joined) {
      ptx::tc_fence_before_sync();
      // A pair joins across both CTAs: the peer signals the leader's barriers, which must be initialised by then.
      if constexpr (PAIR) ptx::cluster_sync_all();
      else asm volatile("bar.sync 0;" ::: "memory");
      ptx::tc_fence_after_sync();
      tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
      joined = true;
      ptx::grid_dep_wait();  // everything above overlapped the previous kernel; global memory is touched only below
    }
  };

  if (warp < kProducerWarps) {
    // ---------------- TMA producers ----------------
    // One TMA instruction keeps its issuing warp busy for a few hundred cycles whatever the box size, so a single
    // producer cannot feed the ring faster than about one slab per 600 cycles.  kProducerWarps warps therefore take
    // the slabs round-robin (warp j owns the CTA's slabs j, j + np, ...), each issuing the activation
    // boxes and the weight tile of its slab.  A warp walks its loop converged (every lane polls the barrier); lane l
    // issues activation box l, so the boxes of one slab leave in ONE instruction.  Ring slot, phase and filter-tap
    // counters advance incrementally: no integer division inside the slab loop.
    // No more producers than ring slots: a warp must never be a full ring ahead of its own previous slab, or the
    // parity of the slot's barrier could not tell its phases apart.
    const int np = min(kProducerWarps, stages);
    const int esh = p.is_tf32 ? 1 : (p.is_fp8 ? -1 : 0);  // channel coordinates from 2-byte-unit counts: halved for FP32, doubled for FP8
    auto ch = [esh](int units) { return esh > 0 ? units >> 1 : (esh < 0 ? units << 1 : units); };
    int s = warp;        // ring slot of this warp's next slab (the ring and its phases continue across tiles)
    uint32_t phase = 0;
    while (s >= stages) { s -= stages; phase ^= 1u; }
    int skip = warp;     // slabs of the coming tile that belong to other warps before this warp's first one
    bool alive = warp < np && !(p.debug_skip & 1u);  // (test hook: producers that load nothing)
    // a pair counts the bytes of both CTAs on the leader's barrier
    const uint32_t full0 = PAIR ? ptx::map_to_cta(ptx::smem_u32(&full_bar[0]), 0u) : 0u;
    for (int tile = tile_first; alive && tile < p.num_tiles; tile += tile_step) {
      int z, rest;
      if (cluster) {  // slices of a tile sit side by side in one cluster
        rest = p.fd_cluster.div(tile);
        z = tile - rest * p.cluster_split;
      } else {
        z = p.fd_tiles_mn.div(tile);
        rest = tile - z * tiles_mn;
      }
      const int m_blk = p.fd_tiles_n.div(rest);
      const int n0 = (rest - m_blk * p.tiles_n) * BN;
      // A pair's tile is 256 pixels, this CTA's half starts at pixel m0.  The peer of a trailing tile may own no pixel
      // at all: it still loads a full box (from pixel 0; the rows are never stored) so that the byte count is the same.
      int m0 = PAIR ? m_blk * (2 * kTileM) + int(pair_rank) * kTileM : m_blk * (kTileM * MH);
      if (PAIR && m0 >= p.m_total) m0 = 0;
      const int halves = (MH == 2 && m0 + kTileM < p.m_total) ? 2 : 1;  // a trailing tile may own one half only
      const int kb_begin = z * p.kb_per_split;
      const int num_kb = min(p.total_kb, kb_begin + p.kb_per_split) - kb_begin;
      // this lane's activation box: a 128-pixel half (modes 0, 1) or a 64-pixel box of one image (mode 2)
      const int nbox = p.a_mode == 2 ? 2 * halves : halves;
      uint32_t a_off;
      int c1, c2, c3;  // box coordinates besides the channel coordinate
      if (p.a_mode == 3) {
        // one 128-row box per output row of an image; its operand is the strip of positions of ONE input row per slab
        const int box = (m0 >> 7) + lane;
        c3 = p.fd_out_h.div(box);                                    // image
        c2 = (box - c3 * p.out_h) * p.stride_h - p.pad_h;           // topmost input row of that output row
        c1 = 0;
        a_off = uint32_t(lane) * A_HALF_BYTES;
      } else if (p.a_mode == 2) {
        const int box = (m0 >> 6) + lane;
        c3 = p.fd_boxes.div(box);                        // image
        c1 = (box - c3 * p.boxes_per_image) << 6;       // first pixel
        c2 = 0;
        a_off = uint32_t(lane) * (A_HALF_BYTES / 2);
      } else {
        const int mh = m0 + lane * kTileM;
        c3 = p.fd_pq.div(mh);                            // image
        const int rem = mh - c3 * p.pq;
        const int p0 = p.fd_out_w.div(rem);
        c1 = (rem - p0 * p.out_w) * p.stride_w - p.pad_w;  // leftmost input column of the first pixel
        c2 = p0 * p.stride_h - p.pad_h;                    // topmost input row
        if (p.a_mode == 1) c1 = mh;                        // row of the pixel matrix
        a_off = uint32_t(lane) * A_HALF_BYTES;
      }
      // filter tap (r, sx), channel block cb and weight column k0 of this warp's first slab in the tile
      int tap = p.fd_kb_per_tap.div(kb_begin + skip);
      int cb = kb_begin + skip - tap * p.kb_per_tap;
      int r = p.fd_kernel_w.div(tap);
      int sx = tap - r * p.kernel_w;
      int k0 = tap * p.c_padded;
      const uint32_t tx_bytes = PAIR ? 2u * (A_HALF_BYTES + B_BYTES)
                                     : uint32_t(halves) * (p.a_mode == 3 ? uint32_t(p.strip_bytes) : A_HALF_BYTES) + B_BYTES;
      const int wrow0 = n0 + int(pair_rank) * B_ROWS;  // first weight row (output channel) this CTA loads
      int i = skip;
      join_setup();
      for (; i < num_kb; i += np) {
        const bool ok = ptx::mbar_wait(&empty_bar[s], phase ^ 1u, p.status, kStatusProducerTimeout, p.wait_limit);
        if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
        uint8_t* a_dst = stage_base + size_t(s) * STAGE_BYTES;
        if (lane == 0 && leader) ptx::mbar_arrive_expect_tx(&full_bar[s], tx_bytes);
        __syncwarp();
        if constexpr (PAIR) {
          const uint32_t fb = full0 + uint32_t(s) * 8u;  // the leader's full barrier of this slot
          if (lane < nbox) {
            if (p.a_mode == 2) ptx::tma_load_3d_pair(a_dst + a_off, &tm_act, fb, c1, ch(cb * BK), c3);
            else if (p.a_mode == 1) ptx::tma_load_2d_pair(a_dst + a_off, &tm_act, fb, ch(cb * BK), c1);
            else ptx::tma_load_im2col_4d_pair(a_dst + a_off, &tm_act, fb, ch(cb * BK), c1, c2, c3, uint16_t(sx), uint16_t(r));
          }
          if (lane == 0) ptx::tma_load_2d_pair(a_dst + A_BYTES, &tm_wgt, fb, ch(k0 + cb * BK), wrow0);
        } else {
          if (lane < nbox) {
            if (p.a_mode == 3) {
              ptx::tma_load_4d(a_dst + a_off, &tm_act, &full_bar[s], 0, 0, c2 + r, c3);   // positions 0.. of input row c2 + r
            } else if (p.a_mode == 2) {
              // 64 pixels x BK channels, [channel][pixel] in shared memory
              ptx::tma_load_3d(a_dst + a_off, &tm_act, &full_bar[s], c1, ch(cb * BK), c3);
            } else if (p.a_mode == 1) {
              ptx::tma_load_2d(a_dst + a_off, &tm_act, &full_bar[s], ch(cb * BK), c1);
            } else {
              ptx::tma_load_im2col_4d(a_dst + a_off, &tm_act, &full_bar[s], ch(cb * BK), c1, c2, c3, uint16_t(sx), uint16_t(r));
            }
          }
          if (lane == 0) ptx::tma_load_2d(a_dst + A_BYTES, &tm_wgt, &full_bar[s], ch(k0 + cb * BK), n0);
        }
        cb += np;
        while (cb >= p.kb_per_tap) {
          cb -= p.kb_per_tap;
          k0 += p.c_padded;
          if (++sx == p.kernel_w) { sx = 0; ++r; }
        }
        s += np;
        while (s >= stages) { s -= stages; phase ^= 1u; }
      }
      skip = i - num_kb;  // how far this warp's next slab lies into the next tile
    }
    join_setup();  // warps without a slab of their own
    if (cluster) {  // the two cluster barriers of the epilogue's reduction count every thread
      ptx::cluster_sync_all();
      ptx::cluster_sync_all();
    }
  } else if (warp == kProducerWarps) {
    // ---------------- MMA issuer ----------------
    // The warp stays converged (all lanes wait and compute the descriptors); one elected lane issues the MMAs and
    // the commits.  A single diverged lane pays markedly more issue latency per tcgen05.mma than an elected lane
    // of a converged warp, enough to make 128-column tiles issue-bound.
    int s = 0, tcount = 0;
    uint32_t phase = 0;
    if (p.debug_skip & 2u) join_setup();  // (test hook: an issuer that does nothing, not even signal the epilogue)
    bool alive = leader && !(p.debug_skip & 2u);  // the peer CTA of a pair issues nothing: the leader's instructions drive both tensor cores
    for (int tile = tile_first; alive && tile < p.num_tiles; tile += tile_step, ++tcount) {
      int z, rest;
      if (cluster) {  // slices of a tile sit side by side in one cluster
        rest = p.fd_cluster.div(tile);
        z = tile - rest * p.cluster_split;
      } else {
        z = p.fd_tiles_mn.div(tile);
        rest = tile - z * tiles_mn;
      }
      const int m0 = p.fd_tiles_n.div(rest) * (kTileM * MH);
      const int halves = (MH == 2 && m0 + kTileM < p.m_total) ? 2 : 1;  // (a pair always computes both of its halves)
      const int kb_begin = z * p.kb_per_split;
      const int num_kb = min(p.total_kb, kb_begin + p.kb_per_split) - kb_begin;
      const int buf = ACC_BUFS == 2 ? (tcount & 1) : 0;
      const uint32_t acc_phase = (ACC_BUFS == 2 ? (tcount >> 1) : tcount) & 1;
      join_setup();
      // the epilogue must have drained this accumulator set (first use passes at once)
      const bool drained = ptx::mbar_wait(&acc_empty[buf], acc_phase ^ 1u, p.status, kStatusMmaTimeout, p.wait_limit);
      if (!__all_sync(0xffffffffu, drained)) break;
      ptx::tc_fence_after_sync();
      const uint32_t acc = tmem_base + buf * ACC_COLS;
      // The slab loop exists three times (16-bit K-major A, 16-bit pixel-major A, TF32): the operand form and the MMA
      // kind are compile-time inside it, so the elected lane's issue sequence carries no branch per instruction.
      auto slab_loop = [&](auto form_tag) {
        constexpr int FORM = decltype(form_tag)::value;  // 0: kind::f16, K-major A; 1: kind::f16, pixel-major A; 2: kind::tf32; 3: kind::f8f6f4 (E4M3); 4: kind::f16, A = overlapping windows of an unswizzled strip
        // one slab's MMAs and the commit that frees its ring slot (elected lane only)
        auto issue_slab = [&](int slot, bool first) {
          const uint32_t a_addr = ptx::smem_u32(stage_base + size_t(slot) * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
          if constexpr (SWAP) {
            // A = 128 weight rows (output channels), B = all MH * 128 activation rows (pixels) of the slab
#pragma unroll
            for (int hc = 0; hc < BN / 128; ++hc) {
#pragma unroll
              for (int k = 0; k < MMAS_PER_SLAB; ++k) {
                const uint64_t wdesc = ptx::smem_desc_kmajor<ROW_BYTES>(b_addr + hc * (128 * ROW_BYTES) + k * 32);
                const uint64_t xdesc = FORM == 1 ? ptx::smem_desc_mnmajor_sw128(a_addr + k * 2048, A_HALF_BYTES / 2, 1024)
                                                 : ptx::smem_desc_kmajor<ROW_BYTES>(a_addr + k * 32);
                ptx::mma_f16_ss(acc + hc * (MH * 128), wdesc, xdesc, p.idesc, !first || k != 0);
              }
            }
          } else {
#pragma unroll
          for (int h = 0; h < MH; ++h) {
            if (h < halves) {
#pragma unroll
              for (int k = 0; k < MMAS_PER_SLAB; ++k) {
                // K-major A: one MMA's K extent (16 two-byte or 8 four-byte values) = 32 bytes along a row.
                // Pixel-major A (form 1): 16 channels = 16 rows of 128 B.
                const uint64_t adesc = FORM == 1   ? ptx::smem_desc_mnmajor_sw128(a_addr + h * A_HALF_BYTES + k * 2048, A_HALF_BYTES / 2, 1024)
                                       : FORM == 4 ? ptx::smem_desc_kmajor_plain(a_addr + h * A_HALF_BYTES + k * 32, 16, 128)
                                                   : ptx::smem_desc_kmajor<ROW_BYTES>(a_addr + h * A_HALF_BYTES + k * 32);
                const uint64_t bdesc = ptx::smem_desc_kmajor<ROW_BYTES>(b_addr + k * 32);
                if constexpr (PAIR && FORM == 3) ptx::mma_f8_ss_pair(acc, adesc, bdesc, p.idesc, !first || k != 0);
                else if constexpr (PAIR) ptx::mma_f16_ss_pair(acc, adesc, bdesc, p.idesc, !first || k != 0);
                else if constexpr (FORM == 2) ptx::mma_tf32_ss(acc + h * BN, adesc, bdesc, p.idesc, !first || k != 0);
                else if constexpr (FORM == 3) ptx::mma_f8_ss(acc + h * BN, adesc, bdesc, p.idesc, !first || k != 0);
                else ptx::mma_f16_ss(acc + h * BN, adesc, bdesc, p.idesc, !first || k != 0);
              }
            }
          }
          }
          // frees the slot (in both CTAs of a pair) once these MMAs have read it
          if constexpr (PAIR) ptx::mma_commit_pair(&empty_bar[slot], 3);
          else ptx::mma_commit(&empty_bar[slot]);
        };
        for (int i = 0; i < num_kb;) {
          const bool ok = ptx::mbar_wait(&full_bar[s], phase, p.status, kStatusMmaTimeout, p.wait_limit);
          if (!__all_sync(0xffffffffu, ok)) { alive = false; break; }
          // When the next slab has landed as well (the issue, not the feed, is the bottleneck), both go out in one
          // elected block: the wait / vote / fence sequence between slabs costs as much as three MMA issues.
          const int s2 = s + 1 == stages ? 0 : s + 1;
          const uint32_t phase2 = s + 1 == stages ? phase ^ 1u : phase;
          const bool two = PAIR_SLABS && i + 1 < num_kb && __all_sync(0xffffffffu, ptx::mbar_try_wait(&full_bar[s2], phase2));
          ptx::tc_fence_after_sync();
          if (ptx::elect_one()) {
            issue_slab(s, i == 0);
            if (two) issue_slab(s2, false);
          }
          __syncwarp();
          const int adv = two ? 2 : 1;
          i += adv;
          s += adv;
          if (s >= stages) { s -= stages; phase ^= 1u; }
        }
      };
      if (!PAIR && !SWAP && p.is_tf32) slab_loop(std::integral_constant<int, 2>{});
      else if (!SWAP && p.is_fp8) slab_loop(std::integral_constant<int, 3>{});
      else if (p.a_mode == 2) slab_loop(std::integral_constant<int, 1>{});
      else if (!PAIR && !SWAP && p.a_mode == 3) slab_loop(std::integral_constant<int, 4>{});
      else slab_loop(std::integral_constant<int, 0>{});
      // accumulator set complete (also reached after a time-out in the slab loop, so nobody hangs)
      if (ptx::elect_one()) {
        if constexpr (PAIR) ptx::mma_commit_pair(&acc_full[buf], 3);  // wakes the epilogue warps of both CTAs
        else ptx::mma_commit(&acc_full[buf]);
      }
      __syncwarp();
    }
    join_setup();  // the peer CTA's warp joins here (a no-op for a warp that had a tile)
    if (cluster) {
      ptx::cluster_sync_all();
      ptx::cluster_sync_all();
    }
  } else {
    // ---------------- epilogue: EW = 8 or 16 warps.  Warp w may read TMEM lanes 32*(w%4)..+31; the EW / 4 warps of a lane
    // quarter take the 32-column chunks of a tile in turn (several warps per scheduler hide each other's latencies).
    const int quad = warp & 3;
    const int par = (warp - kProducerWarps - 1) >> 2;  // 0 .. EG-1: which chunks this warp owns
    const int et = threadIdx.x - 32 * (kProducerWarps + 1);  // index among the epilogue threads
    const int we = warp - kProducerWarps - 1;                // index among the epilogue warps
    uint32_t res_phase = 0;                                  // bit k: parity of this warp's residual barrier k (TMA epilogue)
    // GEMM row -> (image, pixel within the image, row holds an output pixel at all)
    auto decode_row = [&](int m, bool& m_ok, int& img, int& pix) {
      m_ok = m < p.m_total;
      img = pix = 0;
      if (p.a_mode == 3) {  // rows are numbered in 128-row boxes per output row
        const int box = m >> 7, q = m & 127;
        img = p.fd_out_h.div(box);
        pix = (box - img * p.out_h) * p.out_w + q;
        m_ok = m_ok && q < p.out_w;
        if (!m_ok) img = pix = 0;
      } else if (p.a_mode == 2) {  // rows are numbered in 64-pixel boxes per image
        const int box = m >> 6;
        img = p.fd_boxes.div(box);
        pix = ((box - img * p.boxes_per_image) << 6) + (m & 63);
        m_ok = m_ok && pix < p.pq;
        if (!m_ok) img = pix = 0;
      } else if (m_ok) {
        img = p.fd_pq.div(m);
        pix = m - img * p.pq;
      }
    };
    int tcount = 0;
    const uint32_t acc_empty0 = PAIR ? ptx::map_to_cta(ptx::smem_u32(&acc_empty[0]), 0u) : 0u;  // the leader's barriers
    for (int tile = tile_first; tile < p.num_tiles; tile += tile_step, ++tcount) {
      int z, rest;
      if (cluster) {  // slices of a tile sit side by side in one cluster
        rest = p.fd_cluster.div(tile);
        z = tile - rest * p.cluster_split;
      } else {
        z = p.fd_tiles_mn.div(tile);
        rest = tile - z * tiles_mn;
      }
      const int m_blk = p.fd_tiles_n.div(rest);
      const int n0 = (rest - m_blk * p.tiles_n) * BN;
      // first pixel row this CTA holds in its tensor memory (a pair: the leader the first 128 of the tile, the peer the rest)
      const int m0 = PAIR ? m_blk * (2 * kTileM) + int(pair_rank) * kTileM : m_blk * (kTileM * MH);
      const int halves = (MH == 2 && m0 + kTileM < p.m_total) ? 2 : 1;
      const int buf = tcount % ACC_BUFS;
      const uint32_t acc_phase = (tcount / ACC_BUFS) & 1;
      float* bias_t = bias_s + (tcount & 1) * 256;

      join_setup();
      // stage this tile's bias as float (two buffers: a fast warp may already be one tile ahead of a slow one)
      for (int i = et; i < BN; i += 32 * EW) {
        const int oc = n0 + i;
        float b = 0.f;
        if (p.has_bias && p.partial == nullptr && oc < p.out_channels) {
          if (p.bias_fp32) b = static_cast<const float*>(p.bias)[oc];
          else if (p.is_bf16) b = __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[oc]);
          else b = __half2float(static_cast<const __half*>(p.bias)[oc]);
        }
        bias_t[i] = b;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(32 * EW) : "memory");  // epilogue warps only

      // TMA epilogue (channel-contiguous output): this warp's chunk c of half h is staged in its own 2 KiB box and
      // leaves as one TMA store; with a residual, TMA first loads the residual box into the same place, issued here
      // (before the accumulator is even complete) so that the load overlaps the main loop.
      auto stage_box = [&](int k) { return epi_base + size_t(we * kEpiBufs + k) * 2048; };
      auto prefetch_residual = [&](int h) {
        if (lane == 0) ptx::bulk_wait_group_read0();  // earlier stores of this warp have left the boxes
        __syncwarp();
        if (p.res_tma && lane == 0) {
          for (int k = 0; k < kEpiBufs; ++k) {
            const int chunk = par + EG * k;
            if (chunk >= BN / 32 || n0 + chunk * 32 >= p.out_channels) break;
            ptx::mbar_arrive_expect_tx(&res_bar[we * kEpiBufs + k], 2048);
            ptx::tma_load_2d(stage_box(k), &tm_res, &res_bar[we * kEpiBufs + k], n0 + chunk * 32, m0 + h * kTileM + quad * 32);
          }
        }
      };
      if (p.out_tma) prefetch_residual(0);

      // Row decode and output addresses, done while the main loop still runs (the accumulator is not needed for them).
      const int64_t cstride = p.out_nhwc ? 1 : p.pq;
      bool m_ok_h[MH];
      int64_t base_h[MH];
#pragma unroll
      for (int h = 0; h < MH; ++h) {
        int img, pix;
        decode_row(m0 + h * kTileM + quad * 32 + lane, m_ok_h[h], img, pix);
        base_h[h] = p.out_nhwc ? (int64_t(img) * p.pq + pix) * p.out_channels + n0 : (int64_t(img) * p.out_channels + n0) * p.pq + pix;
      }

      // A residual in NCHW layout is read by plain loads, eight channels at a time: too few bytes in flight to pull a large
      // tensor from HBM.  Its lines start their way into L2 now, while the main loop of this tile still runs: lane j asks
      // for the run of channel j of every chunk this warp owns (from the warp's first and last pixel: the 32 pixels may
      // lie in two images).
      if (!SWAP && p.residual != nullptr && !p.out_nhwc && !p.out_tma) {
        const int esz = p.is_tf32 ? 4 : 2;
        const uint8_t* rb = static_cast<const uint8_t*>(p.residual);
#pragma unroll
        for (int h = 0; h < MH; ++h) {
          if (h >= halves) break;
          const int64_t b_first = __shfl_sync(0xffffffffu, base_h[h], 0), b_last = __shfl_sync(0xffffffffu, base_h[h], 31);
          const bool ok_first = __shfl_sync(0xffffffffu, int(m_ok_h[h]), 0) != 0, ok_last = __shfl_sync(0xffffffffu, int(m_ok_h[h]), 31) != 0;
          for (int chunk = par; chunk < BN / 32; chunk += EG) {
            const int ch = chunk * 32 + lane;
            if (n0 + ch >= p.out_channels) break;
            if (ok_first) ptx::prefetch_l2(rb + (b_first + int64_t(ch) * cstride) * esz);
            if (ok_last) ptx::prefetch_l2(rb + (b_last + int64_t(ch) * cstride) * esz);
          }
        }
      }

      const bool ok = ptx::mbar_wait(&acc_full[buf], acc_phase, p.status, kStatusEpilogueTimeout, p.wait_limit);
      __syncwarp();
      ptx::tc_fence_after_sync();
      if (!__all_sync(0xffffffffu, ok)) {
        if (cluster) {  // keep the cluster's barriers balanced so that the peers can leave as well
          ptx::cluster_sync_all();
          ptx::cluster_sync_all();
        }
        break;
      }
      const uint32_t acc = tmem_base + buf * ACC_COLS;
      if (cluster) {
        // Split-K inside a cluster (MH = 1, one tile per CTA).  CTA `rank` holds the partial sums of K-slice `rank`
        // for the whole tile and owns the 32-column chunks [rank * cpr, (rank + 1) * cpr): every CTA pushes the
        // chunks it does not own into the owner's (now idle) operand ring through distributed shared memory, then
        // each owner adds the received slices to its own in a fixed order (results are run-to-run identical), applies
        // bias + ReLU and stores.  Receive layout: [sender slot][chunk][group of 4 columns][row][16 bytes]: one warp
        // instruction writes (and later reads) 512 contiguous bytes.
        const int nsplit = p.cluster_split;
        const int rank = int(ptx::cluster_ctarank());
        const int cpr = (BN / 32) / nsplit;  // chunks per owner
        const int row = quad * 32 + lane;
        const uint32_t recv = ptx::smem_u32(stage_base);
        ptx::cluster_sync_all();  // every CTA of the cluster has finished its MMAs: all rings are idle
        for (int chunk = par; chunk < BN / 32; chunk += EG) {
          if (n0 + chunk * 32 >= p.out_channels) break;  // warp-uniform, same in every CTA of the cluster
          const int owner = chunk / cpr;
          if (owner == rank) continue;
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(acc + (uint32_t(quad * 32) << 16) + uint32_t(chunk * 32), v);
          ptx::tmem_ld_wait();
          const int slot = rank < owner ? rank : rank - 1;
          const uint32_t dst = ptx::map_to_cta(recv + uint32_t((slot * cpr + (chunk - owner * cpr)) * (kTileM * 128) + row * 16), uint32_t(owner));
#pragma unroll
          for (int g = 0; g < 8; ++g)
            ptx::st_cluster_v4(dst + uint32_t(g * (kTileM * 16)), v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
        }
        ptx::cluster_sync_all();  // all pushes have landed
        const int m = m0 + row;
        bool m_ok;
        int img, pix;
        decode_row(m, m_ok, img, pix);
        // element offset of (this row, channel n0) and the distance between consecutive channels
        const int64_t base = p.out_nhwc ? (int64_t(img) * p.pq + pix) * p.out_channels + n0
                                        : (int64_t(img) * p.out_channels + n0) * p.pq + pix;
        for (int chunk = par; chunk < BN / 32; chunk += EG) {
          if (n0 + chunk * 32 >= p.out_channels) break;
          if (chunk / cpr != rank) continue;
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(acc + (uint32_t(quad * 32) << 16) + uint32_t(chunk * 32), v);
          ptx::tmem_ld_wait();
          const uint8_t* src0 = stage_base + size_t(chunk - rank * cpr) * (kTileM * 128) + row * 16;
          for (int slot = 0; slot < nsplit - 1; ++slot) {  // own slice first, then the others in a fixed order
            const uint8_t* src = src0 + size_t(slot) * cpr * (kTileM * 128);
#pragma unroll
            for (int gh = 0; gh < 2; ++gh) {  // 4 independent 16-byte loads in flight, then their adds
              float4 q[4];
#pragma unroll
              for (int g = 0; g < 4; ++g) q[g] = *reinterpret_cast<const float4*>(src + (gh * 4 + g) * (kTileM * 16));
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                const int j = (gh * 4 + g) * 4;
                v[j] = __float_as_uint(__uint_as_float(v[j]) + q[g].x);
                v[j + 1] = __float_as_uint(__uint_as_float(v[j + 1]) + q[g].y);
                v[j + 2] = __float_as_uint(__uint_as_float(v[j + 2]) + q[g].z);
                v[j + 3] = __float_as_uint(__uint_as_float(v[j + 3]) + q[g].w);
              }
            }
          }
          if (m_ok) {
            const int nvalid = min(32, p.out_channels - (n0 + chunk * 32));
            const int64_t off = base + int64_t(chunk * 32) * cstride;
            with_output_type(p, [&](auto* yp, auto* rp) {
              store_chunk(v, bias_t + chunk * 32, yp + off, rp ? rp + off : nullptr, cstride, nvalid, p.relu);
            });
          }
        }
        break;  // one tile per CTA in this mode
      }
      if constexpr (SWAP) {
        // Transposed accumulator: lane = output channel, 32 columns = 32 consecutive pixels.  Work units = (128-channel
        // half, 32-pixel column chunk); the EG warps of a lane quarter take them in turn.  A unit is rounded and written
        // into the warp's staging box as 32 rows (channels) of 64 bytes, 64-byte swizzled (16-byte cell q of row r at
        // cell q ^ ((r >> 1) & 3): conflict-free), and leaves as ONE TMA store when its pixels lie in one image;
        // otherwise (the unit crosses into the next image, or y is not 16-byte aligned) the lanes read the box back as
        // runs of out_vec pixels and store them.
        constexpr int PC = MH * 4;                 // 32-pixel chunks per channel half
        constexpr int UNITS = (BN / 128) * PC;
        uint8_t* box = epi_base + size_t(we) * 2048;
        // fallback geometry: lane owns the pixel group g of rows r0, r0 + rstep, ...
        const int vec = p.out_vec;                                   // 4, 2 or 1 pixels per store
        const int gsh = vec == 4 ? 3 : (vec == 2 ? 4 : 5);           // log2(groups per row)
        const int g = lane & ((1 << gsh) - 1), r0 = lane >> gsh, rstep = 32 >> gsh;
#pragma unroll 1
        for (int u = par; u < UNITS; u += EG) {
          const int hc = u / PC, pc = u - hc * PC;
          const int ch0 = n0 + hc * 128 + quad * 32;                 // channel of lane 0
          const int mstart = m0 + pc * 32;                           // first pixel row of the unit
          if (ch0 >= p.out_channels || mstart >= p.m_total) continue;  // warp-uniform
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(acc + (uint32_t(quad * 32) << 16) + uint32_t(hc * (MH * 128) + pc * 32), v);
          // Fused residual (same NCHW layout as the output): this lane's channel, four groups of 8 consecutive pixels.  A
          // group never straddles an image (P*Q % 8 == 0); its address is decoded on its own because a unit may.  The
          // loads are in flight while the tensor-memory load completes.
          uint4 rr[4];
          const bool with_res = p.residual != nullptr;
          if (with_res) {
            const uint8_t* rb = static_cast<const uint8_t*>(p.residual);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              bool q_ok;
              int qimg, qpix;
              decode_row(mstart + q * 8, q_ok, qimg, qpix);
              rr[q] = make_uint4(0u, 0u, 0u, 0u);
              if (q_ok && ch0 + lane < p.out_channels) {
                const uint8_t* src = rb + ((int64_t(qimg) * p.out_channels + ch0 + lane) * p.pq + qpix) * 2;
                if (p.res_vec) rr[q] = *reinterpret_cast<const uint4*>(src);
                else {  // residual not 16-byte aligned: element by element
                  const uint16_t* s16 = reinterpret_cast<const uint16_t*>(src);
                  rr[q] = make_uint4(uint32_t(s16[0]) | (uint32_t(s16[1]) << 16), uint32_t(s16[2]) | (uint32_t(s16[3]) << 16),
                                     uint32_t(s16[4]) | (uint32_t(s16[5]) << 16), uint32_t(s16[6]) | (uint32_t(s16[7]) << 16));
                }
              }
            }
          }
          ptx::tmem_ld_wait();
          const float bv = bias_t[hc * 128 + quad * 32 + lane];
          if (lane == 0) ptx::bulk_wait_group_read0();  // the previous store of this warp has left the box
          __syncwarp();
          const bool relu = p.relu != 0;
          if (p.is_bf16) {
            if (with_res) row_to_staging<__nv_bfloat16, true>(v, bv, rr, relu, box, lane);
            else row_to_staging<__nv_bfloat16, false>(v, bv, rr, relu, box, lane);
          } else {
            if (with_res) row_to_staging<__half, true>(v, bv, rr, relu, box, lane);
            else row_to_staging<__half, false>(v, bv, rr, relu, box, lane);
          }
          bool u_ok;
          int img, pix0;
          decode_row(mstart, u_ok, img, pix0);
          // one image holds the whole unit (rows numbered in 64-pixel boxes never leave their image: the map clips the tail)
          const bool whole = p.swap_tma && u_ok && (p.a_mode == 2 || pix0 + 32 <= p.pq);
          if (whole) {
            ptx::fence_proxy_async_smem();  // generic-proxy writes above -> visible to the TMA store below
            __syncwarp();
            if (lane == 0) {
              ptx::tma_store_3d(&tm_out, box, pix0, ch0, img);  // channels beyond O are clipped by the tensor map
              ptx::bulk_commit_group();
            }
          } else {
            __syncwarp();
            bool g_ok;
            int gimg, gpix;
            decode_row(mstart + g * vec, g_ok, gimg, gpix);  // a group never straddles an image (P*Q % vec == 0)
            const int64_t gb = (int64_t(gimg) * p.out_channels + ch0) * p.pq + gpix;
            uint8_t* yb = static_cast<uint8_t*>(p.y);
            for (int row = r0; row < 32; row += rstep) {
              if (!g_ok || ch0 + row >= p.out_channels) continue;
              const int byte = g * vec * 2;  // offset of the group inside the 64-byte row
              const uint8_t* src = box + row * 64 + (((byte >> 4) ^ ((row >> 1) & 3)) << 4) + (byte & 15);
              uint8_t* dst = yb + (gb + int64_t(row) * p.pq) * 2;
              if (vec == 4) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(src);
              else if (vec == 2) *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(src);
              else *reinterpret_cast<uint16_t*>(dst) = *reinterpret_cast<const uint16_t*>(src);
            }
            __syncwarp();
          }
        }
      } else {
      float* part = p.partial ? p.partial + int64_t(z) * ((p.y_elems + 3) & ~int64_t(3)) : nullptr;
#pragma unroll
      for (int h = 0; h < MH; ++h) {
        if (h >= halves) break;
        const bool m_ok = m_ok_h[h];
        const int64_t base = base_h[h];
        if (p.out_tma && h > 0) prefetch_residual(h);
#pragma unroll 1
        for (int chunk = par; chunk < BN / 32; chunk += EG) {
          if (n0 + chunk * 32 >= p.out_channels) break;  // warp-uniform
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(acc + (uint32_t(quad * 32) << 16) + uint32_t(h * BN + chunk * 32), v);
          ptx::tmem_ld_wait();
          if (p.out_tma) {
            const int k = chunk / EG;
            uint8_t* box = stage_box(k);
            bool landed = true;
            if (p.res_tma) {
              landed = ptx::mbar_wait(&res_bar[we * kEpiBufs + k], (res_phase >> k) & 1u, p.status, kStatusEpilogueTimeout, p.wait_limit);
              res_phase ^= 1u << k;  // barrier k has been used once more (a tile at the channel edge skips some)
            }
            if (__all_sync(0xffffffffu, landed)) {
              if (p.is_bf16) chunk_to_staging<__nv_bfloat16>(v, bias_t + chunk * 32, box, lane, p.relu, p.res_tma != 0);
              else chunk_to_staging<__half>(v, bias_t + chunk * 32, box, lane, p.relu, p.res_tma != 0);
              ptx::fence_proxy_async_smem();  // generic-proxy writes above -> visible to the TMA store below
              __syncwarp();
              if (lane == 0) {
                // rows beyond the last pixel and channels beyond O are clipped by the tensor map
                ptx::tma_store_2d(&tm_out, box, n0 + chunk * 32, m0 + h * kTileM + quad * 32);
                ptx::bulk_commit_group();
              }
            }
            continue;
          }
          if (m_ok) {
            const int nvalid = min(32, p.out_channels - (n0 + chunk * 32));
            const int64_t off = base + int64_t(chunk * 32) * cstride;
            if (part) {  // FP32 partials in the output's own element order
              float* dst = part + off;
              if (cstride == 1 && nvalid == 32 && (off & 3) == 0) {
#pragma unroll
                for (int g = 0; g < 8; ++g) reinterpret_cast<uint4*>(dst)[g] = make_uint4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (j < nvalid) dst[int64_t(j) * cstride] = __uint_as_float(v[j]);
              }
            } else {
              with_output_type(p, [&](auto* yp, auto* rp) {
                store_chunk(v, bias_t + chunk * 32, yp + off, rp ? rp + off : nullptr, cstride, nvalid, p.relu);
              });
            }
          }
        }
      }
      }  // !SWAP
      // all TMEM reads of this warp are complete (wait::ld above): hand the accumulator set back to the MMA issuer
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if constexpr (PAIR) ptx::mbar_arrive_cluster(acc_empty0 + uint32_t(buf) * 8u);
        else ptx::mbar_arrive(&acc_empty[buf]);
      }
    }
  }

  if ((p.out_tma || SWAP) && warp > kProducerWarps && lane == 0) ptx::bulk_wait_group0();  // this warp's TMA stores are complete
  join_setup();  // no-op for every warp that had a tile (all of them: the grid never exceeds the tile count)
  ptx::tc_fence_before_sync();
  if constexpr (PAIR) {
    // Neither CTA of a pair may leave (or free tensor memory) while the other can still signal its barriers or while the
    // leader's MMAs can still read its shared memory: both meet here once all their roles have finished.
    ptx::cluster_sync_all();
    if (warp == kProducerWarps) {
      ptx::tc_fence_after_sync();
      ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
  } else {
    __syncthreads();
    if (warp == kProducerWarps) {
      ptx::tc_fence_after_sync();
      ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
  }
}

}  // namespace
}  // namespace gieb
