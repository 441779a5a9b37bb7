// Strict-FP32 convolution (no tensor cores, no TF32): register-blocked SIMT implicit GEMM straight from NCHW with
// the bias + ReLU epilogue fused.  Stands in for implicit_gemm_kernel (src/kernels/implicit_gemm.cu:47-189).
//
// GEMM view: rows = output pixels (b, oh, ow), columns = output channels, k = (c, r, s) in OIHW order so a weight
// row is contiguous in k.  Per CTA: a TP x TO output tile, 4x4 outputs per thread, BK = 16 reduction slab staged in
// shared memory (pixels contiguous in the X slab, so the gather from NCHW is coalesced along ow), next slab
// prefetched into registers while the current one is consumed.  Accumulation is fmaf in k order.
#include <stdint.h>

#include "internal.h"

namespace gieb {
namespace {

constexpr int kBK = 16;
constexpr int kLutMax = 2048;  // reduction length up to which the (c, r, s) decode of k is tabulated in shared memory

struct Fp32Args {
  const float* x;
  const float* w;
  const float* bias;
  float* y;
  int batch, c, h, wd, o, r, s, stride_h, stride_w, pad_h, pad_w, out_h, out_w, relu;
  int pixels;  // batch * out_h * out_w
  int k;       // c * r * s
  FastDiv fd_rs, fd_s, fd_pq, fd_out_w;  // multiply-high reciprocals of r*s, s, out_h*out_w, out_w
};

// KG = number of thread groups that split the reduction inside one CTA (slab s goes to group s % KG); their partial
// accumulators are summed in a fixed order at the end, so results are deterministic.  KG > 1 gives small problems
// (few CTAs, long dependent slab chains) enough warps per SM to hide global-load latency.
// LUT: k -> (offset of (c, r, s) inside one image, r, s) comes from a table built once per CTA (the analogue of
// build_conv_lut, src/kernels/conv_common.cu:25-37) instead of two divisions per gathered element: the gather is
// instruction-bound, and the table cuts a load from ~30 to ~10 instructions.
template <int TP, int TO, int KG, bool LUT>
__global__ void __launch_bounds__((TP / 4) * (TO / 4) * KG)
conv_fp32_kernel(const Fp32Args a) {
  constexpr int NT = (TP / 4) * (TO / 4);  // threads per group
  constexpr int XE = kBK * TP / NT;        // X-slab elements loaded per thread
  constexpr int WE = kBK * TO / NT;        // W-slab elements loaded per thread
  constexpr int XS_FLOATS = KG * kBK * TP, WS_FLOATS = KG * kBK * (TO + 4);
  __shared__ __align__(16) float tiles[XS_FLOATS + WS_FLOATS];  // operand tiles; reused for the group reduction
  float (*xs)[kBK][TP] = reinterpret_cast<float (*)[kBK][TP]>(tiles);
  float (*ws)[kBK][TO + 4] = reinterpret_cast<float (*)[kBK][TO + 4]>(tiles + XS_FLOATS);
  __shared__ int2 lut[LUT ? kLutMax : 1];

  const int grp = threadIdx.x / NT;
  const int t = threadIdx.x - grp * NT;
  const int tx = t % (TP / 4), ty = t / (TP / 4);
  const int pix0 = blockIdx.x * TP, oc0 = blockIdx.y * TO;
  const int rs = a.r * a.s;
  const int pq = a.out_h * a.out_w;

  // Loader roles. X: thread owns pixel (t % TP) and slab rows (t / TP) + i * (NT / TP).
  const int lp = t % TP;
  const int lpix = pix0 + lp;
  const bool lp_ok = lpix < a.pixels;
  int ih0 = 0, iw0 = 0;
  const float* xb = a.x;
  if (lp_ok) {
    const int b = a.fd_pq.div(lpix), rem = lpix - b * pq;
    const int oh = a.fd_out_w.div(rem), ow = rem - oh * a.out_w;
    ih0 = oh * a.stride_h - a.pad_h;
    iw0 = ow * a.stride_w - a.pad_w;
    xb = a.x + size_t(b) * a.c * a.h * a.wd;
  }
  const int xoff0 = ih0 * a.wd + iw0;  // offset of tap (0, 0) of this pixel inside a channel plane (may be negative)
  if (LUT) {
    const int kend = (a.k + kBK * KG - 1) / (kBK * KG) * (kBK * KG);  // slabs beyond K read zeros
    for (int k = threadIdx.x; k < kend; k += NT * KG) {
      int2 e = make_int2(0, 0x7fff0000);  // r far outside every image: never loaded
      if (k < a.k) {
        const int c = a.fd_rs.div(k), q = k - c * rs;
        const int r = a.fd_s.div(q), sx = q - r * a.s;
        e = make_int2((c * a.h + r) * a.wd + sx, (r << 16) | sx);
      }
      lut[k] = e;
    }
    __syncthreads();
  }
  // W: thread owns k offset (t % kBK) and channels (t / kBK) + i * (NT / kBK)  -> coalesced along k.
  const int wk = t % kBK;

  float xr[XE], wr[WE];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < XE; ++i) {
      const int kk = t / TP + i * (NT / TP);
      const int k = k0 + kk;
      float v = 0.f;
      if (LUT) {
        const int2 e = lut[k];
        const int ih = ih0 + (e.y >> 16), iw = iw0 + (e.y & 0xffff);
        if (lp_ok && unsigned(ih) < unsigned(a.h) && unsigned(iw) < unsigned(a.wd)) v = __ldg(xb + (e.x + xoff0));
      } else if (lp_ok && k < a.k) {
        const int c = a.fd_rs.div(k), q = k - c * rs;
        const int r = a.fd_s.div(q), s = q - r * a.s;
        const int ih = ih0 + r, iw = iw0 + s;
        if (ih >= 0 && ih < a.h && iw >= 0 && iw < a.wd) v = __ldg(xb + (size_t(c) * a.h + ih) * a.wd + iw);
      }
      xr[i] = v;
    }
#pragma unroll
    for (int i = 0; i < WE; ++i) {
      const int oc = oc0 + t / kBK + i * (NT / kBK);
      const int k = k0 + wk;
      wr[i] = (oc < a.o && k < a.k) ? __ldg(a.w + size_t(oc) * a.k + k) : 0.f;
    }
  };
  auto stash = [&]() {
#pragma unroll
    for (int i = 0; i < XE; ++i) xs[grp][t / TP + i * (NT / TP)][lp] = xr[i];
#pragma unroll
    for (int i = 0; i < WE; ++i) ws[grp][wk][t / kBK + i * (NT / kBK)] = wr[i];
  };

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // every group runs the same number of rounds (slabs beyond K load zeros), so the barriers stay uniform
  const int rounds = (a.k + kBK * KG - 1) / (kBK * KG);
  fetch(grp * kBK);
  for (int rd = 0; rd < rounds; ++rd) {
    stash();
    __syncthreads();
    if (rd + 1 < rounds) fetch(((rd + 1) * KG + grp) * kBK);
#pragma unroll
    for (int kk = 0; kk < kBK; ++kk) {
      const float4 xv = *reinterpret_cast<const float4*>(&xs[grp][kk][tx * 4]);
      const float4 wv = *reinterpret_cast<const float4*>(&ws[grp][kk][ty * 4]);
      const float xa[4] = {xv.x, xv.y, xv.z, xv.w};
      const float wa[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xa[i], wa[j], acc[i][j]);
    }
    __syncthreads();
  }

  if (KG > 1) {  // fold groups 1..KG-1 into group 0, in group order (the operand tiles are free now)
    float* red = tiles;
    static_assert(KG == 1 || (KG - 1) * NT * 16 <= XS_FLOATS + WS_FLOATS, "reduction scratch must fit the operand tiles");
    if (grp > 0) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) red[((grp - 1) * 16 + i * 4 + j) * NT + t] = acc[i][j];
    }
    __syncthreads();
    if (grp > 0) return;
    for (int g = 0; g < KG - 1; ++g)
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += red[(g * 16 + i * 4 + j) * NT + t];
  }

  // Epilogue (fused_epilogue.cuh:11-16 order): + bias, ReLU, store.  Pixels are the fast index of NCHW.
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int oc = oc0 + ty * 4 + j;
    if (oc >= a.o) continue;
    const float bv = a.bias ? __ldg(a.bias + oc) : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int pix = pix0 + tx * 4 + i;
      if (pix >= a.pixels) continue;
      const int b = a.fd_pq.div(pix), rem = pix - b * pq;
      float v = acc[i][j] + bv;
      if (a.relu) v = fmaxf(v, 0.f);
      a.y[(size_t(b) * a.o + oc) * pq + rem] = v;
    }
  }
}

bool use_small_tile(int64_t pixels, int o) {
  const int64_t big = ((pixels + 63) / 64) * ((o + 63) / 64);
  return big < 2 * 148;
}

}  // namespace

int conv_fp32_tile(int64_t pixels, int o) { return use_small_tile(pixels, o) ? 32 : 64; }

int64_t conv_fp32_num_blocks(int64_t pixels, int o) {
  return use_small_tile(pixels, o) ? ((pixels + 31) / 32) * ((o + 31) / 32) : ((pixels + 63) / 64) * ((o + 63) / 64);
}

cudaError_t conv_fp32_launch(const void* x, const void* w, const void* bias, void* y, int batch, int c, int h, int wd, int o,
                             int r, int s, int stride_h, int stride_w, int pad_h, int pad_w, int out_h, int out_w, int relu,
                             cudaStream_t stream) {
  Fp32Args a;
  a.x = static_cast<const float*>(x);
  a.w = static_cast<const float*>(w);
  a.bias = static_cast<const float*>(bias);
  a.y = static_cast<float*>(y);
  a.batch = batch; a.c = c; a.h = h; a.wd = wd; a.o = o; a.r = r; a.s = s;
  a.stride_h = stride_h; a.stride_w = stride_w; a.pad_h = pad_h; a.pad_w = pad_w;
  a.out_h = out_h; a.out_w = out_w; a.relu = relu;
  a.pixels = batch * out_h * out_w;
  a.k = c * r * s;
  a.fd_rs = FastDiv::make(r * s);
  a.fd_s = FastDiv::make(s);
  a.fd_pq = FastDiv::make(out_h * out_w);
  a.fd_out_w = FastDiv::make(out_w);
  const bool lut = (a.k + 63) / 64 * 64 <= kLutMax && int64_t(c) * h * wd < (int64_t(1) << 31) && r < 0x7fff && s <= 0xffff;
  if (use_small_tile(a.pixels, o)) {
    dim3 grid(unsigned((a.pixels + 31) / 32), unsigned((o + 31) / 32));
    if (lut) conv_fp32_kernel<32, 32, 4, true><<<grid, 256, 0, stream>>>(a);
    else conv_fp32_kernel<32, 32, 4, false><<<grid, 256, 0, stream>>>(a);
  } else {
    dim3 grid(unsigned((a.pixels + 63) / 64), unsigned((o + 63) / 64));
    if (lut) conv_fp32_kernel<64, 64, 1, true><<<grid, 256, 0, stream>>>(a);
    else conv_fp32_kernel<64, 64, 1, false><<<grid, 256, 0, stream>>>(a);
  }
  return cudaGetLastError();
}

}  // namespace gieb
