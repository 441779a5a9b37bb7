// Strict-FP32 convolution (no tensor cores, no TF32): register-blocked SIMT implicit GEMM straight from NCHW with
// the bias + ReLU epilogue fused.  Stands in for implicit_gemm_kernel (src/kernels/implicit_gemm.cu:47-189).
//
// GEMM view: rows = output pixels (b, oh, ow), columns = output channels, k = (c, r, s) in OIHW order so a weight
// row is contiguous in k.  Per CTA: a TP x TO output tile, 4x4 outputs per thread, BK = 16 reduction slab staged in
// shared memory by asynchronous copies (pixels contiguous in the X slab, so the gather from NCHW is coalesced along ow;
// 128-bit copies of W along k), a ring of slabs in flight while one is consumed.  Accumulation is fmaf in k order.
#include <stdint.h>

#include <mutex>
#include <set>
#include <utility>

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

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
// 4-byte asynchronous copy global -> shared; `valid` false writes zero (nothing is read: the source size is 0).
__device__ __forceinline__ void cp_async4(void* dst, const float* src, bool valid) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(valid ? 4 : 0) : "memory");
}
// 16-byte asynchronous copy (both addresses 16-byte aligned); `bytes` of the source are read, the rest is zero-filled.
__device__ __forceinline__ void cp_async16(void* dst, const float* src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

constexpr int kWPitch = kBK + 4;  // floats per weight row in shared memory: 16-byte aligned rows, conflict-free 128-bit reads

// KG = number of thread groups that split the reduction inside one CTA (slab s goes to group s % KG); their partial
// accumulators are summed in a fixed order at the end, so results are deterministic.  KG > 1 gives small problems
// (few CTAs, long dependent slab chains) enough warps per SM to hide global-load latency.
// Operands reach shared memory through asynchronous copies (cp.async) into a ring of NS slabs per group, so the loads of
// the next NS - 1 slabs are in flight while one is consumed and no register or store instruction is spent on staging:
//   X slab [kBK][TP]: one 4-byte copy per element, gathered from NCHW with zero-fill for padding (pixels contiguous);
//   W slab [TO][kBK]: 128-bit copies along k (OIHW rows are contiguous in k) when W16, else 4-byte copies.
// LUT: k -> (offset of (c, r, s) inside one image, r, s) comes from a table built once per CTA (the analogue of
// build_conv_lut, src/kernels/conv_common.cu:25-37) instead of two divisions per gathered element.
template <int TP, int TO, int KG, int NS, bool LUT, bool W16>
__global__ void __launch_bounds__((TP / 4) * (TO / 4) * KG)
conv_fp32_kernel(const Fp32Args a) {
  constexpr int NT = (TP / 4) * (TO / 4);  // threads per group
  constexpr int XE = kBK * TP / NT;        // X-slab elements copied per thread
  constexpr int XS = kBK * TP, WS = TO * kWPitch;  // floats per X / W slab
  extern __shared__ __align__(16) float tiles[];    // [KG][NS] X slabs, then [KG][NS] W slabs; reused for the group reduction
  __shared__ int2 lut[LUT ? kLutMax : 1];

  const int grp = threadIdx.x / NT;
  const int t = threadIdx.x - grp * NT;
  const int tx = t % (TP / 4), ty = t / (TP / 4);
  const int pix0 = blockIdx.x * TP, oc0 = blockIdx.y * TO;
  const int rs = a.r * a.s;
  const int pq = a.out_h * a.out_w;
  float* xs_base = tiles + size_t(grp) * NS * XS;
  float* ws_base = tiles + size_t(KG) * NS * XS + size_t(grp) * NS * WS;

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

  // issue the copies of the slab that starts at reduction index k0 into ring slot `slot`
  auto fetch = [&](int k0, int slot) {
    float* xs = xs_base + slot * XS;
    float* ws = ws_base + slot * WS;
#pragma unroll
    for (int i = 0; i < XE; ++i) {
      const int kk = t / TP + i * (NT / TP);
      const int k = k0 + kk;
      const float* src = a.x;
      bool ok = false;
      if (LUT) {
        const int2 e = lut[k];
        const int ih = ih0 + (e.y >> 16), iw = iw0 + (e.y & 0xffff);
        ok = lp_ok && unsigned(ih) < unsigned(a.h) && unsigned(iw) < unsigned(a.wd);
        if (ok) src = xb + (e.x + xoff0);
      } else if (lp_ok && k < a.k) {
        const int c = a.fd_rs.div(k), q = k - c * rs;
        const int r = a.fd_s.div(q), sx = q - r * a.s;
        const int ih = ih0 + r, iw = iw0 + sx;
        ok = ih >= 0 && ih < a.h && iw >= 0 && iw < a.wd;
        if (ok) src = xb + (size_t(c) * a.h + ih) * a.wd + iw;
      }
      cp_async4(xs + kk * TP + lp, src, ok);
    }
    if (W16) {  // TO rows x 4 vectors of 4 k-values
#pragma unroll
      for (int i = 0; i < (TO * 4 + NT - 1) / NT; ++i) {
        const int v = t + i * NT;
        if (v < TO * 4) {
          const int row = v >> 2, kq = (v & 3) * 4;
          const int oc = oc0 + row, k = k0 + kq;
          const int left = (oc < a.o && k < a.k) ? min(4, a.k - k) * 4 : 0;
          cp_async16(ws + row * kWPitch + kq, left ? a.w + size_t(oc) * a.k + k : a.w, left);
        }
      }
    } else {
      const int wk = t % kBK;
#pragma unroll
      for (int i = 0; i < kBK * TO / NT; ++i) {
        const int row = t / kBK + i * (NT / kBK);
        const int oc = oc0 + row, k = k0 + wk;
        const bool ok = oc < a.o && k < a.k;
        cp_async4(ws + row * kWPitch + wk, ok ? a.w + size_t(oc) * a.k + k : a.w, ok);
      }
    }
  };

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // every group runs the same number of rounds (slabs beyond K copy zeros), so the barriers stay uniform
  const int rounds = (a.k + kBK * KG - 1) / (kBK * KG);
#pragma unroll
  for (int s = 0; s < NS - 1; ++s) {  // prologue: NS - 1 slabs in flight
    if (s < rounds) fetch((s * KG + grp) * kBK, s);
    cp_async_commit();
  }
  for (int rd = 0; rd < rounds; ++rd) {
    cp_async_wait<NS - 2>();  // this thread's copies of slab rd have landed
    __syncthreads();          // everyone's have; and everyone has finished reading the slot refilled below
    if (rd + NS - 1 < rounds) fetch(((rd + NS - 1) * KG + grp) * kBK, (rd + NS - 1) % NS);
    cp_async_commit();
    const float* xs = xs_base + (rd % NS) * XS;
    const float* ws = ws_base + (rd % NS) * WS;
    // Operands of four k steps at a time (four 128-bit reads of W, four of X), the next four read from shared memory
    // while the current ones are multiplied: with two or three warps per scheduler nothing else hides that latency.
    float4 wv[2][4], xv[2][4];
    auto read_operands = [&](int k4, int buf) {
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[buf][j] = *reinterpret_cast<const float4*>(ws + (ty * 4 + j) * kWPitch + k4);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) xv[buf][kk] = *reinterpret_cast<const float4*>(xs + (k4 + kk) * TP + tx * 4);
    };
    read_operands(0, 0);
#pragma unroll
    for (int q = 0; q < kBK / 4; ++q) {
      const int cur = q & 1;
      if (q + 1 < kBK / 4) read_operands((q + 1) * 4, cur ^ 1);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {  // k order: the accumulation order of the strict-FP32 contract
        const float xa[4] = {xv[cur][kk].x, xv[cur][kk].y, xv[cur][kk].z, xv[cur][kk].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float wk = kk == 0 ? wv[cur][j].x : (kk == 1 ? wv[cur][j].y : (kk == 2 ? wv[cur][j].z : wv[cur][j].w));
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i][j] = fmaf(xa[i], wk, acc[i][j]);
        }
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();  // all slabs consumed: the tiles may be reused

  if (KG > 1) {  // fold groups 1..KG-1 into group 0, in group order
    float* red = tiles;
    static_assert(KG == 1 || (KG - 1) * NT * 16 <= KG * NS * (XS + WS), "reduction scratch must fit the operand tiles");
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

  // Epilogue (fused_epilogue.cuh:11-16 order): + bias, ReLU, store.  Pixels are the fast index of NCHW: a thread's four
  // pixels leave as one 128-bit store when they lie in one image and the address is 16-byte aligned.
  const int pixq = pix0 + tx * 4;
  const int bq = pixq < a.pixels ? a.fd_pq.div(pixq) : 0, remq = pixq - bq * pq;
  const bool quad_ok = pixq + 3 < a.pixels && remq + 3 < pq;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int oc = oc0 + ty * 4 + j;
    if (oc >= a.o) continue;
    const float bv = a.bias ? __ldg(a.bias + oc) : 0.f;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = acc[i][j] + bv;
      if (a.relu) v[i] = fmaxf(v[i], 0.f);
    }
    float* dst = a.y + (size_t(bq) * a.o + oc) * pq + remq;
    if (quad_ok && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
      *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int pix = pixq + i;
        if (pix >= a.pixels) continue;
        const int b = a.fd_pq.div(pix), rem = pix - b * pq;
        a.y[(size_t(b) * a.o + oc) * pq + rem] = v[i];
      }
    }
  }
}

bool use_small_tile(int64_t pixels, int o) {
  const int64_t big = ((pixels + 63) / 64) * ((o + 63) / 64);
  return big < 2 * kNumSms;
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
  const bool lut = (a.k + 63) / 64 * 64 <= kLutMax && int64_t(c) * h * wd < (int64_t(1) << 31) && r < 0x7fff && s <= 0xffff && h < 0x7fff;
  const bool w16 = a.k % 4 == 0 && (reinterpret_cast<uintptr_t>(w) & 15u) == 0;  // 128-bit copies along k
  auto go = [&](auto kernel, dim3 grid, int threads, size_t smem) -> cudaError_t {
    // the opt-in to more than 48 KiB of dynamic shared memory is per function and device: done once each, under a mutex
    // (set_max_dynamic_smem of the reference, src/kernels/conv_common.cu:9-21)
    if (smem > 48 * 1024) {
      static std::mutex mu;
      static std::set<std::pair<const void*, int>> done;
      int dev = 0;
      cudaError_t e = cudaGetDevice(&dev);
      if (e != cudaSuccess) return e;
      std::lock_guard<std::mutex> lock(mu);
      const auto key = std::make_pair(reinterpret_cast<const void*>(kernel), dev);
      if (done.find(key) == done.end()) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return e;
        done.insert(key);
      }
    }
    kernel<<<grid, threads, smem, stream>>>(a);
    return cudaGetLastError();
  };
  if (use_small_tile(a.pixels, o)) {
    constexpr int TP = 32, TO = 32, KG = 4, NS = 4;
    const size_t smem = size_t(KG) * NS * (kBK * TP + TO * kWPitch) * sizeof(float);
    dim3 grid(unsigned((a.pixels + 31) / 32), unsigned((o + 31) / 32));
    if (lut) return w16 ? go(conv_fp32_kernel<TP, TO, KG, NS, true, true>, grid, (TP / 4) * (TO / 4) * KG, smem) : go(conv_fp32_kernel<TP, TO, KG, NS, true, false>, grid, (TP / 4) * (TO / 4) * KG, smem);
    return w16 ? go(conv_fp32_kernel<TP, TO, KG, NS, false, true>, grid, (TP / 4) * (TO / 4) * KG, smem) : go(conv_fp32_kernel<TP, TO, KG, NS, false, false>, grid, (TP / 4) * (TO / 4) * KG, smem);
  }
  constexpr int TP = 64, TO = 64, KG = 1, NS = 4;
  const size_t smem = size_t(KG) * NS * (kBK * TP + TO * kWPitch) * sizeof(float);
  dim3 grid(unsigned((a.pixels + 63) / 64), unsigned((o + 63) / 64));
  if (lut) return w16 ? go(conv_fp32_kernel<TP, TO, KG, NS, true, true>, grid, (TP / 4) * (TO / 4) * KG, smem) : go(conv_fp32_kernel<TP, TO, KG, NS, true, false>, grid, (TP / 4) * (TO / 4) * KG, smem);
  return w16 ? go(conv_fp32_kernel<TP, TO, KG, NS, false, true>, grid, (TP / 4) * (TO / 4) * KG, smem) : go(conv_fp32_kernel<TP, TO, KG, NS, false, false>, grid, (TP / 4) * (TO / 4) * KG, smem);
}

}  // namespace gieb
