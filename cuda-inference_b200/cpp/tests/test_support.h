// Shared helpers of the C++ layer's GPU tests: problems, data bundles with their CPU reference, one-call runners.
#pragma once

#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "check.h"
#include "gpu_inference/conv2d.h"
#include "gpu_inference/dispatcher.h"
#include "gpu_inference/execution_plan.h"
#include "gpu_inference/reference.h"
#include "gpu_inference/testing.h"

namespace ts {

inline gie::Conv2DParams geom(int b, int c, int h, int w, int o, int kh, int kw, int sh, int sw, int ph, int pw) {
  gie::Conv2DParams p;
  p.batch = b; p.in_channels = c; p.in_h = h; p.in_w = w; p.out_channels = o;
  p.kernel_h = kh; p.kernel_w = kw; p.stride_h = sh; p.stride_w = sw; p.pad_h = ph; p.pad_w = pw;
  return p;
}

inline gie::ConvProblem problem(const gie::Conv2DParams& p, gie::Precision prec, bool bias, bool relu) {
  gie::ConvProblem pr;
  pr.p = p;
  pr.precision = prec;
  pr.has_bias = bias;
  pr.activation = relu ? gie::Activation::kReLU : gie::Activation::kNone;
  return pr;
}

// Synthetic tensors on the device plus the CPU reference of the same values.
struct Bundle {
  gie::ConvData data;
  gie::ReferenceOutput ref;
};

inline Bundle make_bundle(const gie::ConvProblem& prob, uint64_t seed, gie::Distribution dist = gie::Distribution::kUniform) {
  Bundle b;
  b.data = gie::make_conv_data(prob, seed, dist);
  gie::cpu_conv2d_reference(prob, b.data.hx.data(), b.data.hw.data(), prob.has_bias ? b.data.hb.data() : nullptr, &b.ref);
  return b;
}

inline gie::ErrorMetrics compare_device(const void* y_dev, const Bundle& b) {
  const gie::ConvProblem& prob = b.data.prob;
  const int64_t n = prob.p.output_shape().numel();
  const std::vector<float> out = gie::download_as_float(y_dev, prob.dtype(), n);
  return gie::compare_outputs(out.data(), b.ref.y.data(), b.ref.scale.data(), n, gie::TolerancePolicy::for_problem(prob));
}

inline std::vector<uint8_t> download_bytes(const void* dev, size_t bytes) {
  std::vector<uint8_t> h(bytes);
  GIE_CUDA_CHECK(cudaMemcpy(h.data(), dev, bytes, cudaMemcpyDeviceToHost));
  return h;
}

// Runs one registered kernel once on the bundle (output poisoned first) and compares with the CPU reference.
inline gie::ErrorMetrics run_kernel(const gie::KernelDesc& k, Bundle& b, bool* ran, std::string* why) {
  const gie::ConvProblem& prob = b.data.prob;
  std::string reason;
  if (!k.supports(prob, gie::DeviceInfo::current(), &reason)) {
    *ran = false;
    if (why != nullptr) *why = reason;
    return {};
  }
  *ran = true;
  auto plan = gie::ExecutionPlan::create(prob, k);
  gie::DeviceBuffer ws(plan->workspace_bytes());
  GIE_CUDA_CHECK(cudaMemset(b.data.dy.data(), 0xFF, b.data.dy.size()));
  const gie::ConstTensorRef bias = b.data.b_ref();
  plan->execute(b.data.x_ref(), b.data.w_ref(), prob.has_bias ? &bias : nullptr, b.data.y_ref(), ws.data(), ws.size(), nullptr);
  GIE_CUDA_CHECK(cudaDeviceSynchronize());
  return compare_device(b.data.dy.data(), b);
}

struct NamedShape { const char* name; gie::Conv2DParams p; };

// A cross-section of the reference suite's correctness shapes (tests/shapes.h): small, odd, strided, padded, 1x1.
inline const std::vector<NamedShape>& shapes() {
  static const std::vector<NamedShape> s = {
      {"tiny_1ch_5x5_k3", geom(1, 1, 5, 5, 1, 3, 3, 1, 1, 0, 0)},
      {"scalar_1x1_k1", geom(1, 1, 1, 1, 1, 1, 1, 1, 1, 0, 0)},
      {"rgb_32x32_k3p1_b2", geom(2, 3, 32, 32, 16, 3, 3, 1, 1, 1, 1)},
      {"odd_unequal_k5s2", geom(1, 3, 33, 31, 8, 5, 5, 2, 2, 2, 2)},
      {"pointwise_odd_b2", geom(2, 16, 15, 17, 24, 1, 1, 1, 1, 0, 0)},
      {"resnet_14x14_b8_k3", geom(8, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1)},
      {"resnet_down_28_s2_b2", geom(2, 64, 28, 28, 128, 3, 3, 2, 2, 1, 1)},
      {"deep_512ch_7x7", geom(1, 512, 7, 7, 512, 3, 3, 1, 1, 1, 1)},
      {"irregular_c7_o9_s2", geom(2, 7, 11, 13, 9, 3, 3, 2, 2, 0, 0)},
      {"c130_o130_9x9", geom(2, 130, 9, 9, 130, 3, 3, 1, 1, 1, 1)},
      {"o255_pointwise_13", geom(1, 64, 13, 13, 255, 1, 1, 1, 1, 0, 0)},
      {"stem_7x7_s2_64", geom(2, 3, 64, 64, 64, 7, 7, 2, 2, 3, 3)},
      {"boundary_pad4_k5", geom(1, 16, 10, 10, 16, 5, 5, 1, 1, 4, 4)},
      {"aniso_k3x5_s2x1", geom(2, 8, 17, 23, 12, 3, 5, 2, 1, 1, 2)},
      {"wide_1x1_b32", geom(32, 24, 7, 7, 40, 1, 1, 1, 1, 0, 0)},
  };
  return s;
}

}  // namespace ts
