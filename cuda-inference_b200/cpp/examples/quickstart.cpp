// Smallest complete use of the operator API: one FP16 3x3 convolution with fused bias + ReLU, checked on the host.
#include <cstdio>
#include <vector>

#include "gpu_inference/conv2d.h"
#include "gpu_inference/testing.h"  // test-support library: synthetic data + CPU reference

int main() {
  try {
    gie::ConvProblem prob;
    prob.p.batch = 4;
    prob.p.in_channels = 64;
    prob.p.in_h = prob.p.in_w = 28;
    prob.p.out_channels = 128;
    prob.p.kernel_h = prob.p.kernel_w = 3;
    prob.p.pad_h = prob.p.pad_w = 1;
    prob.precision = gie::Precision::kFp16;
    prob.has_bias = true;
    prob.activation = gie::Activation::kReLU;

    gie::ConvData data = gie::make_conv_data(prob, 42);
    cudaStream_t stream = nullptr;
    GIE_CUDA_CHECK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    gie::DeviceBuffer workspace(gie::Conv2D::workspace_size(prob));
    const gie::ConstTensorRef bias = data.b_ref();
    gie::Conv2D::forward(data.x_ref(), data.w_ref(), &bias, prob, data.y_ref(), workspace.data(), workspace.size(), stream);
    GIE_CUDA_CHECK(cudaStreamSynchronize(stream));
    cudaStreamDestroy(stream);

    const int64_t n = prob.p.output_shape().numel();
    const std::vector<float> y = gie::download_as_float(data.dy.data(), prob.dtype(), n);
    gie::ReferenceOutput ref;
    gie::cpu_conv2d_reference(prob, data.hx.data(), data.hw.data(), data.hb.data(), &ref);
    const gie::ErrorMetrics m = gie::compare_outputs(y.data(), ref.y.data(), ref.scale.data(), n, gie::TolerancePolicy::for_problem(prob));
    std::printf("output %s  workspace %zu B  %s\n", prob.p.output_shape().to_string().c_str(), workspace.size(), m.summary().c_str());
    return m.passed() ? 0 : 2;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
}
