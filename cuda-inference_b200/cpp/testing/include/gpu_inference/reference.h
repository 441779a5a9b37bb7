// TEST SUPPORT (not part of the product library): CPU reference convolution, tolerance model, error metrics and
// rounding helpers with the reference's names and signatures (include/gpu_inference/reference.h), implemented on top
// of the repository's test oracle (oracle/gie_oracle.c).  Linked only into tests and examples.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <string>
#include <vector>

#include "gpu_inference/conv2d.h"

namespace gie {

struct ReferenceOutput {
  std::vector<float> y;
  std::vector<float> scale;  // sqrt(sum (x*w)^2 + (sum x*w)^2 + bias^2): magnitude that governs rounding error
};

// Double-accumulating direct convolution on host arrays holding storage-rounded values; bias may be null.
void cpu_conv2d_reference(const ConvProblem& prob, const float* x, const float* w, const float* bias, ReferenceOutput* out);

// tol_i = c_acc*u_acc*sqrt(K)*scale_i + c_out*u_out*|ref_i| + c_inter*u_out*scale_i + c_in*u_in*scale_i + abs_floor
struct TolerancePolicy {
  double c_acc = 8.0;
  double c_out = 1.0;
  double c_inter = 0.0;
  double c_in = 0.0;
  double u_in = 0.00048828125;
  double u_acc = 5.9604644775390625e-08;
  double u_out = 5.9604644775390625e-08;
  double abs_floor = 1e-30;
  int64_t k = 1;
  static TolerancePolicy for_problem(const ConvProblem& prob, bool intermediate_rounding = false);
  double tol(double ref, double scale) const;
  std::string describe() const;
};

struct ErrorMetrics {
  int64_t n = 0;
  double max_abs = 0, mean_abs = 0, rms = 0;
  double max_rel = 0;
  double frac_over_tol = 0;
  int64_t over_tol = 0, nan_count = 0, inf_count = 0;
  double worst_tol_ratio = 0;
  bool passed() const { return n > 0 && nan_count == 0 && inf_count == 0 && over_tol == 0; }
  std::string summary() const;
};

ErrorMetrics compare_outputs(const float* test, const float* ref, const float* scale, int64_t n, const TolerancePolicy& tol);

float quantize_to(Precision p, float v);
float round_to_tf32(float v);
std::vector<float> download_as_float(const void* d_ptr, DataType dt, int64_t n);

}  // namespace gie
