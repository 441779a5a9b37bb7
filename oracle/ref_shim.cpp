// TEST INFRASTRUCTURE ONLY.  C-callable wrapper around the reference library's OWN oracle sources
// (src/cpu/cpu_reference.cpp, src/runtime/{conv2d.cpp,error.cpp,tensor.cpp,reference.cu,testing.cu}),
// which oracle/Makefile compiles unmodified, from where they lie in the reference checkout, into
// oracle/_ref/libgie_ref.so.  This file contains no reference code: it only calls the reference's public
// functions so that Python tests can (a) validate oracle/gie_oracle.c against the real thing, (b) generate the
// golden fixtures under tests/golden/, and (c) time the reference's CPU convolution as the CPU baseline.
//
// The four stubs at the bottom satisfy the linker for Conv2D::forward's dependencies (dispatcher, execution
// plan, device query); the oracle path never reaches them and they throw if called.
#include <omp.h>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#include "gpu_inference/dispatcher.h"
#include "gpu_inference/execution_plan.h"
#include "gpu_inference/reference.h"
#include "gpu_inference/testing.h"

namespace {

// Same field order as orc_conv_desc in oracle/gie_oracle.c.
struct Desc {
  int32_t batch, in_channels, in_h, in_w, out_channels, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w,
      dilation_h, dilation_w, groups, precision, has_bias, relu;
};

gie::ConvProblem to_problem(const Desc& d) {
  gie::ConvProblem pr;
  pr.p.batch = d.batch;
  pr.p.in_channels = d.in_channels;
  pr.p.in_h = d.in_h;
  pr.p.in_w = d.in_w;
  pr.p.out_channels = d.out_channels;
  pr.p.kernel_h = d.kernel_h;
  pr.p.kernel_w = d.kernel_w;
  pr.p.stride_h = d.stride_h;
  pr.p.stride_w = d.stride_w;
  pr.p.pad_h = d.pad_h;
  pr.p.pad_w = d.pad_w;
  pr.p.dilation_h = d.dilation_h;
  pr.p.dilation_w = d.dilation_w;
  pr.p.groups = d.groups;
  pr.precision = static_cast<gie::Precision>(d.precision);
  pr.has_bias = d.has_bias != 0;
  pr.activation = d.relu ? gie::Activation::kReLU : gie::Activation::kNone;
  return pr;
}

float draw(gie::Rng& rng, int dist) {  // same choices as the reference's data generator, via its public Rng
  switch (dist) {
    case 1: return rng.normal();
    case 2: return rng.uniform() < 0.7 ? 0.f : rng.uniform(-2.f, 2.f);
    case 3: return rng.uniform(0.f, 1.f);
    default: return rng.uniform(-1.f, 1.f);
  }
}

}  // namespace

extern "C" {

int ref_validate(const Desc* d) {
  try {
    gie::validate_problem(to_problem(*d));
  } catch (const gie::Error& e) {
    return int(e.code());
  }
  return 0;
}

int ref_out_hw(const Desc* d, int* oh, int* ow, int64_t* flops) {
  const gie::ConvProblem pr = to_problem(*d);
  *oh = pr.p.out_h();
  *ow = pr.p.out_w();
  *flops = pr.p.flops();
  return 0;
}

int ref_conv2d(const Desc* d, const float* x, const float* w, const float* bias, float* y, float* scale) {
  try {
    gie::ReferenceOutput out;
    const gie::ConvProblem pr = to_problem(*d);
    gie::cpu_conv2d_reference(pr, x, w, bias, &out);
    std::memcpy(y, out.y.data(), out.y.size() * sizeof(float));
    if (scale) std::memcpy(scale, out.scale.data(), out.scale.size() * sizeof(float));
  } catch (const gie::Error& e) {
    return int(e.code());
  }
  return 0;
}

// The reference's GPU double-precision convolution (src/runtime/reference.cu:31-93) on device pointers.
int ref_gpu_conv2d(const Desc* d, const void* x, const void* w, const void* bias, float* y, float* scale,
                   void* stream) {
  try {
    gie::gpu_conv2d_reference(to_problem(*d), x, w, bias, y, scale, static_cast<cudaStream_t>(stream));
  } catch (const gie::Error& e) {
    return int(e.code());
  }
  return 0;
}

void ref_rng_u64(uint64_t seed, int64_t n, uint64_t* out) {
  gie::Rng rng(seed);
  for (int64_t i = 0; i < n; ++i) out[i] = rng.next_u64();
}

void ref_rng_draw(uint64_t seed, int dist, int64_t n, float* out) {
  gie::Rng rng(seed);
  for (int64_t i = 0; i < n; ++i) out[i] = draw(rng, dist);
}

// Host half of the reference's make_conv_data (src/runtime/testing.cu:75-99): one generator, x then w then bias,
// weights scaled by sqrt(3/K), bias U(-1,1), everything rounded to the storage precision.
void ref_make_conv_host(const Desc* d, uint64_t seed, int dist, float* x, float* w, float* b) {
  const gie::ConvProblem pr = to_problem(*d);
  gie::Rng rng(seed);
  const int64_t nx = pr.p.input_shape().numel(), nw = pr.p.weight_shape().numel();
  for (int64_t i = 0; i < nx; ++i) x[i] = draw(rng, dist);
  const float wscale = std::sqrt(3.0f / float(pr.p.gemm_k()));
  for (int64_t i = 0; i < nw; ++i) w[i] = draw(rng, dist) * wscale;
  for (int i = 0; i < pr.p.out_channels; ++i) b[i] = rng.uniform(-1.f, 1.f);
  for (int64_t i = 0; i < nx; ++i) x[i] = gie::quantize_to(pr.precision, x[i]);
  for (int64_t i = 0; i < nw; ++i) w[i] = gie::quantize_to(pr.precision, w[i]);
  if (pr.dtype() != gie::DataType::kFloat32)
    for (int i = 0; i < pr.p.out_channels; ++i) b[i] = gie::quantize_to(pr.precision, b[i]);
}

void ref_quantize(int precision, const float* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = gie::quantize_to(static_cast<gie::Precision>(precision), in[i]);
}

// out[0..9] = n, over_tol, nan, inf, max_abs, mean_abs, rms, max_rel, frac_over_tol, worst_tol_ratio
void ref_compare(const Desc* d, int intermediate_rounding, const float* test, const float* ref, const float* scale,
                 int64_t n, double* out) {
  const gie::TolerancePolicy tol = gie::TolerancePolicy::for_problem(to_problem(*d), intermediate_rounding != 0);
  const gie::ErrorMetrics m = gie::compare_outputs(test, ref, scale, n, tol);
  out[0] = double(m.n); out[1] = double(m.over_tol); out[2] = double(m.nan_count); out[3] = double(m.inf_count);
  out[4] = m.max_abs; out[5] = m.mean_abs; out[6] = m.rms; out[7] = m.max_rel; out[8] = m.frac_over_tol;
  out[9] = m.worst_tol_ratio;
}

// The reference's CPU convolution is an OpenMP loop over the outputs (src/cpu/cpu_reference.cpp:23): these set and
// report the number of threads it will use, whatever OMP_NUM_THREADS a launcher exported.
void ref_set_num_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
}
int ref_num_threads(void) { return omp_get_max_threads(); }

double ref_tol(const Desc* d, int intermediate_rounding, double ref, double scale) {
  return gie::TolerancePolicy::for_problem(to_problem(*d), intermediate_rounding != 0).tol(ref, scale);
}

}  // extern "C"

// ---- link-only stubs (never reached by the oracle path) -----------------------------------------------------
namespace gie {
const DeviceInfo& DeviceInfo::get(int) { throw Error(StatusCode::kInternal, "oracle build: DeviceInfo is not available"); }
Selection Dispatcher::select(const ConvProblem&, const DeviceInfo&, const Conv2DOptions&) {
  throw Error(StatusCode::kInternal, "oracle build: the dispatcher is not available");
}
std::shared_ptr<ExecutionPlan> ExecutionPlan::create(const ConvProblem&, const KernelDesc&, int) {
  throw Error(StatusCode::kInternal, "oracle build: execution plans are not available");
}
void ExecutionPlan::execute(const ConstTensorRef&, const ConstTensorRef&, const ConstTensorRef*, const TensorRef&, void*,
                            size_t, cudaStream_t, cudaEvent_t*) const {
  throw Error(StatusCode::kInternal, "oracle build: execution plans are not available");
}
ExecutionPlan::~ExecutionPlan() = default;
}  // namespace gie
