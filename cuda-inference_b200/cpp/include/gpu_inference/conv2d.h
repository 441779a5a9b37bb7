// Convolution problem descriptor and the public entry point gie::Conv2D -- drop-in for the reference's
// include/gpu_inference/conv2d.h (same names, fields, defaults and signatures).
//
// The operator is a cross-correlation with zero padding followed by an optional bias add and ReLU:
//   Y[b,o,p,q] = act( bias[o] + sum_{c,r,s} X[b,c, p*stride_h - pad_h + r, q*stride_w - pad_w + s] * W[o,c,r,s] )
//   P = (H + 2*pad_h - (R-1) - 1) / stride_h + 1     (integer division; likewise Q)
// X is NCHW, W is OIHW, Y is NCHW; everything contiguous, everything (bias included) in the precision's storage type.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "gpu_inference/tensor.h"

namespace gie {

// Storage type + multiplier precision.  Accumulation is always FP32.
//   kFp32  FP32 storage, plain FP32 FMA arithmetic (never TF32)
//   kFp16  FP16 storage, tensor cores, FP32 accumulate
//   kBf16  BF16 storage, tensor cores, FP32 accumulate
//   kTf32  FP32 storage, inputs rounded to TF32 (ties away), tensor-core contraction (kind::tf32), FP32 accumulate / output
enum class Precision { kFp32, kFp16, kBf16, kTf32 };

DataType tensor_dtype(Precision p);
const char* to_string(Precision p);
Precision precision_from_string(const std::string& s);  // throws Error(kInvalidArgument) on an unknown name

enum class Activation { kNone, kReLU };
const char* to_string(Activation a);

// Kept value-for-value so option structs and string names stay interchangeable.  This library serves kAuto,
// kTensorCore (FP16/BF16) and kImplicitGemm (FP32); asking for any other backend yields kUnsupported.
enum class Backend {
  kAuto,
  kCpuReference,
  kDirect,
  kIm2colGemm,
  kSimtTiled,
  kImplicitGemm,
  kTensorCore,
};
const char* to_string(Backend b);
Backend backend_from_string(const std::string& s);  // throws Error(kInvalidArgument) on an unknown name

struct Conv2DParams {
  int batch = 1;
  int in_channels = 1, in_h = 1, in_w = 1;
  int out_channels = 1, kernel_h = 1, kernel_w = 1;
  int stride_h = 1, stride_w = 1;
  int pad_h = 0, pad_w = 0;
  int dilation_h = 1, dilation_w = 1;  // must be 1
  int groups = 1;                      // must be 1

  int out_h() const { return (in_h + 2 * pad_h - dilation_h * (kernel_h - 1) - 1) / stride_h + 1; }
  int out_w() const { return (in_w + 2 * pad_w - dilation_w * (kernel_w - 1) - 1) / stride_w + 1; }

  // GEMM view kept in the reference's orientation: M = C_out, N = B*P*Q, K = C_in*R*S.
  int64_t gemm_m() const { return out_channels; }
  int64_t gemm_n() const { return int64_t(batch) * out_h() * out_w(); }
  int64_t gemm_k() const { return int64_t(in_channels) * kernel_h * kernel_w; }
  int64_t flops() const { return 2 * gemm_m() * gemm_n() * gemm_k(); }

  TensorShape input_shape() const { return {batch, in_channels, in_h, in_w}; }
  TensorShape weight_shape() const { return {out_channels, in_channels, kernel_h, kernel_w}; }
  TensorShape output_shape() const { return {batch, out_channels, out_h(), out_w()}; }
  TensorShape bias_shape() const { return {1, out_channels, 1, 1}; }

  std::string to_string() const;
  bool operator==(const Conv2DParams& o) const;
};

struct ConvProblem {
  Conv2DParams p;
  Precision precision = Precision::kFp32;
  bool has_bias = false;
  Activation activation = Activation::kNone;

  DataType dtype() const { return tensor_dtype(precision); }
  std::string key() const;  // canonical text form; plan-cache key
  bool operator==(const ConvProblem& o) const { return key() == o.key(); }
};

// Throws Error(kInvalidArgument) for malformed geometry and Error(kUnsupported) for dilation / groups != 1.
void validate_problem(const ConvProblem& prob);

struct Conv2DOptions {
  Backend backend = Backend::kAuto;
  std::string kernel;         // name of one registered configuration to force (optional)
  bool autotune = false;      // search the registered configurations now when the tuning cache has no entry
  bool force_retune = false;  // ignore the cached winner and search again (with autotune)
  std::string cache_path;     // tuning cache file; empty -> TuneCache::default_path()
};

class Conv2D {
 public:
  // Y = act(conv(X, W) [+ bias]) enqueued on `stream`; never synchronises the device.  `workspace` must be 256-byte
  // aligned and hold workspace_size() bytes.  The first call for a new (problem, options, device) creates and caches a
  // plan (may allocate and synchronise a private stream); later calls only launch.
  static void forward(const ConstTensorRef& input, const ConstTensorRef& weights, const ConstTensorRef* bias,
                      const ConvProblem& problem, const TensorRef& output, void* workspace, size_t workspace_bytes,
                      cudaStream_t stream, const Conv2DOptions& options = {});

  static size_t workspace_size(const ConvProblem& problem, const Conv2DOptions& options = {});
  static void clear_plan_cache();
};

}  // namespace gie
