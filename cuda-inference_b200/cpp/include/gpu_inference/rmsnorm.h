// Fused RMSNorm / residual-add + RMSNorm -- drop-in for the reference's rmsnorm.h (fused operator only; the
// reference's three-kernel unfused comparator is not part of this library).
//   y[r,:] = s[r,:] * rsqrt(mean(s[r,:]^2) + eps) * gamma[:],   s = x   or   s = round(x + residual_in)
#pragma once

#include <cuda_runtime.h>

#include "gpu_inference/conv2d.h"

namespace gie {

struct RmsNormParams {
  int rows = 1;
  int hidden = 1;
  float eps = 1e-6f;
  DataType dtype = DataType::kFloat32;
};

// Both residual pointers null: plain RMSNorm.  Both given: residual_out = round(x + residual_in) is written and
// normalised (residual_out may alias x).  y must not alias any other argument.  Asynchronous on `stream`.
void rmsnorm_forward(const RmsNormParams& p, const void* x, const void* gamma, void* y, const void* residual_in,
                     void* residual_out, cudaStream_t stream);

}  // namespace gie
