// Stand-alone bias / ReLU passes over an NCHW tensor (the unfused comparator of the fusion tests) -- drop-in for
// the reference's fused_ops.h.  The convolution kernels never call these: their epilogue is fused.
#pragma once

#include <cuda_runtime.h>

#include "gpu_inference/conv2d.h"

namespace gie {

void launch_bias_add(const Conv2DParams& p, Precision prec, const void* bias, void* y, cudaStream_t stream);
void launch_relu(const Conv2DParams& p, Precision prec, void* y, cudaStream_t stream);
void launch_bias_act(const Conv2DParams& p, Precision prec, const void* bias_or_null, bool relu, void* y, cudaStream_t stream);

}  // namespace gie
