/*
 * C++ side of the drop-in: what cuda-inference_b200/cpp/src/b200_family.cpp adds to the reference library's namespace.
 * Include it next to the reference's own headers (gpu_inference/kernel_registry.h).
 */
#ifndef GIE_B200_FAMILY_H_
#define GIE_B200_FAMILY_H_

#include <cstdint>
#include <vector>

#include "gpu_inference/kernel_registry.h"

namespace gie {
namespace kernels {

/* Appends the sm_100a kernel family to the plug-in table: one KernelDesc per (precision, tile, ring depth, split-K,
 * reduction, CTA-pair) point plus one heuristic entry per precision.  The counterpart of the reference's
 * register_tensor_core_mma / register_implicit_gemm (src/kernels/conv_common.cuh:66-71, called from
 * src/runtime/registry.cpp:22-27). */
void register_b200_family(std::vector<KernelDesc>& out);

/* The kernels of this family bound every device-side wait; a wait that runs out is reported in a status word of the plan
 * instead of trapping, and the output of that launch is incomplete.  This ORs the status words of all live plans (every
 * ExecutionPlan created on a kernel of this family) -- 0 means every launch so far computed everything.  Call it after
 * synchronising the streams whose results you are about to trust.  The reference has no counterpart: its kernels have
 * no asynchronous waits ("never returns a result that was not computed", include/gpu_inference/error.h:3-6). */
uint32_t b200_device_status();

}  // namespace kernels
}  // namespace gie

#endif /* GIE_B200_FAMILY_H_ */
