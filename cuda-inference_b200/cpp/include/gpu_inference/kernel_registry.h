// The internal plug-in table -- drop-in for the reference's include/gpu_inference/kernel_registry.h.
// One KernelDesc = one launchable configuration.  Here every entry is a point (tile_m, tile_n, tile_k, stages,
// split_k) of the single sm_100a kernel family, or the "auto" entry that lets the library's cost model choose; each
// forwards to the C ABI in gie_b200.h.  Field names and meanings follow the reference so that ExecutionPlan,
// Conv2DOptions::kernel, find_kernel() and code written against the table keep working.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "gpu_inference/conv2d.h"
#include "gpu_inference/device_info.h"

namespace gie {

// 100: first version of the sm_100a family (the reference's mma.sync library is version 2).
constexpr int kLibraryVersion = 100;

struct LaunchArgs {
  const ConvProblem* problem = nullptr;
  const DeviceInfo* dev = nullptr;
  const void* x = nullptr;
  const void* w = nullptr;
  const void* bias = nullptr;       // null unless problem->has_bias
  void* y = nullptr;
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  const void* plan_data = nullptr;  // unused by this family (no lookup tables: TMA descriptors replace them)
  void* plan_state = nullptr;       // what KernelDesc::create_state returned
  cudaStream_t stream = nullptr;
  cudaEvent_t* stage_events = nullptr;  // optional: [0] start, [1] after layout repack, [2] after the convolution
};

struct KernelDesc {
  std::string name;
  Backend backend = Backend::kDirect;
  int version = 1;
  std::vector<std::pair<std::string, int>> params;
  int threads_per_block = 0;
  int tile_m = 1, tile_n = 1, tile_k = 1;  // in the reference's GEMM orientation: tile_m = channels, tile_n = pixels
  bool uses_tensor_cores = false;
  bool needs_lut = false;
  bool lut_chunked = false;
  int launches = 1;
  double efficiency_prior = 0;
  double (*extra_traffic_bytes)(const ConvProblem&) = nullptr;
  const void* function = nullptr;

  bool (*supports)(const ConvProblem&, const DeviceInfo&, std::string* why) = nullptr;
  size_t (*workspace_bytes)(const ConvProblem&) = nullptr;
  size_t (*dynamic_smem_bytes)(const ConvProblem&) = nullptr;
  int64_t (*num_blocks)(const ConvProblem&) = nullptr;
  double (*tile_efficiency)(const ConvProblem&) = nullptr;
  std::shared_ptr<void> (*create_state)(const ConvProblem&) = nullptr;
  size_t (*persistent_bytes)(const ConvProblem&) = nullptr;
  void (*launch)(const LaunchArgs&) = nullptr;
  // Not in the reference's table: the family's own time estimate for this configuration in microseconds (stands in
  // for estimate_kernel of src/runtime/perf_model.cpp:130-174); null = unknown, such entries rank last.
  double (*estimate_us)(const ConvProblem&) = nullptr;

  std::string describe() const;
};

const std::vector<KernelDesc>& kernel_registry();
std::vector<KernelDesc>& kernel_registry_for_testing();  // tests only: lets a test inject a faulty entry
const KernelDesc* find_kernel(const std::string& name);
std::vector<const KernelDesc*> kernels_for_backend(Backend b);

// Offset tables of the reference's gather kernels.  Nothing here consumes them; they are kept so that code
// written against the reference still links, and produce the same entries.
struct alignas(16) LutEntry {
  int32_t c_off;
  int32_t r_off;
  int32_t s_off;
  int32_t pad_;
};
std::vector<LutEntry> build_conv_lut(const Conv2DParams& p);
std::vector<LutEntry> build_conv_lut_chunked(const Conv2DParams& p);

}  // namespace gie
