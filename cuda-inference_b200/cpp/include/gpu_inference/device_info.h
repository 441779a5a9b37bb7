// Device query used by capability checks -- drop-in for the reference's include/gpu_inference/device_info.h.
// Peak figures are estimates from the device's clocks and SM count, not measurements.
#pragma once

#include <cuda_runtime.h>

#include <string>

namespace gie {

struct DeviceInfo {
  int device = 0;
  std::string name;
  int cc_major = 0, cc_minor = 0;
  int sm_count = 0;
  size_t global_mem_bytes = 0;
  size_t l2_bytes = 0;
  size_t smem_per_block_default = 0;
  size_t smem_per_block_optin = 0;
  size_t smem_per_sm = 0;
  int regs_per_sm = 0;
  int max_threads_per_sm = 0;
  int max_threads_per_block = 0;
  int max_blocks_per_sm = 0;
  int warp_size = 32;
  int max_sm_clock_khz = 0;
  int mem_clock_khz = 0;
  int mem_bus_bits = 0;
  int driver_version = 0;
  int runtime_version = 0;

  int cc() const { return cc_major * 10 + cc_minor; }
  bool supports_fp16_tensor_cores() const { return cc() >= 70; }
  bool supports_bf16_tensor_cores() const { return cc() >= 80; }
  bool supports_tf32_tensor_cores() const { return cc() >= 80; }
  bool supports_cp_async() const { return cc() >= 80; }
  bool supports_tcgen05() const { return cc_major == 10; }  // what this library actually needs

  double est_peak_fp32_tflops() const;
  double est_peak_fp16_tc_tflops() const;  // dense, FP32 accumulate
  double est_peak_bw_gbs() const;

  std::string describe() const;

  static const DeviceInfo& get(int device);  // cached per device, thread-safe
  static const DeviceInfo& current();
};

}  // namespace gie
