// CUDA-event timing with robust summary statistics -- drop-in for the reference's include/gpu_inference/timing.h
// (protocol of src/runtime/timing.cpp:21-83: warm-up, then `samples` event pairs around `inner` back-to-back launches
// each; short kernels are batched until a sample lasts min_sample_ms; optional cold-cache samples).
#pragma once

#include <cuda_runtime.h>

#include <functional>
#include <vector>

namespace gie {

struct TimingStats {
  int samples = 0;
  int inner_iters = 1;  // launches averaged inside each sample
  double median_us = 0, mean_us = 0, min_us = 0, max_us = 0;
  double p10_us = 0, p90_us = 0, p99_us = 0;
  double stddev_us = 0;
  double iqr_us = 0;
  std::vector<double> raw_us;  // per-sample latency of one launch
};

struct TimingOptions {
  int warmup_iters = 5;
  int samples = 20;
  int inner = 0;               // <= 0: chosen so that one sample lasts at least min_sample_ms
  double min_sample_ms = 1.0;
  int max_inner = 4096;
  void* flush_buffer = nullptr;  // cold-cache protocol: with flush_bytes > 0 every sample is ONE launch preceded by an
  size_t flush_bytes = 0;        // untimed memset of this buffer (make it larger than L2)
};

// `launch` must enqueue the work on `stream` without synchronising.
TimingStats time_stream_work(const std::function<void(cudaStream_t)>& launch, cudaStream_t stream, const TimingOptions& opt = {});

TimingStats summarize(std::vector<double> per_launch_us, int inner);

}  // namespace gie
