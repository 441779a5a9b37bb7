// Capture / replay helper for a sequence of asynchronous launches -- drop-in for the reference's cuda_graph.h.
#pragma once

#include <cuda_runtime.h>

#include <functional>

#include "gpu_inference/error.h"

namespace gie {

class CudaGraphExecutor {
 public:
  // The callable enqueues work on the given stream and must neither allocate nor synchronise.
  using Enqueue = std::function<void(cudaStream_t)>;

  CudaGraphExecutor() = default;
  ~CudaGraphExecutor();
  CudaGraphExecutor(const CudaGraphExecutor&) = delete;
  CudaGraphExecutor& operator=(const CudaGraphExecutor&) = delete;

  // One eager run on a private stream (so lazy one-time initialisation happens outside capture), then capture and
  // instantiate.  Throws on failure.
  void capture(const Enqueue& enqueue);

  // Capture again (same topology, e.g. other buffers) and patch the instantiated graph in place when possible;
  // otherwise re-instantiate.  Returns true when patched in place.
  bool recapture_update(const Enqueue& enqueue);

  void launch(cudaStream_t stream) const;

  bool valid() const { return exec_ != nullptr; }
  size_t node_count() const { return nodes_; }
  double capture_us() const { return capture_us_; }
  double instantiate_us() const { return instantiate_us_; }

 private:
  void capture_graph(const Enqueue& enqueue, cudaGraph_t* g, double* us);
  void reset();
  cudaGraph_t graph_ = nullptr;
  cudaGraphExec_t exec_ = nullptr;
  size_t nodes_ = 0;
  double capture_us_ = 0, instantiate_us_ = 0;
};

}  // namespace gie
