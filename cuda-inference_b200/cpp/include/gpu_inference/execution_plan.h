// ExecutionPlan: one problem bound to one KernelDesc -- drop-in for the reference's execution_plan.h.
// create() does all one-time work (capability check, plan-owned device state); execute() validates the call's
// arguments and launches; execute_unchecked() only launches (graph capture, timing loops).
#pragma once

#include <cuda_runtime.h>

#include <memory>

#include "gpu_inference/kernel_registry.h"

namespace gie {

class ExecutionPlan {
 public:
  // device < 0 = the current device.  Throws Error(kUnsupported) when `kernel` cannot run `problem` there.
  static std::shared_ptr<ExecutionPlan> create(const ConvProblem& problem, const KernelDesc& kernel, int device = -1);
  ~ExecutionPlan();
  ExecutionPlan(const ExecutionPlan&) = delete;
  ExecutionPlan& operator=(const ExecutionPlan&) = delete;

  // Checks dtypes, shapes, null pointers, bias presence, output/workspace aliasing, workspace alignment and size and
  // the current device, then launches on `stream`.  Never synchronises.
  void execute(const ConstTensorRef& x, const ConstTensorRef& w, const ConstTensorRef* bias, const TensorRef& y,
               void* workspace, size_t workspace_bytes, cudaStream_t stream, cudaEvent_t* stage_events = nullptr) const;

  // Launch only; the caller has validated the arguments once.  Safe inside stream capture.
  void execute_unchecked(const void* x, const void* w, const void* bias, void* y, void* workspace, size_t workspace_bytes,
                         cudaStream_t stream, cudaEvent_t* stage_events = nullptr) const;

  const ConvProblem& problem() const { return problem_; }
  const KernelDesc& kernel() const { return *kernel_; }
  size_t workspace_bytes() const { return workspace_bytes_; }
  size_t persistent_bytes() const { return persistent_bytes_; }
  int device() const { return device_; }

 private:
  ExecutionPlan() = default;
  ConvProblem problem_;
  const KernelDesc* kernel_ = nullptr;
  int device_ = 0;
  size_t workspace_bytes_ = 0;
  size_t persistent_bytes_ = 0;
  std::shared_ptr<void> state_;
};

}  // namespace gie
