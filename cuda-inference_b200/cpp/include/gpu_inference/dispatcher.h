// Kernel selection -- drop-in for the reference's dispatcher.h for one kernel family.  Priority: an explicit kernel
// name > the persisted tuning cache > a search now (Conv2DOptions::autotune) > the first compatible registry entry of
// the requested backend (the "auto" entries come first; the library's own cost model then picks tile, stages and
// split-K).
#pragma once

#include <string>
#include <utility>
#include <vector>

#include "gpu_inference/kernel_registry.h"

namespace gie {

enum class SelectionSource { kForcedKernel, kForcedBackend, kTuningCache, kTuned, kCostModel };
const char* to_string(SelectionSource s);

struct Selection {
  const KernelDesc* kernel = nullptr;
  SelectionSource source = SelectionSource::kCostModel;
  double predicted_us = 0;
  std::string reason;
};

struct Rejection {
  std::string kernel;
  std::string reason;
};

class Dispatcher {
 public:
  static std::vector<const KernelDesc*> compatible_kernels(const ConvProblem& prob, const DeviceInfo& dev,
                                                           Backend only = Backend::kAuto,
                                                           std::vector<Rejection>* rejected = nullptr);
  static Selection select(const ConvProblem& prob, const DeviceInfo& dev, const Conv2DOptions& opt);
  // Compatible kernels with an estimated time in microseconds, best first (the estimate is the library's cycle
  // model through gieb_conv_query; the "auto" entry of a family ranks first among equals).
  static std::vector<std::pair<const KernelDesc*, double>> rank_by_model(const ConvProblem& prob, const DeviceInfo& dev,
                                                                         const std::vector<const KernelDesc*>& cands);
};

}  // namespace gie
