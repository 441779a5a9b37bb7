// TEST SUPPORT (not part of the product library): deterministic synthetic data with the reference's names and
// signatures (include/gpu_inference/testing.h), implemented on top of the repository's test oracle.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include "gpu_inference/conv2d.h"
#include "gpu_inference/reference.h"

namespace gie {

class Rng {  // SplitMix64
 public:
  explicit Rng(uint64_t seed) : s_(seed) {}
  uint64_t next_u64();
  double uniform();
  float uniform(float lo, float hi);
  float normal();

 private:
  uint64_t s_;
};

enum class Distribution { kUniform, kNormal, kSparseSigned, kPositive };
const char* to_string(Distribution d);

struct ConvData {
  ConvProblem prob;
  std::vector<float> hx, hw, hb;  // what the reference consumes (storage-rounded)
  DeviceBuffer dx, dw, db, dy;    // device tensors in the storage type; dy is poisoned with 0xFF bytes

  ConstTensorRef x_ref() const;
  ConstTensorRef w_ref() const;
  ConstTensorRef b_ref() const;
  TensorRef y_ref();
};

ConvData make_conv_data(const ConvProblem& prob, uint64_t seed, Distribution dist = Distribution::kUniform);
DeviceBuffer upload_as(const std::vector<float>& v, DataType dt);

}  // namespace gie
