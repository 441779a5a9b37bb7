// Tensor vocabulary of the operator API: element types, an owning device allocation and non-owning views.
// Drop-in for the reference's include/gpu_inference/tensor.h.  All tensors are dense and contiguous:
// activations NCHW, weights OIHW, a bias vector has the logical shape {1, C_out, 1, 1}.
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>

#include "gpu_inference/error.h"

namespace gie {

enum class DataType { kFloat32, kFloat16, kBFloat16 };

inline size_t dtype_size(DataType t) { return t == DataType::kFloat32 ? 4 : 2; }
const char* to_string(DataType t);

// RAII wrapper around one cudaMalloc'd block; movable, not copyable.
class DeviceBuffer {
 public:
  DeviceBuffer() = default;
  explicit DeviceBuffer(size_t bytes);
  ~DeviceBuffer();
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;
  DeviceBuffer(DeviceBuffer&& other) noexcept : ptr_(other.ptr_), bytes_(other.bytes_) {
    other.ptr_ = nullptr;
    other.bytes_ = 0;
  }
  DeviceBuffer& operator=(DeviceBuffer&& other) noexcept;

  void* data() const { return ptr_; }
  size_t size() const { return bytes_; }
  explicit operator bool() const { return ptr_ != nullptr; }
  void memset_async(int value, cudaStream_t stream = nullptr);
  void reset();

 private:
  void* ptr_ = nullptr;
  size_t bytes_ = 0;
};

struct TensorShape {
  int64_t n = 1;
  int64_t c = 1;
  int64_t h = 1;
  int64_t w = 1;
  int64_t numel() const { return n * c * h * w; }
  bool operator==(const TensorShape& o) const { return n == o.n && c == o.c && h == o.h && w == o.w; }
  bool operator!=(const TensorShape& o) const { return !(*this == o); }
  std::string to_string() const;
};

// Views: a device pointer plus what the caller claims it holds; forward()/execute() check the claim.
struct ConstTensorRef {
  const void* data = nullptr;
  DataType dtype = DataType::kFloat32;
  TensorShape shape;
};

struct TensorRef {
  void* data = nullptr;
  DataType dtype = DataType::kFloat32;
  TensorShape shape;
  operator ConstTensorRef() const { return {data, dtype, shape}; }
};

}  // namespace gie
