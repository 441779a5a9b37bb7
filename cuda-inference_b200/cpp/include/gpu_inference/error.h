// gie::Error and status codes -- the error vocabulary of the operator API.
// Drop-in for the reference header of the same name (include/gpu_inference/error.h): same enumerators in the same
// order (their numeric values are what the C ABI returns), same exception type, same two macros.
// Policy: a failed call throws; nothing is launched and no partially computed result is ever handed back.
#pragma once

#include <cuda_runtime.h>

#include <stdexcept>
#include <string>

namespace gie {

enum class StatusCode {
  kOk = 0,
  kInvalidArgument,    // the caller passed something wrong (shape, null pointer, aliasing, alignment, device)
  kUnsupported,        // a well-formed request this library / this GPU cannot serve
  kWorkspaceTooSmall,  // caller-provided scratch is missing or too small
  kCudaError,          // a CUDA runtime or driver call failed
  kCublasError,        // kept for source compatibility; never produced here
  kCudnnError,         // kept for source compatibility; never produced here
  kInternal,
  kIo,
};

const char* to_string(StatusCode code);

class Error : public std::runtime_error {
 public:
  Error(StatusCode code, const std::string& message);
  StatusCode code() const noexcept { return code_; }

 private:
  StatusCode code_;
};

// Clears the (non-sticky) CUDA error state and throws Error(kCudaError) naming the failed expression.
[[noreturn]] void throw_cuda_error(cudaError_t err, const char* expr, const char* file, int line);

}  // namespace gie

#define GIE_CUDA_CHECK(expr)                                                                \
  do {                                                                                      \
    const cudaError_t gie_status_ = (expr);                                                 \
    if (gie_status_ != cudaSuccess) ::gie::throw_cuda_error(gie_status_, #expr, __FILE__, __LINE__); \
  } while (0)

#define GIE_REQUIRE(cond, code, msg)                   \
  do {                                                 \
    if (!(cond)) throw ::gie::Error((code), (msg));    \
  } while (0)
