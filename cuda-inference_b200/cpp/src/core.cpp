// Vocabulary types of the operator API: status codes, errors, element types, device buffers, problem descriptors,
// validation and the device query.  Host code on top of the C ABI (gie_b200.h).
#include <limits>
#include <map>
#include <mutex>
#include <sstream>

#include "gie_b200.h"
#include "gpu_inference/conv2d.h"
#include "gpu_inference/device_info.h"
#include "gpu_inference/tensor.h"

namespace gie {

// ---- errors --------------------------------------------------------------------------------------------------
const char* to_string(StatusCode code) {
  static const char* const names[] = {"ok",         "invalid_argument", "unsupported", "workspace_too_small", "cuda_error",
                                      "cublas_error", "cudnn_error",      "internal",    "io"};
  const int i = int(code);
  return (i >= 0 && i < int(sizeof(names) / sizeof(names[0]))) ? names[i] : "?";
}

Error::Error(StatusCode code, const std::string& message)
    : std::runtime_error(std::string(gie::to_string(code)) + ": " + message), code_(code) {}

void throw_cuda_error(cudaError_t err, const char* expr, const char* file, int line) {
  (void)cudaGetLastError();  // a non-sticky error must not leak into the caller's next CUDA call
  std::ostringstream os;
  os << expr << " failed at " << file << ":" << line << ": " << cudaGetErrorName(err) << " (" << cudaGetErrorString(err) << ")";
  throw Error(StatusCode::kCudaError, os.str());
}

// ---- tensors --------------------------------------------------------------------------------------------------
const char* to_string(DataType t) {
  return t == DataType::kFloat32 ? "float32" : (t == DataType::kFloat16 ? "float16" : "bfloat16");
}

DeviceBuffer::DeviceBuffer(size_t bytes) : bytes_(bytes) {
  if (bytes > 0) GIE_CUDA_CHECK(cudaMalloc(&ptr_, bytes));
}
DeviceBuffer::~DeviceBuffer() { reset(); }
DeviceBuffer& DeviceBuffer::operator=(DeviceBuffer&& other) noexcept {
  if (this != &other) {
    reset();
    ptr_ = other.ptr_;
    bytes_ = other.bytes_;
    other.ptr_ = nullptr;
    other.bytes_ = 0;
  }
  return *this;
}
void DeviceBuffer::memset_async(int value, cudaStream_t stream) {
  if (ptr_ != nullptr) GIE_CUDA_CHECK(cudaMemsetAsync(ptr_, value, bytes_, stream));
}
void DeviceBuffer::reset() {
  if (ptr_ != nullptr) cudaFree(ptr_);
  ptr_ = nullptr;
  bytes_ = 0;
}

std::string TensorShape::to_string() const {
  std::ostringstream os;
  os << "[" << n << "," << c << "," << h << "," << w << "]";
  return os.str();
}

// ---- problem descriptors ------------------------------------------------------------------------------------------
DataType tensor_dtype(Precision p) {
  if (p == Precision::kFp16) return DataType::kFloat16;
  if (p == Precision::kBf16) return DataType::kBFloat16;
  return DataType::kFloat32;
}

namespace {
const char* const kPrecisionNames[] = {"fp32", "fp16", "bf16", "tf32"};
const char* const kBackendNames[] = {"auto", "cpu_reference", "direct", "im2col_gemm", "simt_tiled", "implicit_gemm", "tensor_core"};
}  // namespace

const char* to_string(Precision p) { return kPrecisionNames[int(p) & 3]; }
Precision precision_from_string(const std::string& s) {
  for (int i = 0; i < 4; ++i)
    if (s == kPrecisionNames[i]) return static_cast<Precision>(i);
  throw Error(StatusCode::kInvalidArgument, "unknown precision '" + s + "' (fp32|fp16|bf16|tf32)");
}
const char* to_string(Activation a) { return a == Activation::kReLU ? "relu" : "none"; }
const char* to_string(Backend b) {
  const int i = int(b);
  return (i >= 0 && i < 7) ? kBackendNames[i] : "?";
}
Backend backend_from_string(const std::string& s) {
  for (int i = 0; i < 7; ++i)
    if (s == kBackendNames[i]) return static_cast<Backend>(i);
  throw Error(StatusCode::kInvalidArgument, "unknown backend '" + s + "'");
}

// Same text form as the reference (plan-cache keys and result files are keyed by it).
std::string Conv2DParams::to_string() const {
  std::ostringstream os;
  os << "B" << batch << "_C" << in_channels << "_" << in_h << "x" << in_w << "_O" << out_channels << "_K" << kernel_h << "x"
     << kernel_w << "_s" << stride_h << "x" << stride_w << "_p" << pad_h << "x" << pad_w << "_d" << dilation_h << "x"
     << dilation_w << "_g" << groups;
  return os.str();
}
bool Conv2DParams::operator==(const Conv2DParams& o) const { return to_string() == o.to_string(); }

std::string ConvProblem::key() const {
  std::ostringstream os;
  os << p.to_string() << "_" << gie::to_string(precision) << "_b" << int(has_bias) << "_" << gie::to_string(activation);
  return os.str();
}

gieb_conv_desc to_c_desc(const ConvProblem& pr) {
  const Conv2DParams& p = pr.p;
  gieb_conv_desc d;
  d.batch = p.batch; d.in_channels = p.in_channels; d.in_h = p.in_h; d.in_w = p.in_w;
  d.out_channels = p.out_channels; d.kernel_h = p.kernel_h; d.kernel_w = p.kernel_w;
  d.stride_h = p.stride_h; d.stride_w = p.stride_w; d.pad_h = p.pad_h; d.pad_w = p.pad_w;
  d.dilation_h = p.dilation_h; d.dilation_w = p.dilation_w; d.groups = p.groups;
  d.precision = int(pr.precision);
  d.has_bias = pr.has_bias ? 1 : 0;
  d.relu = pr.activation == Activation::kReLU ? 1 : 0;
  d.flags = 0;
  return d;
}

void validate_problem(const ConvProblem& prob) {
  const gieb_conv_desc d = to_c_desc(prob);
  const int st = gieb_conv_validate(&d);
  if (st != GIEB_OK) throw Error(static_cast<StatusCode>(st), std::string(gieb_last_error()) + ": " + prob.p.to_string());
}

// ---- device query ----------------------------------------------------------------------------------------------
double DeviceInfo::est_peak_fp32_tflops() const { return 2.0 * 128.0 * sm_count * (max_sm_clock_khz * 1e3) / 1e12; }
double DeviceInfo::est_peak_fp16_tc_tflops() const {
  // sm_100: 8192 dense FP16/BF16 FLOP per clock per SM
  return (cc_major == 10 ? 8192.0 : 2048.0) * sm_count * (max_sm_clock_khz * 1e3) / 1e12;
}
double DeviceInfo::est_peak_bw_gbs() const { return 2.0 * (mem_clock_khz * 1e3) * (mem_bus_bits / 8.0) / 1e9; }

std::string DeviceInfo::describe() const {
  std::ostringstream os;
  os << name << " (sm_" << cc_major << cc_minor << ", " << sm_count << " SMs, " << (global_mem_bytes >> 20) << " MiB, L2 "
     << (l2_bytes >> 20) << " MiB, " << (smem_per_block_optin >> 10) << " KiB smem/CTA opt-in)";
  return os.str();
}

const DeviceInfo& DeviceInfo::get(int device) {
  static std::mutex mu;
  static std::map<int, DeviceInfo> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(device);
  if (it != cache.end()) return it->second;
  cudaDeviceProp prop;
  GIE_CUDA_CHECK(cudaGetDeviceProperties(&prop, device));
  DeviceInfo d;
  d.device = device;
  d.name = prop.name;
  d.cc_major = prop.major;
  d.cc_minor = prop.minor;
  d.sm_count = prop.multiProcessorCount;
  d.global_mem_bytes = prop.totalGlobalMem;
  d.l2_bytes = size_t(prop.l2CacheSize);
  d.smem_per_block_default = prop.sharedMemPerBlock;
  d.smem_per_block_optin = prop.sharedMemPerBlockOptin;
  d.smem_per_sm = prop.sharedMemPerMultiprocessor;
  d.regs_per_sm = prop.regsPerMultiprocessor;
  d.max_threads_per_sm = prop.maxThreadsPerMultiProcessor;
  d.max_threads_per_block = prop.maxThreadsPerBlock;
  d.max_blocks_per_sm = prop.maxBlocksPerMultiProcessor;
  d.warp_size = prop.warpSize;
  int v = 0;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, device) == cudaSuccess) d.max_sm_clock_khz = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, device) == cudaSuccess) d.mem_clock_khz = v;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrGlobalMemoryBusWidth, device) == cudaSuccess) d.mem_bus_bits = v;
  (void)cudaGetLastError();
  cudaDriverGetVersion(&d.driver_version);
  cudaRuntimeGetVersion(&d.runtime_version);
  return cache.emplace(device, d).first->second;
}

const DeviceInfo& DeviceInfo::current() {
  int dev = 0;
  GIE_CUDA_CHECK(cudaGetDevice(&dev));
  return get(dev);
}

}  // namespace gie
