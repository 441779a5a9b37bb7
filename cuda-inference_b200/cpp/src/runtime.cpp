// Operator layer on top of the plug-in table: selection, execution plans, the plan cache behind Conv2D::forward,
// CUDA-graph capture, RMSNorm and the stand-alone elementwise passes.
#include <chrono>
#include <map>
#include <mutex>
#include <sstream>
#include <tuple>

#include "gie_b200.h"
#include "gpu_inference/autotuner.h"
#include "gpu_inference/cuda_graph.h"
#include "gpu_inference/dispatcher.h"
#include "gpu_inference/execution_plan.h"
#include "gpu_inference/fused_ops.h"
#include "gpu_inference/nvtx.h"
#include "gpu_inference/rmsnorm.h"

namespace gie {

// ---- selection ------------------------------------------------------------------------------------------------------
const char* to_string(SelectionSource s) {
  switch (s) {
    case SelectionSource::kForcedKernel: return "forced_kernel";
    case SelectionSource::kForcedBackend: return "forced_backend";
    case SelectionSource::kTuningCache: return "tuning_cache";
    case SelectionSource::kTuned: return "tuned";
    case SelectionSource::kCostModel: return "cost_model";
  }
  return "?";
}

std::vector<const KernelDesc*> Dispatcher::compatible_kernels(const ConvProblem& prob, const DeviceInfo& dev, Backend only,
                                                              std::vector<Rejection>* rejected) {
  std::vector<const KernelDesc*> ok;
  for (const KernelDesc& k : kernel_registry()) {
    if (only != Backend::kAuto && k.backend != only) continue;
    std::string why;
    if (k.supports(prob, dev, &why)) ok.push_back(&k);
    else if (rejected != nullptr) rejected->push_back({k.name, why});
  }
  return ok;
}

Selection Dispatcher::select(const ConvProblem& prob, const DeviceInfo& dev, const Conv2DOptions& opt) {
  NvtxRange range("gie::Dispatcher::select");
  validate_problem(prob);
  Selection sel;
  if (!opt.kernel.empty()) {
    const KernelDesc* k = find_kernel(opt.kernel);
    if (k == nullptr) throw Error(StatusCode::kInvalidArgument, "unknown kernel '" + opt.kernel + "'");
    if (opt.backend != Backend::kAuto && k->backend != opt.backend)
      throw Error(StatusCode::kInvalidArgument, "kernel '" + opt.kernel + "' belongs to backend " + to_string(k->backend) +
                                                    ", not " + to_string(opt.backend));
    std::string why;
    if (!k->supports(prob, dev, &why)) throw Error(StatusCode::kUnsupported, k->name + ": " + why);
    sel.kernel = k;
    sel.source = SelectionSource::kForcedKernel;
    sel.reason = "explicit kernel";
    return sel;
  }
  if (opt.backend == Backend::kCpuReference)
    throw Error(StatusCode::kUnsupported, "the CPU reference is not a GPU backend");
  std::vector<Rejection> rejected;
  const std::vector<const KernelDesc*> cands = compatible_kernels(prob, dev, opt.backend, &rejected);
  if (cands.empty()) {
    std::ostringstream os;
    os << "no kernel can run " << prob.key() << " on " << dev.name << " (backend=" << to_string(opt.backend) << ")";
    if (rejected.empty()) os << ": this library has no kernels for that backend (single sm_100a family: tensor_core, implicit_gemm)";
    for (size_t i = 0; i < rejected.size() && i < 4; ++i) os << "\n  - " << rejected[i].kernel << ": " << rejected[i].reason;
    throw Error(StatusCode::kUnsupported, os.str());
  }
  // measured winners first: the persisted tuning cache, then (when asked for) a search now
  {
    TuneCache cache(opt.cache_path);
    std::string name;
    double us = 0;
    if (!opt.force_retune && cache.lookup(prob, dev, &name, &us, nullptr, opt.backend)) {
      if (const KernelDesc* k = find_kernel(name)) {
        sel.kernel = k;
        sel.source = SelectionSource::kTuningCache;
        sel.predicted_us = us;
        sel.reason = "winner recorded in " + cache.path();
        return sel;
      }
    }
    if (opt.autotune) {
      TuneOptions to;
      to.only_backend = opt.backend;
      to.cache_path = opt.cache_path;
      to.force_retune = opt.force_retune;
      to.timing.samples = 10;
      const TuneResult tr = Autotuner::tune(prob, dev, to);
      sel.kernel = find_kernel(tr.best_kernel);
      sel.source = tr.from_cache ? SelectionSource::kTuningCache : SelectionSource::kTuned;
      sel.predicted_us = tr.best_us;
      sel.reason = "measured fastest of " + std::to_string(tr.candidates_measured) + " candidates";
      if (sel.kernel != nullptr) return sel;
    }
  }
  sel.kernel = cands.front();  // the family's "auto" entry: tile, stages and split-K come from the built-in cost model
  sel.source = opt.backend == Backend::kAuto ? SelectionSource::kCostModel : SelectionSource::kForcedBackend;
  sel.reason = "first compatible entry; configuration chosen by the library's cost model";
  return sel;
}

// ---- execution plan -------------------------------------------------------------------------------------------------
namespace {

struct ScopedDevice {
  int previous = 0, wanted = 0;
  explicit ScopedDevice(int dev) : wanted(dev) {
    GIE_CUDA_CHECK(cudaGetDevice(&previous));
    if (previous != wanted) GIE_CUDA_CHECK(cudaSetDevice(wanted));
  }
  ~ScopedDevice() {
    if (previous != wanted) cudaSetDevice(previous);
  }
};

bool ranges_overlap(const void* a, size_t an, const void* b, size_t bn) {
  if (a == nullptr || b == nullptr || an == 0 || bn == 0) return false;
  const uintptr_t pa = reinterpret_cast<uintptr_t>(a), pb = reinterpret_cast<uintptr_t>(b);
  return pa < pb + bn && pb < pa + an;
}

void require_tensor(const char* what, const void* data, DataType dtype, const TensorShape& shape, DataType want_dtype,
                    const TensorShape& want_shape) {
  const std::string w(what);
  GIE_REQUIRE(data != nullptr, StatusCode::kInvalidArgument, w + ": null device pointer");
  GIE_REQUIRE(dtype == want_dtype, StatusCode::kInvalidArgument,
              w + ": dtype " + to_string(dtype) + " but the problem's precision needs " + to_string(want_dtype));
  GIE_REQUIRE(shape == want_shape, StatusCode::kInvalidArgument, w + ": shape " + shape.to_string() + " but expected " + want_shape.to_string());
}

}  // namespace

std::shared_ptr<ExecutionPlan> ExecutionPlan::create(const ConvProblem& problem, const KernelDesc& kernel, int device) {
  NvtxRange range("gie::ExecutionPlan::create");
  validate_problem(problem);
  if (device < 0) GIE_CUDA_CHECK(cudaGetDevice(&device));
  ScopedDevice guard(device);
  const DeviceInfo& dev = DeviceInfo::get(device);
  std::string why;
  if (!kernel.supports(problem, dev, &why))
    throw Error(StatusCode::kUnsupported, kernel.name + " cannot run " + problem.key() + " on " + dev.name + ": " + why);
  std::shared_ptr<ExecutionPlan> plan(new ExecutionPlan());
  plan->problem_ = problem;
  plan->kernel_ = &kernel;
  plan->device_ = device;
  plan->workspace_bytes_ = kernel.workspace_bytes(problem);
  if (kernel.persistent_bytes) plan->persistent_bytes_ = kernel.persistent_bytes(problem);
  if (kernel.create_state) plan->state_ = kernel.create_state(problem);  // creates the C-ABI plan on `device`
  return plan;
}

ExecutionPlan::~ExecutionPlan() = default;

void ExecutionPlan::execute(const ConstTensorRef& x, const ConstTensorRef& w, const ConstTensorRef* bias, const TensorRef& y,
                            void* workspace, size_t workspace_bytes, cudaStream_t stream, cudaEvent_t* stage_events) const {
  const Conv2DParams& p = problem_.p;
  const DataType dt = problem_.dtype();
  require_tensor("input", x.data, x.dtype, x.shape, dt, p.input_shape());
  require_tensor("weights", w.data, w.dtype, w.shape, dt, p.weight_shape());
  require_tensor("output", y.data, y.dtype, y.shape, dt, p.output_shape());
  const void* bias_ptr = nullptr;
  if (problem_.has_bias) {
    GIE_REQUIRE(bias != nullptr, StatusCode::kInvalidArgument, "problem has_bias=true but no bias tensor was given");
    require_tensor("bias", bias->data, bias->dtype, bias->shape, dt, p.bias_shape());
    bias_ptr = bias->data;
  } else {
    GIE_REQUIRE(bias == nullptr || bias->data == nullptr, StatusCode::kInvalidArgument,
                "a bias tensor was given but the problem has has_bias=false");
  }
  const size_t es = dtype_size(dt);
  const size_t xb = size_t(p.input_shape().numel()) * es, wb = size_t(p.weight_shape().numel()) * es;
  const size_t yb = size_t(p.output_shape().numel()) * es, bb = size_t(p.out_channels) * es;
  GIE_REQUIRE(!ranges_overlap(y.data, yb, x.data, xb) && !ranges_overlap(y.data, yb, w.data, wb) && !ranges_overlap(y.data, yb, bias_ptr, bb),
              StatusCode::kInvalidArgument, "output aliases an input tensor (in-place convolution is not supported)");
  if (workspace_bytes_ > 0) {
    GIE_REQUIRE(reinterpret_cast<uintptr_t>(workspace) % 256 == 0, StatusCode::kInvalidArgument,
                "workspace must be 256-byte aligned");
    if (workspace == nullptr || workspace_bytes < workspace_bytes_)
      throw Error(StatusCode::kWorkspaceTooSmall, kernel_->name + " needs " + std::to_string(workspace_bytes_) +
                                                      " bytes of workspace, got " + std::to_string(workspace_bytes));
    GIE_REQUIRE(!ranges_overlap(workspace, workspace_bytes_, x.data, xb) && !ranges_overlap(workspace, workspace_bytes_, w.data, wb) &&
                    !ranges_overlap(workspace, workspace_bytes_, y.data, yb),
                StatusCode::kInvalidArgument, "workspace aliases a tensor");
  }
  int current = 0;
  GIE_CUDA_CHECK(cudaGetDevice(&current));
  GIE_REQUIRE(current == device_, StatusCode::kInvalidArgument,
              "plan was created for device " + std::to_string(device_) + " but device " + std::to_string(current) + " is current");
  execute_unchecked(x.data, w.data, bias_ptr, y.data, workspace, workspace_bytes, stream, stage_events);
}

void ExecutionPlan::execute_unchecked(const void* x, const void* w, const void* bias, void* y, void* workspace,
                                      size_t workspace_bytes, cudaStream_t stream, cudaEvent_t* stage_events) const {
  NvtxRange range(kernel_->name.c_str());
  LaunchArgs la;
  la.problem = &problem_;
  la.dev = nullptr;  // not needed by this family; avoids a mutex on the launch path
  la.x = x;
  la.w = w;
  la.bias = problem_.has_bias ? bias : nullptr;
  la.y = y;
  la.workspace = workspace;
  la.workspace_bytes = workspace_bytes;
  la.plan_state = state_.get();
  la.stream = stream;
  la.stage_events = stage_events;
  kernel_->launch(la);
}

// ---- plan cache + Conv2D ------------------------------------------------------------------------------------------------
namespace {

struct PlanKey {
  std::string problem, backend, kernel, cache;
  int device;
  bool autotune, retune;
  bool operator<(const PlanKey& o) const {
    return std::tie(problem, backend, kernel, device, autotune, retune, cache) <
           std::tie(o.problem, o.backend, o.kernel, o.device, o.autotune, o.retune, o.cache);
  }
};

std::mutex g_cache_mu;
std::map<PlanKey, std::shared_ptr<ExecutionPlan>>& cache() {
  static std::map<PlanKey, std::shared_ptr<ExecutionPlan>> c;
  return c;
}

std::shared_ptr<ExecutionPlan> plan_for(const ConvProblem& prob, const Conv2DOptions& opt) {
  validate_problem(prob);
  int dev = 0;
  GIE_CUDA_CHECK(cudaGetDevice(&dev));
  const PlanKey key{prob.key(), to_string(opt.backend), opt.kernel, opt.cache_path, dev, opt.autotune, opt.force_retune};
  {
    std::lock_guard<std::mutex> lock(g_cache_mu);
    auto it = cache().find(key);
    if (it != cache().end()) return it->second;
  }
  // creation may allocate and synchronise a private stream: keep it outside the lock; the first insert wins
  const Selection sel = Dispatcher::select(prob, DeviceInfo::get(dev), opt);
  std::shared_ptr<ExecutionPlan> plan = ExecutionPlan::create(prob, *sel.kernel, dev);
  std::lock_guard<std::mutex> lock(g_cache_mu);
  return cache().emplace(key, plan).first->second;
}

}  // namespace

void Conv2D::forward(const ConstTensorRef& input, const ConstTensorRef& weights, const ConstTensorRef* bias,
                     const ConvProblem& problem, const TensorRef& output, void* workspace, size_t workspace_bytes,
                     cudaStream_t stream, const Conv2DOptions& options) {
  plan_for(problem, options)->execute(input, weights, bias, output, workspace, workspace_bytes, stream);
}

size_t Conv2D::workspace_size(const ConvProblem& problem, const Conv2DOptions& options) {
  return plan_for(problem, options)->workspace_bytes();
}

void Conv2D::clear_plan_cache() {
  std::lock_guard<std::mutex> lock(g_cache_mu);
  cache().clear();
}

// ---- CUDA graphs ------------------------------------------------------------------------------------------------------
namespace {
double micros_since(std::chrono::steady_clock::time_point t0) {
  return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
}
struct PrivateStream {
  cudaStream_t s = nullptr;
  PrivateStream() { GIE_CUDA_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking)); }
  ~PrivateStream() { cudaStreamDestroy(s); }
};
}  // namespace

CudaGraphExecutor::~CudaGraphExecutor() { reset(); }

void CudaGraphExecutor::reset() {
  if (exec_ != nullptr) cudaGraphExecDestroy(exec_);
  if (graph_ != nullptr) cudaGraphDestroy(graph_);
  exec_ = nullptr;
  graph_ = nullptr;
  nodes_ = 0;
}

void CudaGraphExecutor::capture_graph(const Enqueue& enqueue, cudaGraph_t* g, double* us) {
  PrivateStream ps;
  const auto t0 = std::chrono::steady_clock::now();
  GIE_CUDA_CHECK(cudaStreamBeginCapture(ps.s, cudaStreamCaptureModeThreadLocal));
  try {
    enqueue(ps.s);
  } catch (...) {
    cudaGraph_t partial = nullptr;
    cudaStreamEndCapture(ps.s, &partial);  // end the capture so the stream stays usable; drop what was recorded
    if (partial != nullptr) cudaGraphDestroy(partial);
    (void)cudaGetLastError();
    throw;
  }
  GIE_CUDA_CHECK(cudaStreamEndCapture(ps.s, g));
  *us = micros_since(t0);
}

void CudaGraphExecutor::capture(const Enqueue& enqueue) {
  NvtxRange range("gie::CudaGraphExecutor::capture");
  reset();
  {
    PrivateStream warm;  // eager run: whatever initialises lazily does so outside capture
    enqueue(warm.s);
    GIE_CUDA_CHECK(cudaStreamSynchronize(warm.s));
  }
  capture_graph(enqueue, &graph_, &capture_us_);
  const auto t0 = std::chrono::steady_clock::now();
  GIE_CUDA_CHECK(cudaGraphInstantiate(&exec_, graph_, 0));
  instantiate_us_ = micros_since(t0);
  size_t n = 0;
  GIE_CUDA_CHECK(cudaGraphGetNodes(graph_, nullptr, &n));
  nodes_ = n;
}

bool CudaGraphExecutor::recapture_update(const Enqueue& enqueue) {
  if (exec_ == nullptr) {
    capture(enqueue);
    return false;
  }
  cudaGraph_t fresh = nullptr;
  capture_graph(enqueue, &fresh, &capture_us_);
  cudaGraphExecUpdateResultInfo info;
  const cudaError_t e = cudaGraphExecUpdate(exec_, fresh, &info);
  const bool in_place = e == cudaSuccess && info.result == cudaGraphExecUpdateSuccess;
  if (!in_place) {
    (void)cudaGetLastError();
    cudaGraphExecDestroy(exec_);
    exec_ = nullptr;
  }
  cudaGraphDestroy(graph_);
  graph_ = fresh;
  if (!in_place) {
    const auto t0 = std::chrono::steady_clock::now();
    GIE_CUDA_CHECK(cudaGraphInstantiate(&exec_, graph_, 0));
    instantiate_us_ = micros_since(t0);
  }
  size_t n = 0;
  GIE_CUDA_CHECK(cudaGraphGetNodes(graph_, nullptr, &n));
  nodes_ = n;
  return in_place;
}

void CudaGraphExecutor::launch(cudaStream_t stream) const {
  NvtxRange range("gie::CudaGraphExecutor::launch");
  GIE_REQUIRE(exec_ != nullptr, StatusCode::kInvalidArgument, "CudaGraphExecutor::launch before capture()");
  GIE_CUDA_CHECK(cudaGraphLaunch(exec_, stream));
}

// ---- RMSNorm and elementwise passes ---------------------------------------------------------------------------------------
void rmsnorm_forward(const RmsNormParams& p, const void* x, const void* gamma, void* y, const void* residual_in,
                     void* residual_out, cudaStream_t stream) {
  const gieb_rmsnorm_desc d = {p.rows, p.hidden, p.eps, int(p.dtype), 0u};
  const int rc = gieb_rmsnorm_launch(&d, x, gamma, y, residual_in, residual_out, stream);
  if (rc != GIEB_OK) throw Error(static_cast<StatusCode>(rc), gieb_last_error());
}

void launch_bias_act(const Conv2DParams& p, Precision prec, const void* bias_or_null, bool relu, void* y, cudaStream_t stream) {
  const int storage = prec == Precision::kFp16 ? 1 : (prec == Precision::kBf16 ? 2 : 0);
  const int rc = gieb_bias_act_launch(storage, p.batch, p.out_channels, p.out_h() * p.out_w(), bias_or_null, relu ? 1 : 0, y, stream);
  if (rc != GIEB_OK) throw Error(static_cast<StatusCode>(rc), gieb_last_error());
}
void launch_bias_add(const Conv2DParams& p, Precision prec, const void* bias, void* y, cudaStream_t stream) {
  launch_bias_act(p, prec, bias, false, y, stream);
}
void launch_relu(const Conv2DParams& p, Precision prec, void* y, cudaStream_t stream) { launch_bias_act(p, prec, nullptr, true, y, stream); }

}  // namespace gie
