// The one file a maintainer of the reference library adds to put the sm_100a kernel family behind its plug-in table:
// every KernelDesc (include/gpu_inference/kernel_registry.h:43-75 of the reference) forwards to the C ABI of
// libgie_b200.so.  It is written against the reference's OWN public headers and is compiled, together with the
// reference's unmodified host sources (src/runtime/*.cpp, src/autotuner/*.cpp), by build_refhost.py.
//
// The reference fills its table in src/runtime/registry.cpp:18-37 by calling one register_* function per legacy
// backend.  Built with GIE_B200_REPLACES_LEGACY_BACKENDS this file supplies those six symbols itself -- five register
// nothing, register_tensor_core_mma registers the family -- so registry.cpp is compiled as it is and the legacy
// kernels/*.cu are simply not part of the build.  Without the macro only register_b200_family() is defined, for a
// build that keeps the legacy backends and adds one call.
//
// Also here, because their reference implementations are CUDA kernels that this library replaces: rmsnorm_forward
// (src/transformer/rmsnorm.cu:155-166) and launch_bias_add / launch_relu / launch_bias_act
// (src/kernels/elementwise.cu:13-55).
#include <memory>
#include <mutex>
#include <set>
#include <sstream>
#include <string>
#include <vector>

#include "gie_b200.h"
#include "gie_b200_family.h"
#include "gpu_inference/error.h"
#include "gpu_inference/fused_ops.h"
#include "gpu_inference/kernel_registry.h"
#include "gpu_inference/rmsnorm.h"

namespace gie {
namespace kernels {
namespace {

gieb_conv_desc to_desc(const ConvProblem& pr) {
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

[[noreturn]] void rethrow(int status) { throw Error(static_cast<StatusCode>(status), gieb_last_error()); }

// Live plans, so that b200_device_status() can read their status words.  Both objects are never destroyed: plans held
// by the process-lifetime plan cache (src/runtime/conv2d.cpp:125-128) are released during static destruction, in an order
// this file does not control.
std::mutex& g_live_mu = *new std::mutex;
std::set<gieb_conv_plan*>& live_plans() {
  static std::set<gieb_conv_plan*>* s = new std::set<gieb_conv_plan*>;
  return *s;
}

struct PlanHandle {
  gieb_conv_plan* h = nullptr;
  ~PlanHandle() {
    if (h != nullptr) {
      std::lock_guard<std::mutex> lock(g_live_mu);
      live_plans().erase(h);
    }
    gieb_conv_plan_destroy(h);
  }
};

// One point of the family; all-zero = the library's own heuristic chooses tile, ring depth and split-K.
// RD: how split-K slices are summed (0 auto, 1 workspace + reduction launch, 2 thread-block cluster).
// PAIR: 2 = 256-pixel tiles computed by pairs of CTAs (tcgen05.mma.cta_group::2), 1 = single CTAs, 0 = auto.
template <int PREC, int TM, int TN, int TK, int ST, int SK, int RD = 0, int PAIR = 0>
struct Point {
  static const gieb_conv_cfg* cfg() {
    static const gieb_conv_cfg c = {TN, TK, ST, SK, 0, TM, RD, PAIR};
    return (TM | TN | TK | ST | SK | PAIR) ? &c : nullptr;
  }
  static gieb_conv_info query(const ConvProblem& pr, int device = -1) {
    const gieb_conv_desc d = to_desc(pr);
    gieb_conv_info info;
    if (gieb_conv_query(&d, cfg(), device, &info) != GIEB_OK) info.supported = 0;
    return info;
  }
  static bool supports(const ConvProblem& pr, const DeviceInfo& dev, std::string* why) {
    auto no = [&](const std::string& m) { if (why) *why = m; return false; };
    if (int(pr.precision) != PREC) return no(std::string("kernel is ") + to_string(static_cast<Precision>(PREC)) + " only");
    if (dev.cc_major != 10) return no("this kernel family is sm_100a code (device is sm_" + std::to_string(dev.cc()) + ")");
    const gieb_conv_info info = query(pr, dev.device);
    if (!info.supported) return no(info.reason[0] ? info.reason : "rejected by gieb_conv_query");
    return true;
  }
  static size_t workspace_bytes(const ConvProblem& pr) { return size_t(query(pr).workspace_bytes); }
  static size_t dynamic_smem_bytes(const ConvProblem& pr) { return size_t(query(pr).dynamic_smem_bytes); }
  static int64_t num_blocks(const ConvProblem& pr) { return query(pr).num_blocks; }
  static size_t persistent_bytes(const ConvProblem& pr) { return size_t(query(pr).persistent_bytes); }
  static double extra_traffic(const ConvProblem& pr) { return 2.0 * double(query(pr).workspace_bytes); }  // repacked copies written and read once
  static std::shared_ptr<void> create_state(const ConvProblem& pr) {  // ExecutionPlan::create (src/runtime/execution_plan.cpp:68)
    auto st = std::make_shared<PlanHandle>();
    const gieb_conv_desc d = to_desc(pr);
    const int rc = gieb_conv_plan_create(&d, cfg(), -1, &st->h);
    if (rc != GIEB_OK) rethrow(rc);
    {
      std::lock_guard<std::mutex> lock(g_live_mu);
      live_plans().insert(st->h);
    }
    return st;
  }
  static void launch(const LaunchArgs& la) {  // ExecutionPlan::execute_unchecked (src/runtime/execution_plan.cpp:137)
    auto* st = static_cast<PlanHandle*>(la.plan_state);
    if (st == nullptr || st->h == nullptr) throw Error(StatusCode::kInternal, "kernel launched without plan state");
    const int rc = gieb_conv_launch(st->h, la.x, la.w, la.bias, la.y, la.workspace, la.workspace_bytes, la.stream);
    if (rc != GIEB_OK) rethrow(rc);
  }
  static void add(std::vector<KernelDesc>& out) {
    const Precision prec = static_cast<Precision>(PREC);
    const bool simt = PREC == int(Precision::kFp32);
    KernelDesc k;
    std::ostringstream nm;
    if (simt) nm << "b200_simt_fp32";
    else if (cfg() == nullptr) nm << "b200_tc_" << to_string(prec) << "_auto";
    else nm << "b200_tc_" << to_string(prec) << "_" << (PAIR == 2 ? 256 : TM) << "x" << TN << "x" << TK << "_s" << ST << "_sk" << SK
            << (RD == 2 ? "c" : "") << (PAIR == 2 ? "_pair" : "");
    k.name = nm.str();
    k.backend = simt ? Backend::kImplicitGemm : Backend::kTensorCore;
    k.version = kLibraryVersion;
    k.params = {{"tile_pixels", PAIR == 2 ? 256 : TM}, {"tile_channels", TN}, {"tile_k", TK}, {"stages", ST}, {"split_k", SK},
                {"reduce", RD}, {"cta_pair", PAIR}};
    k.threads_per_block = simt ? 256 : 384;  // nominal: CTAs that own their SM run 640 threads (gieb_conv_info has the plan's value)
    k.tile_m = TN ? TN : 128;  // the reference's orientation: M = output channels, N = output pixels
    k.tile_n = PAIR == 2 ? 256 : (TM ? TM : 128);
    k.tile_k = TK ? TK : 64;
    k.uses_tensor_cores = !simt;
    k.launches = simt ? 1 : (SK > 1 && RD != 2 ? 3 : 2);
    // The heuristic entry is the one an un-tuned dispatcher should pick: it carries the highest prior.
    k.efficiency_prior = cfg() == nullptr ? 0.6 : 0.5;
    k.extra_traffic_bytes = &extra_traffic;
    k.supports = &supports;
    k.workspace_bytes = &workspace_bytes;
    k.dynamic_smem_bytes = &dynamic_smem_bytes;
    k.num_blocks = &num_blocks;
    k.create_state = &create_state;
    k.persistent_bytes = &persistent_bytes;
    k.launch = &launch;
    out.push_back(std::move(k));
  }
};

template <int PREC>
void add_family(std::vector<KernelDesc>& out) {
  Point<PREC, 0, 0, 0, 0, 0>::add(out);  // the heuristic entry: first, so that selection prefers it
  Point<PREC, 128, 32, 16, 4, 1>::add(out);
  Point<PREC, 128, 64, 32, 4, 1>::add(out);
  Point<PREC, 128, 64, 64, 3, 1>::add(out);
  Point<PREC, 128, 128, 64, 2, 1>::add(out);
  Point<PREC, 128, 128, 64, 3, 1>::add(out);
  Point<PREC, 128, 128, 64, 6, 1>::add(out);
  Point<PREC, 128, 256, 64, 2, 1>::add(out);
  Point<PREC, 128, 256, 64, 4, 1>::add(out);
  Point<PREC, 256, 64, 64, 2, 1>::add(out);
  Point<PREC, 256, 128, 64, 2, 1>::add(out);
  Point<PREC, 256, 128, 64, 3, 1>::add(out);
  Point<PREC, 256, 256, 64, 3, 1>::add(out);
  Point<PREC, 128, 64, 64, 4, 2>::add(out);
  Point<PREC, 128, 64, 64, 4, 4>::add(out);
  Point<PREC, 128, 128, 64, 4, 2>::add(out);
  Point<PREC, 128, 128, 64, 4, 8>::add(out);
  Point<PREC, 128, 256, 64, 4, 3>::add(out);
  Point<PREC, 128, 128, 64, 3, 2, 2>::add(out);  // the same slices summed inside a thread-block cluster
  Point<PREC, 128, 128, 64, 4, 4, 2>::add(out);
  Point<PREC, 128, 256, 64, 4, 2, 2>::add(out);
  Point<PREC, 128, 256, 64, 3, 4, 2>::add(out);
  Point<PREC, 0, 64, 64, 4, 1, 0, 2>::add(out);  // 256-pixel tiles of CTA pairs (cta_group::2)
  Point<PREC, 0, 128, 64, 6, 1, 0, 2>::add(out);
  Point<PREC, 0, 256, 64, 6, 1, 0, 2>::add(out);
  Point<PREC, 0, 256, 64, 4, 2, 1, 2>::add(out);
}

}  // namespace

uint32_t b200_device_status() {
  std::vector<gieb_conv_plan*> plans;
  {
    std::lock_guard<std::mutex> lock(g_live_mu);
    plans.assign(live_plans().begin(), live_plans().end());
  }
  uint32_t all = 0;
  for (gieb_conv_plan* pl : plans) {
    uint32_t v = 0;
    const int rc = gieb_conv_plan_device_status(pl, &v);
    if (rc != GIEB_OK) rethrow(rc);
    all |= v;
  }
  return all;
}

void register_b200_family(std::vector<KernelDesc>& out) {
  add_family<int(Precision::kFp16)>(out);
  add_family<int(Precision::kBf16)>(out);
  // FP32 storage on the tensor cores (kind::tf32): slab rows of 32 / 16 FP32 values
  Point<int(Precision::kTf32), 0, 0, 0, 0, 0>::add(out);
  Point<int(Precision::kTf32), 128, 64, 32, 4, 1>::add(out);
  Point<int(Precision::kTf32), 128, 128, 32, 3, 1>::add(out);
  Point<int(Precision::kTf32), 128, 256, 32, 3, 1>::add(out);
  Point<int(Precision::kTf32), 256, 128, 32, 2, 1>::add(out);
  Point<int(Precision::kTf32), 128, 128, 32, 4, 2>::add(out);
  Point<int(Precision::kTf32), 128, 128, 32, 3, 2, 2>::add(out);
  Point<int(Precision::kTf32), 128, 64, 16, 4, 1>::add(out);
  Point<int(Precision::kFp32), 0, 0, 0, 0, 0>::add(out);  // strict FP32: the SIMT kernel
}

#ifdef GIE_B200_REPLACES_LEGACY_BACKENDS
// The six slots src/runtime/registry.cpp:22-27 calls.  The legacy backends are not part of this build.
void register_direct(std::vector<KernelDesc>&) {}
void register_im2col(std::vector<KernelDesc>&) {}
void register_simt_tiled(std::vector<KernelDesc>&) {}
void register_implicit_gemm(std::vector<KernelDesc>&) {}
void register_tensor_core(std::vector<KernelDesc>&) {}
void register_tensor_core_mma(std::vector<KernelDesc>& out) { register_b200_family(out); }
#endif

}  // namespace kernels

// ---- operators whose reference implementations are kernels this library replaces --------------------------------------
namespace {
void check(int status) {
  if (status != GIEB_OK) throw Error(static_cast<StatusCode>(status), gieb_last_error());
}
}  // namespace

void rmsnorm_forward(const RmsNormParams& p, const void* x, const void* gamma, void* y, const void* residual_in, void* residual_out,
                     cudaStream_t stream) {
  const gieb_rmsnorm_desc d = {p.rows, p.hidden, p.eps, int(p.dtype), 0u};
  check(gieb_rmsnorm_launch(&d, x, gamma, y, residual_in, residual_out, stream));
}

// The reference's comparator that runs the residual add and the normalisation as separate passes
// (src/transformer/rmsnorm.cu:168-176).  Here: the element-wise add kernel (one rounding, as the residual stream is
// stored), then the same row kernel without a residual.  `scratch_rows_f32` is not needed.
void rmsnorm_forward_unfused(const RmsNormParams& p, const void* x, const void* gamma, void* y, const void* residual_in,
                             void* residual_out, void* scratch_rows_f32, cudaStream_t stream) {
  GIE_REQUIRE(p.rows > 0 && p.hidden > 0 && x && gamma && y && scratch_rows_f32, StatusCode::kInvalidArgument, "rmsnorm_unfused: bad arguments");
  const gieb_rmsnorm_desc d = {p.rows, p.hidden, p.eps, int(p.dtype), 0u};
  if (residual_in != nullptr && residual_out != nullptr) {
    check(gieb_add_relu_launch(int(p.dtype), 0, x, residual_in, residual_out, int64_t(p.rows) * p.hidden, stream));
    check(gieb_rmsnorm_launch(&d, residual_out, gamma, y, nullptr, nullptr, stream));
  } else {
    check(gieb_rmsnorm_launch(&d, x, gamma, y, nullptr, nullptr, stream));
  }
}

void launch_bias_act(const Conv2DParams& p, Precision prec, const void* bias_or_null, bool relu, void* y, cudaStream_t stream) {
  const int storage = prec == Precision::kTf32 ? int(Precision::kFp32) : int(prec);
  check(gieb_bias_act_launch(storage, p.batch, p.out_channels, p.out_h() * p.out_w(), bias_or_null, relu ? 1 : 0, y, stream));
}
void launch_bias_add(const Conv2DParams& p, Precision prec, const void* bias, void* y, cudaStream_t stream) {
  launch_bias_act(p, prec, bias, false, y, stream);
}
void launch_relu(const Conv2DParams& p, Precision prec, void* y, cudaStream_t stream) { launch_bias_act(p, prec, nullptr, true, y, stream); }

}  // namespace gie
