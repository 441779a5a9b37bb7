// The plug-in table: every KernelDesc forwards to the C ABI.  Entry 0..2 are the "auto" entries (the library's cost
// model picks tile / stages / split-K); the rest pin one point of the family each, which is what
// Conv2DOptions::kernel, find_kernel() and per-configuration tests address.
#include <set>
#include <sstream>

#include "gie_b200.h"
#include "gpu_inference/kernel_registry.h"

namespace gie {

gieb_conv_desc to_c_desc(const ConvProblem& pr);  // core.cpp

std::string KernelDesc::describe() const {
  std::ostringstream os;
  os << name << " [" << to_string(backend) << ", " << threads_per_block << " thr";
  for (const auto& kv : params) os << ", " << kv.first << "=" << kv.second;
  os << "]";
  return os.str();
}

namespace {

struct PlanHandle {
  gieb_conv_plan* h = nullptr;
  ~PlanHandle() { gieb_conv_plan_destroy(h); }
};

[[noreturn]] void rethrow(int status) { throw Error(static_cast<StatusCode>(status), gieb_last_error()); }

// One family point; all-zero = let the library choose.
// RD: how split-K slices are summed (0 auto, 1 workspace + reduction launch, 2 cluster / distributed shared memory).
template <int PREC, int TM, int TN, int TK, int ST, int SK, int RD = 0>
struct Point {
  static const gieb_conv_cfg* cfg() {
    static const gieb_conv_cfg c = {TN, TK, ST, SK, 0, TM, RD, 0};
    return (TM | TN | TK | ST | SK) ? &c : nullptr;
  }
  static gieb_conv_info query(const ConvProblem& pr, int device = -1) {
    const gieb_conv_desc d = to_c_desc(pr);
    gieb_conv_info info;
    const int st = gieb_conv_query(&d, cfg(), device, &info);
    if (st != GIEB_OK) info.supported = 0;
    return info;
  }
  static bool supports(const ConvProblem& pr, const DeviceInfo& dev, std::string* why) {
    auto no = [&](const std::string& m) { if (why) *why = m; return false; };
    if (int(pr.precision) != PREC) return no(std::string("kernel is ") + to_string(static_cast<Precision>(PREC)) + " only");
    if (!dev.supports_tcgen05()) return no("this library contains sm_100a code only (device is sm_" + std::to_string(dev.cc()) + ")");
    const gieb_conv_info info = query(pr, dev.device);
    if (!info.supported) return no(info.reason[0] ? info.reason : "rejected by gieb_conv_query");
    return true;
  }
  static size_t workspace_bytes(const ConvProblem& pr) { return size_t(query(pr).workspace_bytes); }
  static size_t dynamic_smem_bytes(const ConvProblem& pr) { return size_t(query(pr).dynamic_smem_bytes); }
  static int64_t num_blocks(const ConvProblem& pr) { return query(pr).num_blocks; }
  static size_t persistent_bytes(const ConvProblem& pr) { return size_t(query(pr).persistent_bytes); }
  static double extra_traffic(const ConvProblem& pr) {  // repack reads + writes X and W once more; split-K partials
    const gieb_conv_info info = query(pr);
    return 2.0 * double(info.workspace_bytes);
  }
  static std::shared_ptr<void> create_state(const ConvProblem& pr) {
    auto st = std::make_shared<PlanHandle>();
    const gieb_conv_desc d = to_c_desc(pr);
    const int rc = gieb_conv_plan_create(&d, cfg(), -1, &st->h);
    if (rc != GIEB_OK) rethrow(rc);
    return st;
  }
  static double estimate_us(const ConvProblem& pr) {
    const gieb_conv_desc d = to_c_desc(pr);
    double us = 0;
    return gieb_conv_estimate_us(&d, cfg(), &us) == GIEB_OK ? us : 1e30;
  }
  static void launch(const LaunchArgs& la) {
    auto* st = static_cast<PlanHandle*>(la.plan_state);
    if (st == nullptr || st->h == nullptr) throw Error(StatusCode::kInternal, "kernel launched without plan state");
    const int rc = gieb_conv_launch(st->h, la.x, la.w, la.bias, la.y, la.workspace, la.workspace_bytes, la.stream);
    if (rc != GIEB_OK) rethrow(rc);
  }
  static void add(std::vector<KernelDesc>& out) {
    const Precision prec = static_cast<Precision>(PREC);
    KernelDesc k;
    std::ostringstream nm;
    if (PREC == int(Precision::kFp32)) nm << "b200_simt_fp32";
    else if (cfg() == nullptr) nm << "b200_tc_" << to_string(prec) << "_auto";
    else nm << "b200_tc_" << to_string(prec) << "_" << TM << "x" << TN << "x" << TK << "_s" << ST << "_sk" << SK << (RD == 2 ? "c" : "");
    k.name = nm.str();
    k.backend = PREC == int(Precision::kFp32) ? Backend::kImplicitGemm : Backend::kTensorCore;
    k.version = kLibraryVersion;
    k.params = {{"tile_pixels", TM}, {"tile_channels", TN}, {"tile_k", TK}, {"stages", ST}, {"split_k", SK}, {"reduce", RD}};
    k.threads_per_block = PREC == int(Precision::kFp32) ? 256 : 384;  // nominal: a plan whose CTAs own their SM runs 640 (gieb_conv_info reports it)
    k.tile_m = TN ? TN : 128;   // reference orientation: M = output channels
    k.tile_n = TM ? TM : 128;   //                        N = output pixels
    k.tile_k = TK ? TK : 64;
    k.uses_tensor_cores = PREC != int(Precision::kFp32);
    k.launches = PREC == int(Precision::kFp32) ? 1 : (SK > 1 && RD != 2 ? 3 : 2);
    k.efficiency_prior = 0.5;
    k.extra_traffic_bytes = &extra_traffic;
    k.supports = &supports;
    k.workspace_bytes = &workspace_bytes;
    k.dynamic_smem_bytes = &dynamic_smem_bytes;
    k.num_blocks = &num_blocks;
    k.create_state = &create_state;
    k.persistent_bytes = &persistent_bytes;
    k.launch = &launch;
    k.estimate_us = &estimate_us;
    out.push_back(std::move(k));
  }
};

template <int PREC>
void add_family(std::vector<KernelDesc>& out) {
  Point<PREC, 0, 0, 0, 0, 0>::add(out);  // auto: must stay first so that selection prefers it
  Point<PREC, 128, 32, 16, 4, 1>::add(out);
  Point<PREC, 128, 64, 32, 4, 1>::add(out);
  Point<PREC, 128, 64, 64, 3, 1>::add(out);
  Point<PREC, 128, 128, 64, 2, 1>::add(out);
  Point<PREC, 128, 128, 64, 3, 1>::add(out);
  Point<PREC, 128, 128, 64, 6, 1>::add(out);
  Point<PREC, 128, 256, 64, 2, 1>::add(out);
  Point<PREC, 128, 256, 64, 4, 1>::add(out);
  Point<PREC, 256, 128, 64, 2, 1>::add(out);
  Point<PREC, 256, 256, 64, 3, 1>::add(out);
  Point<PREC, 128, 64, 64, 4, 2>::add(out);
  Point<PREC, 128, 64, 64, 4, 4>::add(out);
  Point<PREC, 128, 128, 64, 4, 8>::add(out);
  Point<PREC, 128, 256, 64, 4, 3>::add(out);
  Point<PREC, 128, 128, 64, 4, 2>::add(out);
  Point<PREC, 128, 128, 64, 3, 2, 2>::add(out);  // the same slices summed inside a cluster
  Point<PREC, 128, 128, 64, 4, 4, 2>::add(out);
  Point<PREC, 128, 256, 64, 4, 2, 2>::add(out);
  Point<PREC, 128, 256, 64, 3, 4, 2>::add(out);
  Point<PREC, 256, 64, 64, 2, 1>::add(out);
  Point<PREC, 256, 128, 64, 3, 1>::add(out);
}

std::vector<KernelDesc>& storage() {
  static std::vector<KernelDesc> reg = [] {
    std::vector<KernelDesc> r;
    r.reserve(256);  // element addresses stay valid when a test appends entries
    add_family<int(Precision::kFp16)>(r);
    add_family<int(Precision::kBf16)>(r);
    // FP32 storage on the tensor cores (kind::tf32): slab rows of 32 / 16 FP32 values
    Point<int(Precision::kTf32), 0, 0, 0, 0, 0>::add(r);
    Point<int(Precision::kTf32), 128, 64, 32, 4, 1>::add(r);
    Point<int(Precision::kTf32), 128, 128, 32, 3, 1>::add(r);
    Point<int(Precision::kTf32), 128, 256, 32, 3, 1>::add(r);
    Point<int(Precision::kTf32), 256, 128, 32, 2, 1>::add(r);
    Point<int(Precision::kTf32), 128, 128, 32, 4, 2>::add(r);
    Point<int(Precision::kTf32), 128, 128, 32, 3, 2, 2>::add(r);
    Point<int(Precision::kTf32), 128, 64, 16, 4, 1>::add(r);
    Point<int(Precision::kFp32), 0, 0, 0, 0, 0>::add(r);
    std::set<std::string> names;
    for (const KernelDesc& k : r)
      if (!names.insert(k.name).second) throw Error(StatusCode::kInternal, "duplicate kernel name " + k.name);
    return r;
  }();
  return reg;
}

}  // namespace

const std::vector<KernelDesc>& kernel_registry() { return storage(); }
std::vector<KernelDesc>& kernel_registry_for_testing() { return storage(); }

const KernelDesc* find_kernel(const std::string& name) {
  for (const KernelDesc& k : storage())
    if (k.name == name) return &k;
  return nullptr;
}

std::vector<const KernelDesc*> kernels_for_backend(Backend b) {
  std::vector<const KernelDesc*> out;
  for (const KernelDesc& k : storage())
    if (b == Backend::kAuto || k.backend == b) out.push_back(&k);
  return out;
}

// ---- offset tables kept for source compatibility ----------------------------------------------------------------
std::vector<LutEntry> build_conv_lut(const Conv2DParams& p) {
  std::vector<LutEntry> lut;
  lut.reserve(size_t(p.gemm_k()));
  for (int c = 0; c < p.in_channels; ++c)
    for (int r = 0; r < p.kernel_h; ++r)
      for (int s = 0; s < p.kernel_w; ++s) lut.push_back({c * p.in_h * p.in_w, r * p.dilation_h, s * p.dilation_w, 0});
  return lut;
}

std::vector<LutEntry> build_conv_lut_chunked(const Conv2DParams& p) {
  GIE_REQUIRE(p.in_channels % 8 == 0, StatusCode::kInvalidArgument, "the chunked table needs C_in % 8 == 0");
  const int chunks = p.in_channels / 8;
  std::vector<LutEntry> lut;
  lut.reserve(size_t(p.kernel_h) * p.kernel_w * chunks);
  for (int r = 0; r < p.kernel_h; ++r)
    for (int s = 0; s < p.kernel_w; ++s)
      for (int q = 0; q < chunks; ++q) lut.push_back({8 * q, r * p.dilation_h, s * p.dilation_w, 0});
  return lut;
}

}  // namespace gie
