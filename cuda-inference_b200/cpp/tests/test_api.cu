// GPU tests of the C++ operator layer (namespace gie) running on the sm_100a library.  They restate, against this
// library's registry, the hot-path subset of the reference's test programs: tests/test_validation.cpp,
// test_dispatcher.cpp, test_tensor_core.cpp / test_implicit_gemm.cpp (suite protocol of conv_test_common.h),
// test_fusion.cpp, test_cuda_graph.cu, test_runtime_concurrency.cu and test_rmsnorm.cpp.
#include <atomic>
#include <chrono>
#include <cmath>
#include <thread>

#include <unistd.h>

#include <fstream>

#include "gie_b200_family.h"
#include "gpu_inference/autotuner.h"
#include "gpu_inference/cuda_graph.h"
#include "gpu_inference/fused_ops.h"
#include "gpu_inference/rmsnorm.h"
#include "test_support.h"

using namespace gie;

// ---------------------------------------------------------------------------------------------------------------
// argument validation (tests/test_validation.cpp:23-95): exact status codes
// ---------------------------------------------------------------------------------------------------------------
namespace {
struct Fixture {
  ConvProblem prob = ts::problem(ts::geom(2, 8, 10, 10, 8, 3, 3, 1, 1, 1, 1), Precision::kFp16, true, false);
  ConvData d = make_conv_data(prob, 1);
  const KernelDesc* k = find_kernel("b200_tc_fp16_auto");
  std::shared_ptr<ExecutionPlan> plan = ExecutionPlan::create(prob, *k);
  DeviceBuffer ws{plan->workspace_bytes()};
};
}  // namespace

CASE(valid_call_succeeds) {
  Fixture f;
  const ConstTensorRef bias = f.d.b_ref();
  f.plan->execute(f.d.x_ref(), f.d.w_ref(), &bias, f.d.y_ref(), f.ws.data(), f.ws.size(), nullptr);
  GIE_CUDA_CHECK(cudaDeviceSynchronize());
  EXPECT(f.plan->workspace_bytes() > 0);
  EXPECT(f.plan->device() == 0 || f.plan->device() > 0);
  EXPECT(&f.plan->kernel() == f.k);
}

CASE(rejects_null_pointers_and_bad_shapes) {
  Fixture f;
  const ConstTensorRef bias = f.d.b_ref();
  ConstTensorRef x = f.d.x_ref();
  x.data = nullptr;
  EXPECT_THROWS(f.plan->execute(x, f.d.w_ref(), &bias, f.d.y_ref(), f.ws.data(), f.ws.size(), nullptr), StatusCode::kInvalidArgument);
  x = f.d.x_ref();
  x.shape.h += 1;
  EXPECT_THROWS(f.plan->execute(x, f.d.w_ref(), &bias, f.d.y_ref(), f.ws.data(), f.ws.size(), nullptr), StatusCode::kInvalidArgument);
  ConstTensorRef w = f.d.w_ref();
  w.dtype = DataType::kFloat32;
  EXPECT_THROWS(f.plan->execute(f.d.x_ref(), w, &bias, f.d.y_ref(), f.ws.data(), f.ws.size(), nullptr), StatusCode::kInvalidArgument);
  TensorRef y = f.d.y_ref();
  y.shape.c += 1;
  EXPECT_THROWS(f.plan->execute(f.d.x_ref(), f.d.w_ref(), &bias, y, f.ws.data(), f.ws.size(), nullptr), StatusCode::kInvalidArgument);
}

CASE(rejects_bias_mismatch) {
  Fixture f;
  EXPECT_THROWS(f.plan->execute(f.d.x_ref(), f.d.w_ref(), nullptr, f.d.y_ref(), f.ws.data(), f.ws.size(), nullptr), StatusCode::kInvalidArgument);
  ConvProblem nb = f.prob;
  nb.has_bias = false;
  auto plan = ExecutionPlan::create(nb, *f.k);
  const ConstTensorRef bias = f.d.b_ref();
  EXPECT_THROWS(plan->execute(f.d.x_ref(), f.d.w_ref(), &bias, f.d.y_ref(), f.ws.data(), f.ws.size(), nullptr), StatusCode::kInvalidArgument);
  ConstTensorRef bad = f.d.b_ref();
  bad.shape.c = 3;
  EXPECT_THROWS(f.plan->execute(f.d.x_ref(), f.d.w_ref(), &bad, f.d.y_ref(), f.ws.data(), f.ws.size(), nullptr), StatusCode::kInvalidArgument);
}

CASE(rejects_output_aliasing_inputs) {
  Fixture f;
  const ConstTensorRef bias = f.d.b_ref();
  TensorRef y = f.d.y_ref();
  y.data = f.d.dx.data();
  EXPECT_THROWS(f.plan->execute(f.d.x_ref(), f.d.w_ref(), &bias, y, f.ws.data(), f.ws.size(), nullptr), StatusCode::kInvalidArgument);
  DeviceBuffer big(size_t(f.prob.p.output_shape().numel()) * 2 + 4096);
  TensorRef y2 = f.d.y_ref();
  y2.data = big.data();
  ConstTensorRef x2 = f.d.x_ref();
  x2.data = static_cast<char*>(big.data()) + 1024;  // the input starts inside the output range
  EXPECT_THROWS(f.plan->execute(x2, f.d.w_ref(), &bias, y2, f.ws.data(), f.ws.size(), nullptr), StatusCode::kInvalidArgument);
  TensorRef y3 = f.d.y_ref();
  y3.data = f.ws.data();                            // output inside the workspace
  EXPECT_THROWS(f.plan->execute(f.d.x_ref(), f.d.w_ref(), &bias, y3, f.ws.data(), f.ws.size(), nullptr), StatusCode::kInvalidArgument);
}

CASE(rejects_small_missing_or_misaligned_workspace) {
  Fixture f;
  const ConstTensorRef bias = f.d.b_ref();
  EXPECT_THROWS(f.plan->execute(f.d.x_ref(), f.d.w_ref(), &bias, f.d.y_ref(), nullptr, 0, nullptr), StatusCode::kWorkspaceTooSmall);
  EXPECT_THROWS(f.plan->execute(f.d.x_ref(), f.d.w_ref(), &bias, f.d.y_ref(), f.ws.data(), f.ws.size() - 1, nullptr), StatusCode::kWorkspaceTooSmall);
  DeviceBuffer odd(f.ws.size() + 512);
  EXPECT_THROWS(f.plan->execute(f.d.x_ref(), f.d.w_ref(), &bias, f.d.y_ref(), static_cast<char*>(odd.data()) + 16, f.ws.size(), nullptr),
                StatusCode::kInvalidArgument);
}

CASE(plan_rejects_unsupported_kernel_precision_combo) {
  const ConvProblem fp32 = ts::problem(ts::geom(1, 8, 8, 8, 8, 3, 3, 1, 1, 1, 1), Precision::kFp32, false, false);
  EXPECT_THROWS(ExecutionPlan::create(fp32, *find_kernel("b200_tc_fp16_128x128x64_s3_sk1")), StatusCode::kUnsupported);
  const ConvProblem tf32 = ts::problem(ts::geom(1, 8, 8, 8, 8, 3, 3, 1, 1, 1, 1), Precision::kTf32, false, false);
  EXPECT_THROWS(ExecutionPlan::create(tf32, *find_kernel("b200_simt_fp32")), StatusCode::kUnsupported);
  ConvProblem dil = fp32;
  dil.p.dilation_h = 2;
  EXPECT_THROWS(validate_problem(dil), StatusCode::kUnsupported);
  ConvProblem empty = fp32;
  empty.p.batch = 0;
  EXPECT_THROWS(validate_problem(empty), StatusCode::kInvalidArgument);
}

CASE(forward_api_end_to_end_with_validation) {
  for (Precision prec : {Precision::kFp32, Precision::kFp16, Precision::kBf16}) {
    const ConvProblem prob = ts::problem(ts::geom(2, 8, 10, 10, 8, 3, 3, 1, 1, 1, 1), prec, true, true);
    ts::Bundle b = ts::make_bundle(prob, 3, Distribution::kNormal);
    const size_t need = Conv2D::workspace_size(prob);
    DeviceBuffer ws(need);
    const ConstTensorRef bias = b.data.b_ref();
    if (need > 0)
      EXPECT_THROWS(Conv2D::forward(b.data.x_ref(), b.data.w_ref(), &bias, prob, b.data.y_ref(), nullptr, 0, nullptr), StatusCode::kWorkspaceTooSmall);
    Conv2D::forward(b.data.x_ref(), b.data.w_ref(), &bias, prob, b.data.y_ref(), ws.data(), ws.size(), nullptr);
    GIE_CUDA_CHECK(cudaDeviceSynchronize());
    const ErrorMetrics m = ts::compare_device(b.data.dy.data(), b);
    EXPECT_MSG(m.passed(), std::string(to_string(prec)) + " " + m.summary());
  }
  Conv2D::clear_plan_cache();
}

// ---------------------------------------------------------------------------------------------------------------
// selection (tests/test_dispatcher.cpp subset that applies to one kernel family)
// ---------------------------------------------------------------------------------------------------------------
CASE(selection_routes_by_precision_and_honours_forced_kernels) {
  const DeviceInfo& dev = DeviceInfo::current();
  EXPECT(dev.cc_major == 10);  // the family is sm_100a code
  const Conv2DParams g = ts::geom(4, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1);
  Conv2DOptions opt;
  Selection s = Dispatcher::select(ts::problem(g, Precision::kFp16, true, true), dev, opt);
  EXPECT(s.kernel != nullptr && s.kernel->backend == Backend::kTensorCore && s.kernel->uses_tensor_cores);
  EXPECT(s.source == SelectionSource::kCostModel);
  s = Dispatcher::select(ts::problem(g, Precision::kFp32, true, true), dev, opt);
  EXPECT(s.kernel != nullptr && s.kernel->backend == Backend::kImplicitGemm && !s.kernel->uses_tensor_cores);
  opt.kernel = "b200_tc_bf16_128x64x64_s3_sk1";
  s = Dispatcher::select(ts::problem(g, Precision::kBf16, true, true), dev, opt);
  EXPECT(s.source == SelectionSource::kForcedKernel && s.kernel->name == opt.kernel);
  EXPECT_THROWS(Dispatcher::select(ts::problem(g, Precision::kFp16, true, true), dev, opt), StatusCode::kUnsupported);  // bf16 kernel, fp16 problem
  opt.kernel = "no_such_kernel";
  EXPECT_THROWS(Dispatcher::select(ts::problem(g, Precision::kFp16, true, true), dev, opt), StatusCode::kInvalidArgument);
  opt.kernel.clear();
  opt.backend = Backend::kTensorCore;
  s = Dispatcher::select(ts::problem(g, Precision::kFp16, true, true), dev, opt);
  EXPECT(s.source == SelectionSource::kForcedBackend);
  for (Backend b : {Backend::kDirect, Backend::kIm2colGemm, Backend::kSimtTiled, Backend::kCpuReference}) {
    opt.backend = b;
    EXPECT_THROWS(Dispatcher::select(ts::problem(g, Precision::kFp16, true, true), dev, opt), StatusCode::kUnsupported);
  }
  opt.backend = Backend::kTensorCore;  // FP32 has no tensor-core kernel here (TF32 is not offered)
  EXPECT_THROWS(Dispatcher::select(ts::problem(g, Precision::kFp32, true, true), dev, opt), StatusCode::kUnsupported);
  std::vector<Rejection> rej;
  const auto ok = Dispatcher::compatible_kernels(ts::problem(g, Precision::kFp16, true, true), dev, Backend::kAuto, &rej);
  EXPECT(!ok.empty() && !rej.empty());
  for (const Rejection& r : rej) EXPECT(!r.reason.empty());
  // names, string round trips
  EXPECT(backend_from_string("tensor_core") == Backend::kTensorCore && precision_from_string("bf16") == Precision::kBf16);
  EXPECT_THROWS(precision_from_string("fp8"), StatusCode::kInvalidArgument);
  EXPECT(std::string(to_string(StatusCode::kWorkspaceTooSmall)) == "WorkspaceTooSmall");
}

CASE(plan_cache_reuses_plans) {
  Conv2D::clear_plan_cache();
  const ConvProblem prob = ts::problem(ts::geom(2, 16, 12, 12, 16, 3, 3, 1, 1, 1, 1), Precision::kFp16, false, false);
  const auto t0 = std::chrono::steady_clock::now();
  const size_t a = Conv2D::workspace_size(prob);
  const auto t1 = std::chrono::steady_clock::now();
  size_t b = 0;
  for (int i = 0; i < 100; ++i) b = Conv2D::workspace_size(prob);
  const auto t2 = std::chrono::steady_clock::now();
  EXPECT(a == b && a > 0);
  const double first = std::chrono::duration<double, std::micro>(t1 - t0).count();
  const double later = std::chrono::duration<double, std::micro>(t2 - t1).count() / 100.0;
  EXPECT_MSG(later < first, "cached look-ups must be cheaper than plan creation");
}

CASE(device_status_of_live_plans_is_clear_after_forward_calls) {
  // the family's own accessor: no bounded device-side wait has run out in any plan that is still alive
  const ConvProblem prob = ts::problem(ts::geom(2, 32, 12, 12, 48, 3, 3, 1, 1, 1, 1), Precision::kFp16, true, true);
  ts::Bundle b = ts::make_bundle(prob, 77, Distribution::kUniform);
  bool ran = false;
  const ErrorMetrics m = ts::run_kernel(*find_kernel("b200_tc_fp16_auto"), b, &ran, nullptr);
  EXPECT(ran && m.passed());
  auto plan = ExecutionPlan::create(prob, *find_kernel("b200_tc_fp16_256x128x64_s6_sk1_pair"));  // stays alive across the query
  GIE_CUDA_CHECK(cudaDeviceSynchronize());
  EXPECT(kernels::b200_device_status() == 0u);
}

// ---------------------------------------------------------------------------------------------------------------
// correctness suite (protocol of tests/conv_test_common.h:84-127)
// ---------------------------------------------------------------------------------------------------------------
CASE(suite_every_shape_every_precision_has_a_passing_kernel) {
  const Distribution dists[4] = {Distribution::kUniform, Distribution::kNormal, Distribution::kSparseSigned, Distribution::kPositive};
  int cell = 0, runs = 0;
  for (const ts::NamedShape& sh : ts::shapes()) {
    for (Precision prec : {Precision::kFp32, Precision::kFp16, Precision::kBf16, Precision::kTf32}) {
      const int mode = cell % 3;
      ++cell;
      const ConvProblem prob = ts::problem(sh.p, prec, mode >= 1, mode == 2);
      ts::Bundle b = ts::make_bundle(prob, 0xC0FFEEULL + uint64_t(cell), dists[cell % 4]);
      int ran_here = 0;
      for (const KernelDesc* k : kernels_for_backend(Backend::kAuto)) {
        if (k->name.find("auto") == std::string::npos && k->name != "b200_simt_fp32" && sh.p.flops() > 400000000) continue;
        bool ran = false;
        std::string why;
        const ErrorMetrics m = ts::run_kernel(*k, b, &ran, &why);
        if (!ran) continue;
        ++ran_here;
        ++runs;
        EXPECT_MSG(m.passed(), k->name + " on " + sh.name + " " + prob.key() + " -> " + m.summary());
      }
      EXPECT_MSG(ran_here > 0, std::string("no kernel could run ") + sh.name + " " + prob.key());
    }
  }
  std::printf("  %d kernel runs verified\n", runs);
  EXPECT(runs > 100);
}

CASE(relu_outputs_are_exact_zeros) {  // tests/test_fusion.cpp:15-30
  const ConvProblem prob = ts::problem(ts::geom(2, 32, 10, 10, 32, 3, 3, 1, 1, 1, 1), Precision::kFp16, true, true);
  ts::Bundle b = ts::make_bundle(prob, 9, Distribution::kNormal);
  ConvProblem lin = prob;
  lin.activation = Activation::kNone;
  ReferenceOutput pre;
  cpu_conv2d_reference(lin, b.data.hx.data(), b.data.hw.data(), b.data.hb.data(), &pre);
  bool ran = false;
  const ErrorMetrics m = ts::run_kernel(*find_kernel("b200_tc_fp16_auto"), b, &ran, nullptr);
  EXPECT(ran && m.passed());
  const std::vector<float> y = download_as_float(b.data.dy.data(), prob.dtype(), prob.p.output_shape().numel());
  int zeros = 0;
  for (size_t i = 0; i < y.size(); ++i) {
    EXPECT(y[i] >= 0.f);
    if (pre.y[i] < -1e-2f) { EXPECT(y[i] == 0.f); ++zeros; }
  }
  EXPECT(zeros > 100);
}

CASE(fp32_fused_epilogue_equals_unfused_bitwise) {  // tests/test_fusion.cpp:34-58
  const Conv2DParams g = ts::geom(2, 16, 12, 12, 24, 3, 3, 1, 1, 1, 1);
  const ConvProblem fused = ts::problem(g, Precision::kFp32, true, true), plain = ts::problem(g, Precision::kFp32, false, false);
  ts::Bundle b = ts::make_bundle(fused, 31, Distribution::kNormal);
  const KernelDesc* k = find_kernel("b200_simt_fp32");
  const size_t bytes = b.data.dy.size();
  auto pf = ExecutionPlan::create(fused, *k), pp = ExecutionPlan::create(plain, *k);
  DeviceBuffer y2(bytes);
  pf->execute_unchecked(b.data.dx.data(), b.data.dw.data(), b.data.db.data(), b.data.dy.data(), nullptr, 0, nullptr);
  pp->execute_unchecked(b.data.dx.data(), b.data.dw.data(), nullptr, y2.data(), nullptr, 0, nullptr);
  launch_bias_add(g, Precision::kFp32, b.data.db.data(), y2.data(), nullptr);
  launch_relu(g, Precision::kFp32, y2.data(), nullptr);
  GIE_CUDA_CHECK(cudaDeviceSynchronize());
  EXPECT(ts::download_bytes(b.data.dy.data(), bytes) == ts::download_bytes(y2.data(), bytes));
}

// ---------------------------------------------------------------------------------------------------------------
// CUDA graphs (tests/test_cuda_graph.cu:42-137)
// ---------------------------------------------------------------------------------------------------------------
namespace {
void copy_inputs_async(ts::Bundle& dst, const ts::Bundle& src, cudaStream_t s) {
  GIE_CUDA_CHECK(cudaMemcpyAsync(dst.data.dx.data(), src.data.dx.data(), src.data.dx.size(), cudaMemcpyDeviceToDevice, s));
  GIE_CUDA_CHECK(cudaMemcpyAsync(dst.data.dw.data(), src.data.dw.data(), src.data.dw.size(), cudaMemcpyDeviceToDevice, s));
  GIE_CUDA_CHECK(cudaMemcpyAsync(dst.data.db.data(), src.data.db.data(), src.data.db.size(), cudaMemcpyDeviceToDevice, s));
}
}  // namespace

CASE(graph_replay_with_changing_inputs_on_alternating_streams) {
  const ConvProblem prob = ts::problem(ts::geom(4, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), Precision::kFp16, true, true);
  ts::Bundle live = ts::make_bundle(prob, 100);
  std::vector<ts::Bundle> others;
  for (int i = 0; i < 3; ++i) others.push_back(ts::make_bundle(prob, 200 + i, i % 2 ? Distribution::kNormal : Distribution::kUniform));
  auto plan = ExecutionPlan::create(prob, *find_kernel("b200_tc_fp16_auto"));  // creation allocates: before capture
  DeviceBuffer ws(plan->workspace_bytes());
  CudaGraphExecutor g;
  g.capture([&](cudaStream_t s) {
    plan->execute_unchecked(live.data.dx.data(), live.data.dw.data(), live.data.db.data(), live.data.dy.data(), ws.data(), ws.size(), s);
  });
  EXPECT(g.valid() && g.node_count() == 2);  // repack + convolution
  cudaStream_t st[2];
  for (auto& s : st) GIE_CUDA_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  for (int i = 0; i < 3; ++i) {
    cudaStream_t s = st[i % 2];
    copy_inputs_async(live, others[size_t(i)], s);
    GIE_CUDA_CHECK(cudaMemsetAsync(live.data.dy.data(), 0xFF, live.data.dy.size(), s));
    g.launch(s);
    GIE_CUDA_CHECK(cudaStreamSynchronize(s));
    const ErrorMetrics m = ts::compare_device(live.data.dy.data(), others[size_t(i)]);
    EXPECT_MSG(m.passed(), m.summary());
  }
  for (auto& s : st) cudaStreamDestroy(s);
}

CASE(graph_node_counts_and_in_place_update) {
  const ConvProblem prob = ts::problem(ts::geom(1, 512, 7, 7, 512, 3, 3, 1, 1, 1, 1), Precision::kFp16, true, true);
  ts::Bundle a = ts::make_bundle(prob, 7), b = ts::make_bundle(prob, 8);
  auto split = ExecutionPlan::create(prob, *find_kernel("b200_tc_fp16_128x128x64_s4_sk8"));
  DeviceBuffer ws(split->workspace_bytes());
  CudaGraphExecutor g;
  EXPECT_THROWS(g.launch(nullptr), StatusCode::kInvalidArgument);
  ts::Bundle* cur = &a;
  auto enqueue = [&](cudaStream_t s) {
    split->execute_unchecked(cur->data.dx.data(), cur->data.dw.data(), cur->data.db.data(), cur->data.dy.data(), ws.data(), ws.size(), s);
  };
  g.capture(enqueue);
  EXPECT(g.node_count() == 3);  // repack + convolution + split-K reduction
  g.launch(nullptr);
  GIE_CUDA_CHECK(cudaDeviceSynchronize());
  EXPECT(ts::compare_device(a.data.dy.data(), a).passed());
  cur = &b;  // same topology, other buffers: patched in place
  const bool in_place = g.recapture_update(enqueue);
  EXPECT(in_place);
  g.launch(nullptr);
  GIE_CUDA_CHECK(cudaDeviceSynchronize());
  EXPECT(ts::compare_device(b.data.dy.data(), b).passed());
  // a callable that throws during capture leaves the executor and the thread usable
  CudaGraphExecutor bad;
  EXPECT_THROWS(bad.capture([&](cudaStream_t) { throw Error(StatusCode::kInternal, "boom"); }), StatusCode::kInternal);
  g.launch(nullptr);
  GIE_CUDA_CHECK(cudaDeviceSynchronize());
}

CASE(graph_of_a_four_layer_chain_equals_eager_bitwise) {
  const ConvProblem prob = ts::problem(ts::geom(4, 64, 14, 14, 64, 3, 3, 1, 1, 1, 1), Precision::kBf16, true, true);
  ts::Bundle b = ts::make_bundle(prob, 55);
  auto plan = ExecutionPlan::create(prob, *find_kernel("b200_tc_bf16_auto"));
  DeviceBuffer ws(plan->workspace_bytes()), ping(b.data.dx.size()), pong(b.data.dx.size()), eager(b.data.dx.size());
  auto chain = [&](cudaStream_t s) {
    GIE_CUDA_CHECK(cudaMemcpyAsync(ping.data(), b.data.dx.data(), b.data.dx.size(), cudaMemcpyDeviceToDevice, s));
    void* src = ping.data();
    void* dst = pong.data();
    for (int l = 0; l < 4; ++l) {
      plan->execute_unchecked(src, b.data.dw.data(), b.data.db.data(), dst, ws.data(), ws.size(), s);
      std::swap(src, dst);
    }
  };
  chain(nullptr);
  GIE_CUDA_CHECK(cudaDeviceSynchronize());
  GIE_CUDA_CHECK(cudaMemcpy(eager.data(), ping.data(), eager.size(), cudaMemcpyDeviceToDevice));  // 4 swaps: result is in ping
  CudaGraphExecutor g;
  g.capture(chain);
  EXPECT(g.node_count() >= 9);
  GIE_CUDA_CHECK(cudaMemset(ping.data(), 0xFF, ping.size()));
  g.launch(nullptr);
  GIE_CUDA_CHECK(cudaDeviceSynchronize());
  EXPECT(ts::download_bytes(ping.data(), ping.size()) == ts::download_bytes(eager.data(), eager.size()));
}

// ---------------------------------------------------------------------------------------------------------------
// streams and threads (tests/test_runtime_concurrency.cu:53-226)
// ---------------------------------------------------------------------------------------------------------------
// Keeps one stream busy for roughly `cycles` SM cycles and then ends by itself (bounded; nothing waits on it forever).
__global__ void busy_kernel(long long cycles, int* sink) {
  const long long t0 = clock64();
  int spins = 0;
  while (clock64() - t0 < cycles && spins < (1 << 26)) ++spins;
  if (sink != nullptr && spins < 0) *sink = spins;
}

CASE(plan_creation_does_not_wait_for_a_busy_stream) {
  cudaStream_t busy;
  GIE_CUDA_CHECK(cudaStreamCreateWithFlags(&busy, cudaStreamNonBlocking));
  cudaEvent_t done;
  GIE_CUDA_CHECK(cudaEventCreate(&done));
  busy_kernel<<<1, 1, 0, busy>>>(400000000LL, nullptr);  // ~0.2 s
  GIE_CUDA_CHECK(cudaEventRecord(done, busy));
  const ConvProblem prob = ts::problem(ts::geom(2, 16, 9, 9, 16, 3, 3, 1, 1, 1, 1), Precision::kFp16, true, false);
  auto plan = ExecutionPlan::create(prob, *find_kernel("b200_tc_fp16_auto"));
  EXPECT_MSG(cudaEventQuery(done) == cudaErrorNotReady, "plan creation returned only after the unrelated stream drained");
  (void)cudaGetLastError();
  GIE_CUDA_CHECK(cudaStreamSynchronize(busy));
  cudaEventDestroy(done);
  cudaStreamDestroy(busy);
  EXPECT(plan->workspace_bytes() > 0);
}

CASE(create_then_use_immediately_on_fresh_streams) {
  const ConvProblem prob = ts::problem(ts::geom(1, 16, 8, 8, 16, 3, 3, 1, 1, 1, 1), Precision::kFp16, true, true);
  ts::Bundle b = ts::make_bundle(prob, 77);
  const ConstTensorRef bias = b.data.b_ref();
  for (int i = 0; i < 100; ++i) {
    cudaStream_t s;
    GIE_CUDA_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    auto plan = ExecutionPlan::create(prob, *find_kernel("b200_tc_fp16_auto"));
    DeviceBuffer ws(plan->workspace_bytes());
    GIE_CUDA_CHECK(cudaMemsetAsync(b.data.dy.data(), 0xFF, b.data.dy.size(), s));
    plan->execute(b.data.x_ref(), b.data.w_ref(), &bias, b.data.y_ref(), ws.data(), ws.size(), s);
    GIE_CUDA_CHECK(cudaStreamSynchronize(s));
    const ErrorMetrics m = ts::compare_device(b.data.dy.data(), b);
    if (!m.passed()) { EXPECT_MSG(false, "iteration " + std::to_string(i) + ": " + m.summary()); break; }
    cudaStreamDestroy(s);
  }
  EXPECT(true);
}

CASE(one_plan_many_streams_and_threads_with_changing_inputs_and_weights) {
  const ConvProblem prob = ts::problem(ts::geom(2, 32, 12, 12, 48, 3, 3, 1, 1, 1, 1), Precision::kBf16, true, true);
  auto plan = ExecutionPlan::create(prob, *find_kernel("b200_tc_bf16_auto"));
  constexpr int kWorkers = 4, kRounds = 6;
  std::atomic<int> failures{0};
  auto worker = [&](int id) {
    try {
      cudaStream_t s;
      GIE_CUDA_CHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
      DeviceBuffer ws(plan->workspace_bytes());
      ts::Bundle live = ts::make_bundle(prob, 1000 + uint64_t(id));
      for (int r = 0; r < kRounds; ++r) {
        ts::Bundle next = ts::make_bundle(prob, 5000 + uint64_t(id) * 100 + uint64_t(r), r % 2 ? Distribution::kNormal : Distribution::kUniform);
        copy_inputs_async(live, next, s);  // new inputs AND new weights in the same buffers
        GIE_CUDA_CHECK(cudaMemsetAsync(live.data.dy.data(), 0xFF, live.data.dy.size(), s));
        plan->execute_unchecked(live.data.dx.data(), live.data.dw.data(), live.data.db.data(), live.data.dy.data(), ws.data(), ws.size(), s);
        GIE_CUDA_CHECK(cudaStreamSynchronize(s));
        if (!ts::compare_device(live.data.dy.data(), next).passed()) ++failures;
      }
      cudaStreamDestroy(s);
    } catch (const std::exception& e) {
      std::fprintf(stderr, "worker %d: %s\n", id, e.what());
      ++failures;
    }
  };
  std::vector<std::thread> threads;
  for (int i = 0; i < kWorkers; ++i) threads.emplace_back(worker, i);
  for (auto& t : threads) t.join();
  EXPECT(failures.load() == 0);
}

CASE(pointers_offset_by_one_element_work) {  // tests/test_tensor_core.cpp:38-57, test_runtime_concurrency.cu:190-216
  for (Precision prec : {Precision::kFp16, Precision::kFp32}) {
    const ConvProblem prob = ts::problem(ts::geom(2, 16, 9, 11, 24, 3, 3, 1, 1, 1, 1), prec, true, true);
    ts::Bundle b = ts::make_bundle(prob, 5);
    const size_t es = dtype_size(prob.dtype());
    DeviceBuffer x(b.data.dx.size() + 64), w(b.data.dw.size() + 64), y(b.data.dy.size() + 64);
    char* xp = static_cast<char*>(x.data()) + es;
    char* wp = static_cast<char*>(w.data()) + es;
    char* yp = static_cast<char*>(y.data()) + es;
    GIE_CUDA_CHECK(cudaMemcpy(xp, b.data.dx.data(), b.data.dx.size(), cudaMemcpyDeviceToDevice));
    GIE_CUDA_CHECK(cudaMemcpy(wp, b.data.dw.data(), b.data.dw.size(), cudaMemcpyDeviceToDevice));
    GIE_CUDA_CHECK(cudaMemset(y.data(), 0xFF, y.size()));
    const size_t need = Conv2D::workspace_size(prob);
    DeviceBuffer ws(need);
    const ConstTensorRef xr{xp, prob.dtype(), prob.p.input_shape()}, wr{wp, prob.dtype(), prob.p.weight_shape()}, bias = b.data.b_ref();
    const TensorRef yr{yp, prob.dtype(), prob.p.output_shape()};
    Conv2D::forward(xr, wr, &bias, prob, yr, ws.data(), ws.size(), nullptr);
    GIE_CUDA_CHECK(cudaDeviceSynchronize());
    EXPECT(ts::compare_device(yp, b).passed());
    const std::vector<uint8_t> raw = ts::download_bytes(y.data(), y.size());
    bool guard_ok = true;
    for (size_t i = 0; i < es; ++i) guard_ok = guard_ok && raw[i] == 0xFF;
    for (size_t i = es + b.data.dy.size(); i < raw.size(); ++i) guard_ok = guard_ok && raw[i] == 0xFF;
    EXPECT(guard_ok);
  }
}

// ---------------------------------------------------------------------------------------------------------------
// RMSNorm through the C++ entry point (tests/test_rmsnorm.cpp:52-83)
// ---------------------------------------------------------------------------------------------------------------
CASE(rmsnorm_matches_a_double_precision_host_reference) {
  for (DataType dt : {DataType::kFloat32, DataType::kFloat16, DataType::kBFloat16}) {
    const Precision pr = dt == DataType::kFloat32 ? Precision::kFp32 : (dt == DataType::kFloat16 ? Precision::kFp16 : Precision::kBf16);
    const double u = dt == DataType::kFloat32 ? 6e-8 : (dt == DataType::kFloat16 ? 4.9e-4 : 3.9e-3);
    for (int hidden : {1, 33, 127, 1024, 4096, 8191}) {
      for (bool fused : {false, true}) {
        const int rows = 5;
        Rng rng(uint64_t(rows) * 1315423911u + uint64_t(hidden));
        const size_t n = size_t(rows) * hidden;
        std::vector<float> x(n), r(n), g(static_cast<size_t>(hidden));
        for (float& v : x) v = quantize_to(pr, rng.normal() * 3.f);
        for (float& v : r) v = quantize_to(pr, rng.normal());
        for (float& v : g) v = quantize_to(pr, rng.uniform(0.5f, 1.5f));
        DeviceBuffer dx = upload_as(x, dt), dr = upload_as(r, dt), dg = upload_as(g, dt), dy(n * dtype_size(dt)), dres(n * dtype_size(dt));
        RmsNormParams p;
        p.rows = rows; p.hidden = hidden; p.dtype = dt;
        GIE_CUDA_CHECK(cudaMemset(dy.data(), 0xFF, dy.size()));
        rmsnorm_forward(p, dx.data(), dg.data(), dy.data(), fused ? dr.data() : nullptr, fused ? dres.data() : nullptr, nullptr);
        GIE_CUDA_CHECK(cudaDeviceSynchronize());
        const std::vector<float> out = download_as_float(dy.data(), dt, int64_t(n));
        const std::vector<float> res = fused ? download_as_float(dres.data(), dt, int64_t(n)) : std::vector<float>();
        bool ok = true;
        for (int row = 0; row < rows && ok; ++row) {
          double ss = 0;
          std::vector<double> s(static_cast<size_t>(hidden));
          for (int i = 0; i < hidden; ++i) {
            double v = x[size_t(row) * hidden + i];
            if (fused) v = quantize_to(pr, float(v + r[size_t(row) * hidden + i]));
            s[size_t(i)] = v;
            ss += v * v;
          }
          const double inv = 1.0 / std::sqrt(ss / hidden + 1e-6);
          for (int i = 0; i < hidden; ++i) {
            const double ref = s[size_t(i)] * inv * g[size_t(i)];
            const double tol = (dt == DataType::kFloat32 ? 16.0 : 3.0) * u * std::fabs(ref) + 1e-30 + (dt == DataType::kFloat16 ? 1e-7 : 0);
            ok = ok && std::fabs(out[size_t(row) * hidden + i] - ref) <= tol;
            if (fused) ok = ok && res[size_t(row) * hidden + i] == float(s[size_t(i)]);
          }
        }
        EXPECT_MSG(ok, std::string("hidden=") + std::to_string(hidden) + " dtype=" + to_string(dt) + " fused=" + std::to_string(fused));
      }
    }
  }
}

CASE(rmsnorm_rejects_bad_arguments) {
  DeviceBuffer a(64), b(64), c(64);
  RmsNormParams p;
  p.rows = 1; p.hidden = 4;
  EXPECT_THROWS(rmsnorm_forward(p, a.data(), b.data(), a.data(), nullptr, nullptr, nullptr), StatusCode::kInvalidArgument);
  EXPECT_THROWS(rmsnorm_forward(p, a.data(), b.data(), c.data(), a.data(), nullptr, nullptr), StatusCode::kInvalidArgument);
  p.hidden = 0;
  EXPECT_THROWS(rmsnorm_forward(p, a.data(), b.data(), c.data(), nullptr, nullptr, nullptr), StatusCode::kInvalidArgument);
}

// ---------------------------------------------------------------------------------------------------------------
// autotuner and tuning cache (tests/test_autotuner.cu:64-203), with faults injected on the host: a registry entry whose
// launch writes zeros, and one whose launch raises
// ---------------------------------------------------------------------------------------------------------------
namespace {

std::string temp_cache_path(const char* tag) {
  return std::string("/tmp/gie_b200_tune_") + tag + "_" + std::to_string(long(getpid())) + ".json";
}

ConvProblem tune_problem() { return ts::problem(ts::geom(2, 32, 12, 12, 64, 3, 3, 1, 1, 1, 1), Precision::kFp16, true, true); }

void launch_zeros(const LaunchArgs& la) {  // fast, wrong: the output is all zeros
  const size_t bytes = size_t(la.problem->p.output_shape().numel()) * dtype_size(la.problem->dtype());
  GIE_CUDA_CHECK(cudaMemsetAsync(la.y, 0, bytes, la.stream));
}
void launch_throws(const LaunchArgs&) { throw Error(StatusCode::kCudaError, "injected launch failure"); }
bool fp16_only(const ConvProblem& pr, const DeviceInfo&, std::string* why) {
  if (pr.precision == Precision::kFp16) return true;
  if (why) *why = "test entry is fp16 only";
  return false;
}
size_t no_bytes(const ConvProblem&) { return 0; }
int64_t one_block(const ConvProblem&) { return 1; }
double instant(const ConvProblem&) { return 0.01; }  // ranks first
std::shared_ptr<void> no_state(const ConvProblem&) { return nullptr; }

void inject_faulty_entries() {
  if (find_kernel("test_fast_but_wrong_fp16") != nullptr) return;
  for (int which = 0; which < 2; ++which) {
    KernelDesc k;
    k.name = which == 0 ? "test_fast_but_wrong_fp16" : "test_throwing_fp16";
    k.backend = Backend::kTensorCore;
    k.version = kLibraryVersion;
    k.threads_per_block = 32;
    k.supports = &fp16_only;
    k.workspace_bytes = &no_bytes;
    k.dynamic_smem_bytes = &no_bytes;
    k.num_blocks = &one_block;
    k.persistent_bytes = &no_bytes;
    k.create_state = &no_state;
    k.launch = which == 0 ? &launch_zeros : &launch_throws;
    kernel_registry_for_testing().push_back(k);
  }
}

TuneOptions quick_tune(const std::string& cache) {
  TuneOptions o;
  o.timing.samples = 5;
  o.timing.warmup_iters = 2;
  o.timing.min_sample_ms = 0.2;
  o.cache_path = cache;
  return o;
}

}  // namespace

CASE(tuner_never_selects_incorrect_or_failing_candidates) {
  inject_faulty_entries();
  const ConvProblem prob = tune_problem();
  TuneOptions o = quick_tune(temp_cache_path("faults"));
  o.use_cache = false;
  const TuneResult r = Autotuner::tune(prob, DeviceInfo::current(), o);
  EXPECT(r.best_kernel != "test_fast_but_wrong_fp16");
  EXPECT(r.best_kernel != "test_throwing_fp16");
  bool saw_wrong = false, saw_throw = false;
  for (const CandidateResult& c : r.candidates) {
    if (c.kernel == "test_fast_but_wrong_fp16") { saw_wrong = true; EXPECT(!c.measured); EXPECT(c.status.find("failed validation") == 0); }
    if (c.kernel == "test_throwing_fp16") { saw_throw = true; EXPECT(!c.measured); EXPECT(c.status.find("error:") == 0); }
  }
  EXPECT(saw_wrong && saw_throw);
  // the winner is right according to the independent CPU reference as well
  ts::Bundle b = ts::make_bundle(prob, 77);
  bool ran = false;
  const KernelDesc* best = find_kernel(r.best_kernel);
  EXPECT(best != nullptr);
  const ErrorMetrics m = ts::run_kernel(*best, b, &ran, nullptr);
  EXPECT_MSG(ran && m.passed(), r.best_kernel + " " + m.summary());
  EXPECT(r.best_us > 0);
}

CASE(tuner_reports_search_space_and_cost) {
  const ConvProblem prob = tune_problem();
  TuneOptions o = quick_tune(temp_cache_path("space"));
  o.use_cache = false;
  const TuneResult r = Autotuner::tune(prob, DeviceInfo::current(), o);
  EXPECT(r.candidates_total >= 10);
  EXPECT(r.candidates_measured == r.candidates_total);
  EXPECT(r.search_seconds > 0);
  int measured = 0;
  for (const CandidateResult& c : r.candidates)
    if (c.measured) { ++measured; EXPECT(c.timing.median_us > 0); EXPECT(c.timing.samples == 5); EXPECT(c.frac_over_tol == 0); }
  EXPECT(measured >= 5);
}

CASE(tuning_cache_hit_skips_the_search_and_persists) {
  const std::string path = temp_cache_path("persist");
  std::remove(path.c_str());
  const ConvProblem prob = tune_problem();
  const DeviceInfo& dev = DeviceInfo::current();
  TuneOptions o = quick_tune(path);
  o.model_keep = 4;
  const TuneResult cold = Autotuner::tune(prob, dev, o);
  EXPECT(!cold.from_cache);
  const TuneResult warm = Autotuner::tune(prob, dev, o);
  EXPECT(warm.from_cache);
  EXPECT(warm.best_kernel == cold.best_kernel);
  EXPECT(warm.candidates.empty());
  TuneCache fresh(path);
  std::string name;
  double us = 0;
  EXPECT(fresh.lookup(prob, dev, &name, &us));
  EXPECT(name == cold.best_kernel);
  EXPECT(us > 0);
  o.force_retune = true;
  EXPECT(!Autotuner::tune(prob, dev, o).from_cache);
  EXPECT(fresh.lookup(prob, dev, &name, &us));  // the new search may have crowned another configuration
  // selection honours the cache, and Conv2DOptions::autotune fills it
  Conv2DOptions co;
  co.cache_path = path;
  const Selection from_cache = Dispatcher::select(prob, dev, co);
  EXPECT(from_cache.source == SelectionSource::kTuningCache);
  EXPECT(from_cache.kernel != nullptr && from_cache.kernel->name == name);
  fresh.clear();
  EXPECT(fresh.size() == size_t(0));
  EXPECT(!fresh.lookup(prob, dev, &name, &us));
  EXPECT(Dispatcher::select(prob, dev, co).source == SelectionSource::kCostModel);
  co.autotune = true;
  EXPECT(Dispatcher::select(prob, dev, co).source == SelectionSource::kTuned);
  EXPECT(Dispatcher::select(prob, dev, co).source == SelectionSource::kTuningCache);
  std::remove(path.c_str());
}

CASE(tuning_cache_key_separates_problems_precisions_and_fusion) {
  const DeviceInfo& dev = DeviceInfo::current();
  const ConvProblem a = tune_problem();
  ConvProblem b = a, c = a, d = a;
  b.p.batch += 1;
  c.precision = Precision::kBf16;
  d.activation = Activation::kNone;
  const std::string ka = TuneCache::make_key(a, dev);
  EXPECT(ka != TuneCache::make_key(b, dev));
  EXPECT(ka != TuneCache::make_key(c, dev));
  EXPECT(ka != TuneCache::make_key(d, dev));
  EXPECT(ka != TuneCache::make_key(a, dev, Backend::kTensorCore));
  EXPECT(ka.find(dev.name) != std::string::npos);
  EXPECT(ka.find("cudart") != std::string::npos);
}

CASE(tuning_cache_rejects_stale_and_corrupt_entries) {
  const std::string path = temp_cache_path("stale");
  const ConvProblem prob = tune_problem();
  const DeviceInfo& dev = DeviceInfo::current();
  const std::string key = TuneCache::make_key(prob, dev);
  std::string name;
  double us = 0;
  auto write = [&](const std::string& text) { std::ofstream f(path, std::ios::trunc); f << text; };
  write("{ this is not json");
  EXPECT(!TuneCache(path).lookup(prob, dev, &name, &us));
  EXPECT(TuneCache(path).size() == size_t(0));
  write("{\"schema\": 1, \"entries\": {\"" + key + "\": {\"kernel\": \"b200_tc_fp16_auto\", \"kernel_version\": " +
        std::to_string(kLibraryVersion + 1) + ", \"us\": 5.0}}}");
  EXPECT(!TuneCache(path).lookup(prob, dev, &name, &us));  // recorded for another version of the kernel
  write("{\"schema\": 1, \"entries\": {\"" + key + "\": {\"kernel\": \"no_such_kernel\", \"kernel_version\": " +
        std::to_string(kLibraryVersion) + ", \"us\": 5.0}}}");
  EXPECT(!TuneCache(path).lookup(prob, dev, &name, &us));
  write("{\"schema\": 2, \"entries\": {\"" + key + "\": {\"kernel\": \"b200_tc_fp16_auto\", \"kernel_version\": " +
        std::to_string(kLibraryVersion) + ", \"us\": 5.0}}}");
  EXPECT(!TuneCache(path).lookup(prob, dev, &name, &us));  // unknown schema
  write("{\"schema\": 1, \"entries\": {\"" + key + "\": {\"kernel\": \"b200_tc_fp16_auto\", \"kernel_version\": " +
        std::to_string(kLibraryVersion) + ", \"us\": 5.0, \"extra\": {\"nested\": 1}}}}");
  EXPECT(TuneCache(path).lookup(prob, dev, &name, &us));   // well-formed: accepted, unknown fields skipped
  EXPECT(name == "b200_tc_fp16_auto" && us == 5.0);
  write("garbage");
  TuneOptions o = quick_tune(path);
  o.model_keep = 3;
  const TuneResult again = Autotuner::tune(prob, dev, o);
  EXPECT(!again.from_cache);
  EXPECT(TuneCache(path).lookup(prob, dev, &name, &us));   // the corrupt file was rewritten
  std::remove(path.c_str());
}

CASE(tuner_pruning_limits_the_search_and_runs_are_reproducible) {
  const ConvProblem prob = tune_problem();
  TuneOptions o = quick_tune(temp_cache_path("prune"));
  o.use_cache = false;
  o.model_keep = 4;
  const TuneResult a = Autotuner::tune(prob, DeviceInfo::current(), o);
  EXPECT(a.candidates_measured == 4);
  int attempted = 0;
  for (const CandidateResult& c : a.candidates)
    if (c.status.find("rejected") != 0) ++attempted;
  EXPECT(attempted == 4);
  const TuneResult b = Autotuner::tune(prob, DeviceInfo::current(), o);
  EXPECT(a.candidates.size() == b.candidates.size());
  for (size_t i = 0; i < a.candidates.size() && i < b.candidates.size(); ++i) {
    EXPECT(a.candidates[i].kernel == b.candidates[i].kernel);
    EXPECT(a.candidates[i].measured == b.candidates[i].measured);
    EXPECT(a.candidates[i].max_abs_err == b.candidates[i].max_abs_err);  // same seed, same data, same kernels
  }
  o.only_backend = Backend::kImplicitGemm;  // no FP16 kernel in that backend
  EXPECT_THROWS(Autotuner::tune(prob, DeviceInfo::current(), o), StatusCode::kUnsupported);
}

CASE(timing_protocol_batches_short_kernels_and_summarises) {
  const TimingStats s = summarize({5.0, 1.0, 3.0, 2.0, 4.0}, 7);
  EXPECT(s.samples == 5 && s.inner_iters == 7);
  EXPECT(s.median_us == 3.0 && s.min_us == 1.0 && s.max_us == 5.0 && s.mean_us == 3.0);
  EXPECT(s.p10_us > 1.0 && s.p10_us < 2.0 && s.p90_us > 4.0 && s.p90_us < 5.0);
  EXPECT(std::fabs(s.iqr_us - 2.0) < 1e-12);
  DeviceBuffer buf(1 << 20);
  TimingOptions t;
  t.samples = 4;
  t.min_sample_ms = 0.5;
  const TimingStats m = time_stream_work([&](cudaStream_t st) { GIE_CUDA_CHECK(cudaMemsetAsync(buf.data(), 1, buf.size(), st)); }, nullptr, t);
  EXPECT(m.samples == 4 && m.inner_iters > 1 && m.median_us > 0);
  DeviceBuffer flush(64 << 20);
  t.flush_buffer = flush.data();
  t.flush_bytes = flush.size();
  const TimingStats c = time_stream_work([&](cudaStream_t st) { GIE_CUDA_CHECK(cudaMemsetAsync(buf.data(), 1, buf.size(), st)); }, nullptr, t);
  EXPECT(c.inner_iters == 1 && c.samples == 4);
}

int main(int argc, char** argv) {
  // selection must not depend on a tuning cache left in the home directory
  setenv("GIE_TUNE_CACHE", temp_cache_path("default").c_str(), 1);
  std::remove(temp_cache_path("default").c_str());
  return chk::run(argc, argv);
}
