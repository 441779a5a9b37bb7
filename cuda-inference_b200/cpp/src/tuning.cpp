// Timing protocol, tuning cache and the validate-then-time search over the registered configurations.
// Behaviour follows src/runtime/timing.cpp:21-83, src/autotuner/tune_cache.cpp:11-125 and
// src/autotuner/autotuner.cpp:15-140 of the reference; the code is this layer's own.
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <ctime>
#include <fstream>
#include <iostream>
#include <sstream>

#include "gie_b200.h"
#include "gpu_inference/autotuner.h"
#include "gpu_inference/execution_plan.h"
#include "gpu_inference/nvtx.h"

namespace gie {

gieb_conv_desc to_c_desc(const ConvProblem& pr);  // core.cpp

// ---- timing ---------------------------------------------------------------------------------------------------------
TimingStats summarize(std::vector<double> v, int inner) {
  TimingStats s;
  s.samples = int(v.size());
  s.inner_iters = inner;
  s.raw_us = v;
  if (v.empty()) return s;
  std::sort(v.begin(), v.end());
  auto pct = [&](double p) {  // linear interpolation between order statistics
    const double pos = p * double(v.size() - 1);
    const size_t lo = size_t(pos);
    const size_t hi = std::min(lo + 1, v.size() - 1);
    return v[lo] + (v[hi] - v[lo]) * (pos - double(lo));
  };
  s.min_us = v.front();
  s.max_us = v.back();
  s.median_us = pct(0.5);
  s.p10_us = pct(0.10);
  s.p90_us = pct(0.90);
  s.p99_us = pct(0.99);
  s.iqr_us = pct(0.75) - pct(0.25);
  double sum = 0;
  for (double x : v) sum += x;
  s.mean_us = sum / double(v.size());
  double var = 0;
  for (double x : v) var += (x - s.mean_us) * (x - s.mean_us);
  s.stddev_us = v.size() > 1 ? std::sqrt(var / double(v.size() - 1)) : 0.0;
  return s;
}

TimingStats time_stream_work(const std::function<void(cudaStream_t)>& launch, cudaStream_t stream, const TimingOptions& opt) {
  GIE_REQUIRE(opt.samples > 0, StatusCode::kInvalidArgument, "timing needs at least one sample");
  cudaEvent_t e0, e1;
  GIE_CUDA_CHECK(cudaEventCreate(&e0));
  GIE_CUDA_CHECK(cudaEventCreate(&e1));
  struct Events {
    cudaEvent_t a, b;
    ~Events() { cudaEventDestroy(a); cudaEventDestroy(b); }
  } guard{e0, e1};
  for (int i = 0; i < opt.warmup_iters; ++i) launch(stream);
  GIE_CUDA_CHECK(cudaStreamSynchronize(stream));
  const bool cold = opt.flush_buffer != nullptr && opt.flush_bytes > 0;
  int inner = cold ? 1 : opt.inner;
  if (inner <= 0) {  // batch short kernels: time one launch, then size the batch for min_sample_ms
    GIE_CUDA_CHECK(cudaEventRecord(e0, stream));
    launch(stream);
    GIE_CUDA_CHECK(cudaEventRecord(e1, stream));
    GIE_CUDA_CHECK(cudaEventSynchronize(e1));
    float ms = 0;
    GIE_CUDA_CHECK(cudaEventElapsedTime(&ms, e0, e1));
    inner = ms > 0 ? int(std::ceil(opt.min_sample_ms / double(ms))) : opt.max_inner;
    inner = std::max(1, std::min(inner, opt.max_inner));
  }
  std::vector<double> per_launch;
  per_launch.reserve(size_t(opt.samples));
  for (int s = 0; s < opt.samples; ++s) {
    if (cold) GIE_CUDA_CHECK(cudaMemsetAsync(opt.flush_buffer, s & 0xff, opt.flush_bytes, stream));
    GIE_CUDA_CHECK(cudaEventRecord(e0, stream));
    for (int i = 0; i < inner; ++i) launch(stream);
    GIE_CUDA_CHECK(cudaEventRecord(e1, stream));
    GIE_CUDA_CHECK(cudaEventSynchronize(e1));
    float ms = 0;
    GIE_CUDA_CHECK(cudaEventElapsedTime(&ms, e0, e1));
    per_launch.push_back(double(ms) * 1e3 / double(inner));
  }
  return summarize(std::move(per_launch), inner);
}

// ---- ranking --------------------------------------------------------------------------------------------------------
std::vector<std::pair<const KernelDesc*, double>> Dispatcher::rank_by_model(const ConvProblem& prob, const DeviceInfo&,
                                                                            const std::vector<const KernelDesc*>& cands) {
  std::vector<std::pair<const KernelDesc*, double>> out;
  out.reserve(cands.size());
  for (const KernelDesc* k : cands) out.push_back({k, k->estimate_us ? k->estimate_us(prob) : 1e30});
  std::stable_sort(out.begin(), out.end(), [](const auto& a, const auto& b) { return a.second < b.second; });
  return out;
}

// ---- tuning cache ---------------------------------------------------------------------------------------------------
namespace {

std::string json_escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') { o += '\\'; o += c; }
    else if (c == '\n') o += "\\n";
    else if (static_cast<unsigned char>(c) < 0x20) { char b[8]; std::snprintf(b, sizeof(b), "\\u%04x", c); o += b; }
    else o += c;
  }
  return o;
}

// Minimal reader for the cache's own format: objects, strings, numbers.  Anything unexpected throws, and the caller
// treats the file as empty.
struct Reader {
  const std::string& s;
  size_t i = 0;
  explicit Reader(const std::string& text) : s(text) {}
  [[noreturn]] void bad() const { throw Error(StatusCode::kIo, "malformed tuning cache"); }
  void ws() { while (i < s.size() && (s[i] == ' ' || s[i] == '\n' || s[i] == '\t' || s[i] == '\r')) ++i; }
  bool eat(char c) { ws(); if (i < s.size() && s[i] == c) { ++i; return true; } return false; }
  void need(char c) { if (!eat(c)) bad(); }
  std::string str() {
    need('"');
    std::string o;
    while (i < s.size() && s[i] != '"') {
      if (s[i] == '\\') {
        if (++i >= s.size()) bad();
        if (s[i] == 'n') o += '\n';
        else if (s[i] == 'u') { if (i + 4 >= s.size()) bad(); o += char(std::strtol(s.substr(i + 1, 4).c_str(), nullptr, 16)); i += 4; }
        else o += s[i];
      } else {
        o += s[i];
      }
      ++i;
    }
    if (i >= s.size()) bad();
    ++i;
    return o;
  }
  double num() {
    ws();
    char* end = nullptr;
    const double v = std::strtod(s.c_str() + i, &end);
    if (end == s.c_str() + i) bad();
    i = size_t(end - s.c_str());
    return v;
  }
  // value that is either a string or a number; returns the text form and whether it was a string
  void skip_value() {
    ws();
    if (i >= s.size()) bad();
    if (s[i] == '"') { str(); return; }
    if (s[i] == '{') {
      ++i;
      if (eat('}')) return;
      do { str(); need(':'); skip_value(); } while (eat(','));
      need('}');
      return;
    }
    num();
  }
};

}  // namespace

std::string TuneCache::default_path() {
  if (const char* p = std::getenv("GIE_TUNE_CACHE")) return p;
  const char* home = std::getenv("HOME");
  return std::string(home ? home : ".") + "/.cache/gpu_inference/tune_cache.json";
}

TuneCache::TuneCache(std::string path) : path_(path.empty() ? default_path() : std::move(path)) {}

std::string TuneCache::make_key(const ConvProblem& prob, const DeviceInfo& dev, Backend scope) {
  std::ostringstream os;
  os << dev.name << "|sm" << dev.cc() << "|sms" << dev.sm_count << "|cudart" << dev.runtime_version << "|drv" << dev.driver_version
     << "|lib" << kLibraryVersion << "|abi" << gieb_version() << "|" << prob.key();
  if (scope != Backend::kAuto) os << "|only=" << to_string(scope);
  return os.str();
}

void TuneCache::load_locked() const {
  entries_.clear();
  std::ifstream f(path_);
  if (!f) return;  // no file: empty cache
  std::stringstream buf;
  buf << f.rdbuf();
  const std::string text = buf.str();
  try {
    std::map<std::string, Entry> loaded;
    int schema = 0;
    Reader r(text);
    r.need('{');
    if (!r.eat('}')) {
      do {
        const std::string field = r.str();
        r.need(':');
        if (field == "schema") {
          schema = int(r.num());
        } else if (field == "entries") {
          r.need('{');
          if (!r.eat('}')) {
            do {
              const std::string key = r.str();
              r.need(':');
              r.need('{');
              Entry e;
              bool has_kernel = false, has_version = false, has_us = false;
              if (!r.eat('}')) {
                do {
                  const std::string k = r.str();
                  r.need(':');
                  if (k == "kernel") { e.kernel = r.str(); has_kernel = true; }
                  else if (k == "kernel_version") { e.kernel_version = int(r.num()); has_version = true; }
                  else if (k == "us") { e.us = r.num(); has_us = true; }
                  else if (k == "tuned_seconds") e.tuned_seconds = r.num();
                  else if (k == "timestamp") e.timestamp = r.str();
                  else r.skip_value();
                } while (r.eat(','));
                r.need('}');
              }
              if (has_kernel && has_version && has_us) loaded[key] = e;  // malformed entries are dropped
            } while (r.eat(','));
            r.need('}');
          }
        } else {
          r.skip_value();
        }
      } while (r.eat(','));
      r.need('}');
    }
    if (schema == 1) entries_ = std::move(loaded);  // unknown schema: ignore the file
  } catch (const Error&) {
    entries_.clear();  // corrupt file: treated as empty, rewritten on the next store
  }
}

void TuneCache::save_locked() const {
  const size_t slash = path_.find_last_of('/');
  if (slash != std::string::npos && slash > 0) {
    const std::string cmd = "mkdir -p '" + path_.substr(0, slash) + "'";
    if (std::system(cmd.c_str()) != 0) throw Error(StatusCode::kIo, "cannot create the directory of " + path_);
  }
  std::ofstream f(path_, std::ios::trunc);
  if (!f) throw Error(StatusCode::kIo, "cannot write " + path_);
  f << "{\n  \"schema\": 1,\n  \"library_version\": " << kLibraryVersion << ",\n  \"entries\": {";
  bool first = true;
  for (const auto& kv : entries_) {
    char us[64], ts[64];
    std::snprintf(us, sizeof(us), "%.6f", kv.second.us);
    std::snprintf(ts, sizeof(ts), "%.6f", kv.second.tuned_seconds);
    f << (first ? "\n" : ",\n") << "    \"" << json_escape(kv.first) << "\": {\"kernel\": \"" << json_escape(kv.second.kernel)
      << "\", \"kernel_version\": " << kv.second.kernel_version << ", \"us\": " << us << ", \"tuned_seconds\": " << ts
      << ", \"timestamp\": \"" << json_escape(kv.second.timestamp) << "\"}";
    first = false;
  }
  f << (first ? "" : "\n  ") << "}\n}\n";
  if (!f) throw Error(StatusCode::kIo, "short write to " + path_);
}

bool TuneCache::lookup(const ConvProblem& prob, const DeviceInfo& dev, std::string* kernel, double* us, double* tuned_seconds,
                       Backend scope) const {
  std::lock_guard<std::mutex> lock(mu_);
  load_locked();  // always re-read: another process may have tuned meanwhile
  const auto it = entries_.find(make_key(prob, dev, scope));
  if (it == entries_.end()) return false;
  const KernelDesc* k = find_kernel(it->second.kernel);
  if (k == nullptr || k->version != it->second.kernel_version) return false;  // stale: kernel removed or changed
  std::string why;
  if (!k->supports(prob, dev, &why)) return false;
  if (kernel) *kernel = it->second.kernel;
  if (us) *us = it->second.us;
  if (tuned_seconds) *tuned_seconds = it->second.tuned_seconds;
  return true;
}

void TuneCache::store(const TuneResult& r, const DeviceInfo& dev, Backend scope) {
  const KernelDesc* k = find_kernel(r.best_kernel);
  if (k == nullptr) return;
  std::lock_guard<std::mutex> lock(mu_);
  load_locked();
  Entry e;
  e.kernel = r.best_kernel;
  e.kernel_version = k->version;
  e.us = r.best_us;
  e.tuned_seconds = r.search_seconds;
  const std::time_t now = std::time(nullptr);
  char buf[32];
  std::tm tmv;
  gmtime_r(&now, &tmv);
  std::strftime(buf, sizeof(buf), "%Y-%m-%dT%H:%M:%SZ", &tmv);
  e.timestamp = buf;
  entries_[make_key(r.problem, dev, scope)] = e;
  save_locked();
}

void TuneCache::clear() {
  std::lock_guard<std::mutex> lock(mu_);
  entries_.clear();
  save_locked();
}

size_t TuneCache::size() const {
  std::lock_guard<std::mutex> lock(mu_);
  load_locked();
  return entries_.size();
}

// ---- the search -----------------------------------------------------------------------------------------------------
namespace {

struct DeviceMem {
  void* p = nullptr;
  size_t n = 0;
  explicit DeviceMem(size_t bytes) : n(bytes) { GIE_CUDA_CHECK(cudaMalloc(&p, bytes ? bytes : 1)); }
  ~DeviceMem() { cudaFree(p); }
  DeviceMem(const DeviceMem&) = delete;
  DeviceMem& operator=(const DeviceMem&) = delete;
};

void c_check(int status) {
  if (status != GIEB_OK) throw Error(static_cast<StatusCode>(status), gieb_last_error());
}

}  // namespace

TuneResult Autotuner::tune(const ConvProblem& prob, const DeviceInfo& dev, const TuneOptions& opt) {
  NvtxRange range("gie::Autotuner::tune");
  using clock = std::chrono::steady_clock;
  const auto t0 = clock::now();
  validate_problem(prob);

  TuneResult res;
  res.problem = prob;
  TuneCache cache(opt.cache_path);
  if (opt.use_cache && !opt.force_retune) {
    std::string name;
    double us = 0, cold_s = 0;
    if (cache.lookup(prob, dev, &name, &us, &cold_s, opt.only_backend) && find_kernel(name) != nullptr) {
      res.best_kernel = name;
      res.best_us = us;
      res.from_cache = true;
      res.search_seconds = cold_s;  // what the original search cost
      return res;
    }
  }

  int prev_dev = 0;
  GIE_CUDA_CHECK(cudaGetDevice(&prev_dev));
  if (prev_dev != dev.device) GIE_CUDA_CHECK(cudaSetDevice(dev.device));
  struct Restore {
    int d;
    ~Restore() { cudaSetDevice(d); }
  } restore{prev_dev};

  // 1. capability filter
  std::vector<Rejection> rejected;
  const std::vector<const KernelDesc*> cands = Dispatcher::compatible_kernels(prob, dev, opt.only_backend, &rejected);
  for (const Rejection& r : rejected) {
    CandidateResult cr;
    cr.kernel = r.kernel;
    cr.status = "rejected: " + r.reason;
    res.candidates.push_back(cr);
  }
  res.candidates_total = int(cands.size());
  if (cands.empty()) throw Error(StatusCode::kUnsupported, "autotune: no compatible kernel for " + prob.key());

  // 2. ranking and optional pruning
  auto ranked = Dispatcher::rank_by_model(prob, dev, cands);
  if (opt.model_keep > 0 && int(ranked.size()) > opt.model_keep) ranked.resize(size_t(opt.model_keep));
  if (int(ranked.size()) > opt.max_candidates) ranked.resize(size_t(opt.max_candidates));

  // 3. shared synthetic data and the double-accumulating GPU convolution (computed once)
  const gieb_conv_desc d = to_c_desc(prob);
  const int prec = int(d.precision);
  const size_t esize = prec == 0 ? 4 : 2;
  const int64_t nx = prob.p.input_shape().numel(), nw = prob.p.weight_shape().numel(), ny = prob.p.output_shape().numel();
  const int64_t fan_in = int64_t(prob.p.in_channels) * prob.p.kernel_h * prob.p.kernel_w;
  DeviceMem dx(size_t(nx) * esize), dw(size_t(nw) * esize), db(size_t(prob.p.out_channels) * esize), dy(size_t(ny) * esize);
  DeviceMem dref(size_t(ny) * 4), dscale(size_t(ny) * 4);
  cudaStream_t stream;
  GIE_CUDA_CHECK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  struct StreamGuard {
    cudaStream_t s;
    ~StreamGuard() { cudaStreamDestroy(s); }
  } sg{stream};
  const float wb = float(std::sqrt(3.0 / double(fan_in)));
  c_check(gieb_fill_uniform(prec, dx.p, nx, opt.seed, -1.f, 1.f, stream));
  c_check(gieb_fill_uniform(prec, dw.p, nw, opt.seed + 1, -wb, wb, stream));
  c_check(gieb_fill_uniform(prec, db.p, prob.p.out_channels, opt.seed + 2, -1.f, 1.f, stream));
  const void* bias = prob.has_bias ? db.p : nullptr;
  if (opt.validate) {
    c_check(gieb_conv_reference_launch(&d, dx.p, dw.p, bias, static_cast<float*>(dref.p), static_cast<float*>(dscale.p), stream));
    GIE_CUDA_CHECK(cudaStreamSynchronize(stream));
  }

  // 4. validate, then time, each candidate
  double best_us = 0;
  for (const auto& rk : ranked) {
    const KernelDesc& k = *rk.first;
    CandidateResult cr;
    cr.kernel = k.name;
    cr.backend = k.backend;
    cr.predicted_us = rk.second;
    try {
      auto plan = ExecutionPlan::create(prob, k, dev.device);
      DeviceMem ws(plan->workspace_bytes());
      GIE_CUDA_CHECK(cudaMemsetAsync(dy.p, 0xFF, dy.n, stream));  // NaN pattern: an untouched output cannot pass
      plan->execute_unchecked(dx.p, dw.p, bias, dy.p, ws.p, ws.n, stream);
      GIE_CUDA_CHECK(cudaStreamSynchronize(stream));
      GIE_CUDA_CHECK(cudaGetLastError());
      bool ok = true;
      if (opt.validate) {
        int64_t nonfinite = 0;
        c_check(gieb_conv_check_output(&d, dy.p, static_cast<const float*>(dref.p), static_cast<const float*>(dscale.p), &cr.max_abs_err,
                                       &cr.frac_over_tol, &nonfinite, stream));
        if (cr.frac_over_tol > 0 || nonfinite > 0) {
          ok = false;
          std::ostringstream os;
          os << "failed validation: max_abs=" << cr.max_abs_err << " frac_over_tol=" << cr.frac_over_tol << " nonfinite=" << nonfinite;
          cr.status = os.str();
        }
      }
      if (ok) {
        cr.timing = time_stream_work([&](cudaStream_t s) { plan->execute_unchecked(dx.p, dw.p, bias, dy.p, ws.p, ws.n, s); }, stream,
                                     opt.timing);
        GIE_CUDA_CHECK(cudaGetLastError());
        cr.measured = true;
        cr.status = "ok";
        if (res.best_kernel.empty() || cr.timing.median_us < best_us) {
          best_us = cr.timing.median_us;
          res.best_kernel = k.name;
        }
      }
    } catch (const Error& e) {
      cr.status = std::string("error: ") + e.what();
    }
    if (opt.verbose)
      std::cerr << "[tune] " << prob.key() << " " << k.name << ": " << cr.status
                << (cr.measured ? " " + std::to_string(cr.timing.median_us) + " us" : std::string()) << "\n";
    res.candidates.push_back(std::move(cr));
  }
  res.candidates_measured = int(ranked.size());
  if (res.best_kernel.empty()) throw Error(StatusCode::kUnsupported, "autotune: every candidate failed for " + prob.key());
  res.best_us = best_us;
  res.search_seconds = std::chrono::duration<double>(clock::now() - t0).count();
  if (opt.use_cache) cache.store(res, dev, opt.only_backend);
  return res;
}

}  // namespace gie
