// TEST SUPPORT: the reference's testing.h / reference.h surface on top of the C test oracle (oracle/gie_oracle.c).
#include <cmath>
#include <cstring>
#include <sstream>

#include "gpu_inference/testing.h"

extern "C" {
struct orc_conv_desc {
  int32_t batch, in_channels, in_h, in_w, out_channels, kernel_h, kernel_w, stride_h, stride_w, pad_h, pad_w, dilation_h,
      dilation_w, groups, precision, has_bias, relu;
};
struct orc_tolerance { double c_acc, c_out, c_inter, c_in, u_in, u_acc, u_out, abs_floor; int64_t k; };
struct orc_metrics { int64_t n, over_tol, nan_count, inf_count; double max_abs, mean_abs, rms, max_rel, frac_over_tol, worst_tol_ratio; };
int orc_conv2d(const orc_conv_desc*, const float*, const float*, const float*, float*, float*);
uint64_t orc_rng_next_u64(uint64_t*);
double orc_rng_unit(uint64_t*);
void orc_fill_dist(uint64_t*, int, float, float*, int64_t);
void orc_fill_uniform(uint64_t*, float, float, float*, int64_t);
float orc_quantize_one(int, float);
void orc_to_bits16(int, const float*, uint16_t*, int64_t);
void orc_from_bits16(int, const uint16_t*, float*, int64_t);
void orc_tolerance_for(const orc_conv_desc*, int, orc_tolerance*);
void orc_compare(const float*, const float*, const float*, int64_t, const orc_tolerance*, orc_metrics*);
}

namespace gie {
namespace {
orc_conv_desc to_orc(const ConvProblem& pr) {
  const Conv2DParams& p = pr.p;
  return {p.batch, p.in_channels, p.in_h, p.in_w, p.out_channels, p.kernel_h, p.kernel_w, p.stride_h, p.stride_w, p.pad_h, p.pad_w,
          p.dilation_h, p.dilation_w, p.groups, int(pr.precision), int(pr.has_bias), int(pr.activation == Activation::kReLU)};
}
int storage_id(DataType dt) { return dt == DataType::kFloat16 ? 1 : (dt == DataType::kBFloat16 ? 2 : 0); }
}  // namespace

uint64_t Rng::next_u64() { return orc_rng_next_u64(&s_); }
double Rng::uniform() { return orc_rng_unit(&s_); }
float Rng::uniform(float lo, float hi) { float v; orc_fill_uniform(&s_, lo, hi, &v, 1); return v; }
float Rng::normal() { float v; orc_fill_dist(&s_, 1, 1.0f, &v, 1); return v; }

const char* to_string(Distribution d) {
  static const char* const n[] = {"uniform", "normal", "sparse_signed", "positive"};
  return n[int(d) & 3];
}

ConstTensorRef ConvData::x_ref() const { return {dx.data(), prob.dtype(), prob.p.input_shape()}; }
ConstTensorRef ConvData::w_ref() const { return {dw.data(), prob.dtype(), prob.p.weight_shape()}; }
ConstTensorRef ConvData::b_ref() const { return {db.data(), prob.dtype(), prob.p.bias_shape()}; }
TensorRef ConvData::y_ref() { return {dy.data(), prob.dtype(), prob.p.output_shape()}; }

DeviceBuffer upload_as(const std::vector<float>& v, DataType dt) {
  DeviceBuffer buf(v.size() * dtype_size(dt));
  if (dt == DataType::kFloat32) {
    GIE_CUDA_CHECK(cudaMemcpy(buf.data(), v.data(), v.size() * 4, cudaMemcpyHostToDevice));
  } else {
    std::vector<uint16_t> raw(v.size());
    orc_to_bits16(storage_id(dt), v.data(), raw.data(), int64_t(v.size()));
    GIE_CUDA_CHECK(cudaMemcpy(buf.data(), raw.data(), raw.size() * 2, cudaMemcpyHostToDevice));
  }
  return buf;
}

ConvData make_conv_data(const ConvProblem& prob, uint64_t seed, Distribution dist) {
  validate_problem(prob);
  ConvData d;
  d.prob = prob;
  const Conv2DParams& p = prob.p;
  uint64_t state = seed;
  d.hx.resize(size_t(p.input_shape().numel()));
  d.hw.resize(size_t(p.weight_shape().numel()));
  d.hb.resize(size_t(p.out_channels));
  orc_fill_dist(&state, int(dist), 1.0f, d.hx.data(), int64_t(d.hx.size()));
  orc_fill_dist(&state, int(dist), std::sqrt(3.0f / float(p.gemm_k())), d.hw.data(), int64_t(d.hw.size()));
  orc_fill_uniform(&state, -1.f, 1.f, d.hb.data(), int64_t(d.hb.size()));
  const DataType dt = prob.dtype();
  for (float& v : d.hx) v = quantize_to(prob.precision, v);
  for (float& v : d.hw) v = quantize_to(prob.precision, v);
  if (dt != DataType::kFloat32)
    for (float& v : d.hb) v = quantize_to(prob.precision, v);
  d.dx = upload_as(d.hx, dt);
  d.dw = upload_as(d.hw, dt);
  d.db = upload_as(d.hb, dt);
  d.dy = DeviceBuffer(size_t(p.output_shape().numel()) * dtype_size(dt));
  GIE_CUDA_CHECK(cudaMemset(d.dy.data(), 0xFF, d.dy.size()));
  GIE_CUDA_CHECK(cudaDeviceSynchronize());
  return d;
}

void cpu_conv2d_reference(const ConvProblem& prob, const float* x, const float* w, const float* bias, ReferenceOutput* out) {
  validate_problem(prob);
  const size_t n = size_t(prob.p.output_shape().numel());
  out->y.assign(n, 0.f);
  out->scale.assign(n, 0.f);
  const orc_conv_desc d = to_orc(prob);
  if (orc_conv2d(&d, x, w, bias, out->y.data(), out->scale.data()) != 0) throw Error(StatusCode::kInternal, "oracle rejected the problem");
}

TolerancePolicy TolerancePolicy::for_problem(const ConvProblem& prob, bool intermediate_rounding) {
  orc_tolerance o;
  const orc_conv_desc d = to_orc(prob);
  orc_tolerance_for(&d, intermediate_rounding ? 1 : 0, &o);
  TolerancePolicy t;
  t.c_acc = o.c_acc; t.c_out = o.c_out; t.c_inter = o.c_inter; t.c_in = o.c_in; t.u_in = o.u_in; t.u_acc = o.u_acc;
  t.u_out = o.u_out; t.abs_floor = o.abs_floor; t.k = o.k;
  return t;
}
double TolerancePolicy::tol(double ref, double scale) const {
  return c_acc * u_acc * std::sqrt(double(k)) * scale + c_out * u_out * std::fabs(ref) + c_inter * u_out * scale + c_in * u_in * scale + abs_floor;
}
std::string TolerancePolicy::describe() const {
  std::ostringstream os;
  os << "tol = " << c_acc << "*2^-24*sqrt(" << k << ")*scale + " << c_out << "*" << u_out << "*|ref| + " << c_inter << "*u_out*scale + " << abs_floor;
  return os.str();
}

ErrorMetrics compare_outputs(const float* test, const float* ref, const float* scale, int64_t n, const TolerancePolicy& tol) {
  orc_tolerance o = {tol.c_acc, tol.c_out, tol.c_inter, tol.c_in, tol.u_in, tol.u_acc, tol.u_out, tol.abs_floor, tol.k};
  orc_metrics m;
  orc_compare(test, ref, scale, n, &o, &m);
  ErrorMetrics e;
  e.n = m.n; e.max_abs = m.max_abs; e.mean_abs = m.mean_abs; e.rms = m.rms; e.max_rel = m.max_rel; e.frac_over_tol = m.frac_over_tol;
  e.over_tol = m.over_tol; e.nan_count = m.nan_count; e.inf_count = m.inf_count; e.worst_tol_ratio = m.worst_tol_ratio;
  return e;
}
std::string ErrorMetrics::summary() const {
  std::ostringstream os;
  os << "max_abs=" << max_abs << " rms=" << rms << " max_rel=" << max_rel << " over_tol=" << over_tol << "/" << n
     << " worst_tol_ratio=" << worst_tol_ratio << " nan=" << nan_count << " inf=" << inf_count;
  return os.str();
}

float quantize_to(Precision p, float v) { return orc_quantize_one(int(p), v); }
float round_to_tf32(float v) { return orc_quantize_one(3, v); }

std::vector<float> download_as_float(const void* d_ptr, DataType dt, int64_t n) {
  std::vector<float> out(static_cast<size_t>(n));
  if (dt == DataType::kFloat32) {
    GIE_CUDA_CHECK(cudaMemcpy(out.data(), d_ptr, size_t(n) * 4, cudaMemcpyDeviceToHost));
  } else {
    std::vector<uint16_t> raw(static_cast<size_t>(n));
    GIE_CUDA_CHECK(cudaMemcpy(raw.data(), d_ptr, size_t(n) * 2, cudaMemcpyDeviceToHost));
    orc_from_bits16(storage_id(dt), raw.data(), out.data(), n);
  }
  return out;
}

}  // namespace gie
