// CPU oracle for the OxiONNX dense-contraction hot path.  TEST INFRASTRUCTURE ONLY:
// see oxi_oracle.h for the contract.  Each function names the reference file (path inside
// the oxionnx project, v0.1.7) whose arithmetic it restates.
#include "oxi_oracle.h"

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <string>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif
#if defined(__AVX2__) && defined(__FMA__)
#include <immintrin.h>
#endif

namespace {

thread_local std::string g_err;
int g_threads = 1;
int g_float_accum = 0;

struct Fail {
  int code;
};

[[noreturn]] void fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_err = buf;
  throw Fail{code};
}

int64_t numel(const oxo_tensor& t) {
  int64_t n = 1;
  for (int i = 0; i < t.rank; ++i) n *= t.shape[i];
  return n;
}

struct Attrs {
  const oxo_attr* a;
  int n;
  const oxo_attr* find(const char* name, int kind) const {
    for (int i = 0; i < n; ++i)
      if (a[i].kind == kind && std::strcmp(a[i].name, name) == 0) return &a[i];
    return nullptr;
  }
  int64_t i(const char* name, int64_t d) const {
    auto* p = find(name, OXO_ATTR_INT);
    return p ? p->i : d;
  }
  float f(const char* name, float d) const {
    auto* p = find(name, OXO_ATTR_FLOAT);
    return p ? p->f : d;
  }
  std::string s(const char* name) const {
    auto* p = find(name, OXO_ATTR_STRING);
    return p && p->s ? std::string(p->s) : std::string();
  }
  std::vector<int64_t> ints(const char* name) const {
    auto* p = find(name, OXO_ATTR_INTS);
    return p ? std::vector<int64_t>(p->ints, p->ints + p->len) : std::vector<int64_t>();
  }
};

struct Ctx {
  const char* op;
  const oxo_tensor* in;
  int n_in;
  Attrs attrs;
  oxo_tensor* out;
  int n_out;
  // required input (OpContext::input): missing -> TensorNotFound in the reference
  const oxo_tensor& input(int idx) const {
    if (idx >= n_in || !in[idx].present) fail(OXO_ERR_INVALID_MODEL, "%s: missing required input %d", op, idx);
    return in[idx];
  }
  const oxo_tensor* optional(int idx) const {
    if (idx >= n_in || !in[idx].present) return nullptr;
    return &in[idx];
  }
};

void alloc_out(oxo_tensor& t, const std::vector<int64_t>& shape) {
  if ((int)shape.size() > OXO_MAX_RANK) fail(OXO_ERR_UNSUPPORTED, "rank %zu exceeds oracle limit", shape.size());
  t.rank = (int)shape.size();
  int64_t n = 1;
  for (int i = 0; i < t.rank; ++i) {
    t.shape[i] = shape[i];
    n *= shape[i];
  }
  t.len = n;
  t.present = 1;
  t.data = (float*)std::calloc((size_t)std::max<int64_t>(n, 1), sizeof(float));
  if (!t.data) fail(OXO_ERR_INTERNAL, "out of memory");
}

std::vector<int64_t> shape_of(const oxo_tensor& t) { return std::vector<int64_t>(t.shape, t.shape + t.rank); }

// ---------------------------------------------------------------------------------------
// Rounding and requantisation: oxionnx-ops/src/registry/quant_ops/mod.rs:51-70, 79-92,
// 153-245.
// ---------------------------------------------------------------------------------------
double round_ties_even_f64(double v) {
  if (!std::isfinite(v)) return v;
  double fl = std::floor(v);
  double diff = v - fl;
  // rem_euclid(2.0) != 0  <=>  floor is odd
  double rem = std::fmod(fl, 2.0);
  if (rem < 0) rem += 2.0;
  bool up = diff > 0.5 || (diff == 0.5 && rem != 0.0);
  return up ? fl + 1.0 : fl;
}
float round_ties_even_f32_via64(float v) { return (float)round_ties_even_f64((double)v); }

// oxionnx-ops/src/indexing/quantize.rs:14-32 (rounds directly in f32)
float round_ties_even_f32_native(float v) {
  if (!std::isfinite(v)) return v;
  float fl = std::floor(v);
  float diff = v - fl;
  if (diff > 0.5f) return fl + 1.0f;
  if (diff < 0.5f) return fl;
  float rem = std::fmod(fl, 2.0f);
  if (rem < 0) rem += 2.0f;
  return rem == 0.0f ? fl : fl + 1.0f;
}

// lane_to_i32: quant_ops/mod.rs:79-92
int32_t lane_to_i32(float v, const char* what) {
  if (!std::isfinite(v)) fail(OXO_ERR_INVALID_MODEL, "%s: quantized tensor contains a non-finite value (%g)", what, (double)v);
  float r = round_ties_even_f32_via64(v);
  if (r < (float)INT32_MIN || r > (float)INT32_MAX)
    fail(OXO_ERR_INVALID_MODEL, "%s: quantized value %g is outside the int32 range", what, (double)v);
  // Rust `as i32` saturates; (float)INT32_MAX == 2^31 passes the check above and saturates.
  if (r >= 2147483648.0f) return INT32_MAX;
  return (int32_t)r;
}

std::vector<int32_t> tensor_to_i32(const oxo_tensor& t, const char* what) {
  std::vector<int32_t> v((size_t)t.len);
  for (int64_t i = 0; i < t.len; ++i) v[(size_t)i] = lane_to_i32(t.data[i], what);
  return v;
}

// scalar_f32 / scale_input: quant_ops/mod.rs:98-118
float scale_input(const oxo_tensor& t, const char* what) {
  if (t.len < 1) fail(OXO_ERR_INVALID_MODEL, "%s: is empty", what);
  float v = t.data[0];
  if (!std::isfinite(v)) fail(OXO_ERR_INVALID_MODEL, "%s: scale must be finite, got %g", what, (double)v);
  if (v == 0.0f) fail(OXO_ERR_INVALID_MODEL, "%s: scale is zero", what);
  return v;
}

// zero_point_lanes: quant_ops/mod.rs:121-127
std::vector<int32_t> zero_point_lanes(const oxo_tensor* zp, const char* what) {
  if (!zp || zp->len == 0) return {0};
  return tensor_to_i32(*zp, what);
}

struct SatRange {
  int64_t lo, hi;
};
// SatRange::infer: quant_ops/mod.rs:190-200
SatRange sat_infer(const std::vector<int32_t>& y_zp, const std::vector<int32_t>& x_zp) {
  const std::vector<int32_t>* lanes[2] = {&y_zp, &x_zp};
  for (auto* l : lanes) {
    bool gt = false, lt = false;
    for (int32_t v : *l) {
      gt |= v > 127;
    }
    if (gt) return {0, 255};
    for (int32_t v : *l) {
      lt |= v < 0;
    }
    if (lt) return {-128, 127};
  }
  return {-128, 255};
}

// execute_typed (quant_ops/qlinear_matmul.rs, qlinear_conv.rs): SatRange::for_dtype (mod.rs:216-222) of the declared
// type of y_zero_point when it is U8 or I8, otherwise the value cascade of infer.
SatRange sat_range(const oxo_tensor* y_zp_tensor, const std::vector<int32_t>& y_zp, const std::vector<int32_t>& x_zp) {
  if (y_zp_tensor && y_zp_tensor->dtype == OXO_DT_U8) return SatRange{0, 255};
  if (y_zp_tensor && y_zp_tensor->dtype == OXO_DT_I8) return SatRange{-128, 127};
  return sat_infer(y_zp, x_zp);
}

// SatRange::requantize: quant_ops/mod.rs:229-233
float requantize(int64_t acc, float combined, int32_t zp, SatRange r) {
  volatile double prod = (double)acc * (double)combined;  // separately rounded multiply
  double scaled = prod + (double)zp;
  double rounded = round_ties_even_f64(scaled);
  // f64::clamp: NaN stays NaN
  if (rounded < (double)r.lo) rounded = (double)r.lo;
  if (rounded > (double)r.hi) rounded = (double)r.hi;
  return (float)rounded;
}

// saturate_i32: quant_ops/mod.rs:243-245
float saturate_i32(int64_t acc) {
  int64_t c = std::min<int64_t>(std::max<int64_t>(acc, INT32_MIN), INT32_MAX);
  return (float)c;
}

void check_len(const oxo_tensor& t, const char* op, const char* which) {
  if (t.len != numel(t)) fail(OXO_ERR_SHAPE_MISMATCH, "%s: %s data length %lld does not match shape", op, which, (long long)t.len);
}

// ---------------------------------------------------------------------------------------
// QuantizeLinear / DequantizeLinear: oxionnx-ops/src/indexing/quantize.rs:58-193 and
// oxionnx-ops/src/registry/indexing_ops.rs:204-238.
// ---------------------------------------------------------------------------------------
int64_t normalize_axis(int64_t axis, int64_t ndim, const char* op) {
  int64_t a = axis < 0 ? axis + ndim : axis;
  if (a < 0 || a >= ndim) fail(OXO_ERR_INVALID_MODEL, "%s: axis %lld out of range for rank %lld", op, (long long)axis, (long long)ndim);
  return a;
}

struct ChannelIndexer {
  int64_t inner = 1, dim = 1, len = 1;
  int64_t at(int64_t flat) const { return len <= 1 ? 0 : (flat / inner) % dim; }
};
ChannelIndexer make_indexer(const oxo_tensor& x, int64_t axis, int64_t param_len) {
  ChannelIndexer ci;
  ci.len = param_len;
  if (param_len > 1) {
    int64_t inner = 1;
    for (int d = (int)axis + 1; d < x.rank; ++d) inner *= x.shape[d];
    ci.inner = std::max<int64_t>(inner, 1);
    ci.dim = std::max<int64_t>(x.shape[axis], 1);
  }
  return ci;
}

void op_quantize_linear(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  const oxo_tensor& scale = c.input(1);
  const oxo_tensor* zp = c.optional(2);
  int64_t axis = c.attrs.i("axis", 1);
  int64_t scale_len = scale.len;
  if (scale_len == 0) fail(OXO_ERR_INVALID_MODEL, "quantize_linear: y_scale must have at least one element");
  if (zp && zp->len == 0) fail(OXO_ERR_INVALID_MODEL, "quantize_linear: y_zero_point must have at least one element when provided");
  int64_t zp_len = zp ? zp->len : 0;
  int64_t plen = std::max(scale_len, zp_len);
  int64_t ax = plen > 1 ? normalize_axis(axis, x.rank, "quantize_linear") : 0;
  float lo = 0.0f, hi = 255.0f;  // saturation_range: quantize.rs:58-64
  if (zp) {
    bool any_gt = false;
    for (int64_t i = 0; i < zp->len; ++i) any_gt |= zp->data[i] > 127.0f;
    if (!any_gt) {
      lo = -128.0f;
      hi = 127.0f;
    }
  }
  ChannelIndexer si = make_indexer(x, ax, scale_len), zi = make_indexer(x, ax, zp_len);
  // channel_index reads past the parameter vector when its length disagrees with the axis
  // extent; the reference would panic there, the oracle reports it instead.
  if (scale_len > 1 && scale_len < si.dim) fail(OXO_ERR_SHAPE_MISMATCH, "quantize_linear: scale length %lld < axis extent %lld", (long long)scale_len, (long long)si.dim);
  if (zp_len > 1 && zp_len < zi.dim) fail(OXO_ERR_SHAPE_MISMATCH, "quantize_linear: zero point length %lld < axis extent %lld", (long long)zp_len, (long long)zi.dim);
  alloc_out(c.out[0], shape_of(x));
  float* y = c.out[0].data;
#pragma omp parallel for if (g_threads > 1) num_threads(g_threads)
  for (int64_t i = 0; i < x.len; ++i) {
    float s = scale.data[si.at(i)];
    float z = zp ? zp->data[zi.at(i)] : 0.0f;
    volatile float q = x.data[i] / s;
    float v = round_ties_even_f32_native(q) + z;
    // f32::clamp keeps NaN
    if (v < lo) v = lo;
    if (v > hi) v = hi;
    y[i] = v;
  }
}

void op_dequantize_linear(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  const oxo_tensor& scale = c.input(1);
  const oxo_tensor* zp = c.optional(2);
  int64_t axis = c.attrs.i("axis", 1);
  int64_t scale_len = scale.len;
  if (scale_len == 0) fail(OXO_ERR_INVALID_MODEL, "dequantize_linear: x_scale must have at least one element");
  if (zp && zp->len == 0) fail(OXO_ERR_INVALID_MODEL, "dequantize_linear: x_zero_point must have at least one element when provided");
  int64_t zp_len = zp ? zp->len : 0;
  int64_t plen = std::max(scale_len, zp_len);
  int64_t ax = plen > 1 ? normalize_axis(axis, x.rank, "dequantize_linear") : 0;
  ChannelIndexer si = make_indexer(x, ax, scale_len), zi = make_indexer(x, ax, zp_len);
  if (scale_len > 1 && scale_len < si.dim) fail(OXO_ERR_SHAPE_MISMATCH, "dequantize_linear: scale length mismatch");
  if (zp_len > 1 && zp_len < zi.dim) fail(OXO_ERR_SHAPE_MISMATCH, "dequantize_linear: zero point length mismatch");
  alloc_out(c.out[0], shape_of(x));
  float* y = c.out[0].data;
#pragma omp parallel for if (g_threads > 1) num_threads(g_threads)
  for (int64_t i = 0; i < x.len; ++i) {
    float s = scale.data[si.at(i)];
    float z = zp ? zp->data[zi.at(i)] : 0.0f;
    volatile float d = x.data[i] - z;  // subtract, then multiply: two roundings, no FMA
    y[i] = d * s;
  }
}

// DynamicQuantizeLinear: oxionnx-ops/src/registry/quant_ops/dynamic_quantize.rs:51-93
void op_dynamic_quantize_linear(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  if (x.len == 0) fail(OXO_ERR_INVALID_MODEL, "DynamicQuantizeLinear: input is empty");
  for (int64_t i = 0; i < x.len; ++i)
    if (!std::isfinite(x.data[i])) fail(OXO_ERR_INVALID_MODEL, "DynamicQuantizeLinear: input contains a non-finite value (%g)", (double)x.data[i]);
  float max_x = -std::numeric_limits<float>::infinity(), min_x = std::numeric_limits<float>::infinity();
  for (int64_t i = 0; i < x.len; ++i) {
    max_x = std::max(max_x, x.data[i]);
    min_x = std::min(min_x, x.data[i]);
  }
  max_x = std::max(max_x, 0.0f);
  min_x = std::min(min_x, 0.0f);
  float span = (max_x == min_x) ? 1.0f : max_x - min_x;
  volatile float y_scale = span / 255.0f;
  volatile float izp = 0.0f - min_x / y_scale;
  float cl = izp;
  if (cl < 0.0f) cl = 0.0f;
  if (cl > 255.0f) cl = 255.0f;
  float y_zp = round_ties_even_f32_via64(cl);
  alloc_out(c.out[0], shape_of(x));
  float ys = y_scale;
  float* y = c.out[0].data;
#pragma omp parallel for if (g_threads > 1) num_threads(g_threads)
  for (int64_t i = 0; i < x.len; ++i) {
    volatile float q = x.data[i] / ys;
    float v = round_ties_even_f32_via64(q) + y_zp;
    if (v < 0.0f) v = 0.0f;
    if (v > 255.0f) v = 255.0f;
    y[i] = v;
  }
  if (c.n_out > 1) {
    alloc_out(c.out[1], {});
    c.out[1].data[0] = ys;
  }
  if (c.n_out > 2) {
    alloc_out(c.out[2], {});
    c.out[2].data[0] = y_zp;
  }
}

// ---------------------------------------------------------------------------------------
// Integer matmul family: oxionnx-ops/src/registry/quant_ops/qlinear_matmul.rs:30-254
// ---------------------------------------------------------------------------------------
struct MatMulShape {
  int64_t batch, m, k, n;
  std::vector<int64_t> out_shape;
  bool a_broadcast, b_broadcast;
};

MatMulShape resolve_shapes(const oxo_tensor& a, const oxo_tensor& b, const char* op) {
  if (a.rank == 0 || b.rank == 0) fail(OXO_ERR_SHAPE_MISMATCH, "%s: inputs must have rank >= 1", op);
  bool a1 = a.rank == 1, b1 = b.rank == 1;
  std::vector<int64_t> ad = a1 ? std::vector<int64_t>{1, a.shape[0]} : shape_of(a);
  std::vector<int64_t> bd = b1 ? std::vector<int64_t>{b.shape[0], 1} : shape_of(b);
  int64_t m = ad[ad.size() - 2], k = ad[ad.size() - 1], kb = bd[bd.size() - 2], n = bd[bd.size() - 1];
  if (k != kb) fail(OXO_ERR_SHAPE_MISMATCH, "%s: inner dimensions disagree: %lld vs %lld", op, (long long)k, (long long)kb);
  int64_t ba = 1, bb = 1;
  for (size_t i = 0; i + 2 < ad.size(); ++i) ba *= ad[i];
  for (size_t i = 0; i + 2 < bd.size(); ++i) bb *= bd[i];
  int64_t batch;
  if (ba == bb) batch = ba;
  else if (ba == 1) batch = bb;
  else if (bb == 1) batch = ba;
  else fail(OXO_ERR_SHAPE_MISMATCH, "%s: batch dimensions disagree (%lld vs %lld) and neither is 1", op, (long long)ba, (long long)bb);
  const std::vector<int64_t>& pre = ba >= bb ? ad : bd;
  std::vector<int64_t> out(pre.begin(), pre.end() - 2);
  if (!a1) out.push_back(m);
  if (!b1) out.push_back(n);
  return {batch, m, k, n, out, ba == 1 && batch != 1, bb == 1 && batch != 1};
}

inline int32_t zp_at(const std::vector<int32_t>& l, int64_t idx) {
  if (l.size() == 1) return l[0];
  return (size_t)idx < l.size() ? l[(size_t)idx] : 0;
}

void check_zero_point(const std::vector<int32_t>& l, int64_t expected, const char* op, const char* which) {
  if (l.size() == 1 || (int64_t)l.size() == expected) return;
  fail(OXO_ERR_SHAPE_MISMATCH, "%s: %s has %zu entries, expected 1 (per tensor) or %lld", op, which, l.size(), (long long)expected);
}

std::vector<int64_t> integer_matmul(const std::vector<int32_t>& a, const std::vector<int32_t>& b, const std::vector<int32_t>& a_zp,
                                    const std::vector<int32_t>& b_zp, const MatMulShape& s) {
  std::vector<int64_t> out((size_t)(s.batch * s.m * s.n), 0);
  // B is re-read column-wise by the reference loop; a transposed copy changes nothing in
  // the arithmetic and keeps the all-cores variant usable at the benchmark sizes.
  int64_t total_rows = s.batch * s.m;
#pragma omp parallel for if (g_threads > 1) num_threads(g_threads) schedule(static)
  for (int64_t row = 0; row < total_rows; ++row) {
    int64_t bi = row / s.m, i = row % s.m;
    int64_t a_base = s.a_broadcast ? 0 : bi * s.m * s.k;
    int64_t b_base = s.b_broadcast ? 0 : bi * s.k * s.n;
    int64_t azp = zp_at(a_zp, i);
    std::vector<int64_t> acc((size_t)s.n, 0);
    for (int64_t p = 0; p < s.k; ++p) {
      int64_t av = (int64_t)a[(size_t)(a_base + i * s.k + p)] - azp;
      const int32_t* brow = &b[(size_t)(b_base + p * s.n)];
      if (b_zp.size() == 1) {
        int64_t bz = b_zp[0];
        for (int64_t j = 0; j < s.n; ++j) acc[(size_t)j] += av * ((int64_t)brow[j] - bz);
      } else {
        for (int64_t j = 0; j < s.n; ++j) acc[(size_t)j] += av * ((int64_t)brow[j] - (int64_t)zp_at(b_zp, j));
      }
    }
    std::copy(acc.begin(), acc.end(), out.begin() + (size_t)(bi * s.m * s.n + i * s.n));
  }
  return out;
}

void op_matmul_integer(Ctx& c) {
  const char* op = "MatMulInteger";
  const oxo_tensor& a = c.input(0);
  const oxo_tensor& b = c.input(1);
  check_len(a, op, "A");
  check_len(b, op, "B");
  auto a_zp = zero_point_lanes(c.optional(2), "MatMulInteger: a_zero_point");
  auto b_zp = zero_point_lanes(c.optional(3), "MatMulInteger: b_zero_point");
  MatMulShape s = resolve_shapes(a, b, op);
  check_zero_point(a_zp, s.m, op, "a_zero_point");
  check_zero_point(b_zp, s.n, op, "b_zero_point");
  auto ai = tensor_to_i32(a, "MatMulInteger: A");
  auto bi = tensor_to_i32(b, "MatMulInteger: B");
  auto acc = integer_matmul(ai, bi, a_zp, b_zp, s);
  alloc_out(c.out[0], s.out_shape);
  for (size_t i = 0; i < acc.size(); ++i) c.out[0].data[i] = saturate_i32(acc[i]);
}

void op_qlinear_matmul(Ctx& c) {
  const char* op = "QLinearMatMul";
  const oxo_tensor& a = c.input(0);
  float a_scale = scale_input(c.input(1), "QLinearMatMul: a_scale");
  auto a_zp = zero_point_lanes(c.optional(2), "QLinearMatMul: a_zero_point");
  const oxo_tensor& b = c.input(3);
  float b_scale = scale_input(c.input(4), "QLinearMatMul: b_scale");
  auto b_zp = zero_point_lanes(c.optional(5), "QLinearMatMul: b_zero_point");
  float y_scale = scale_input(c.input(6), "QLinearMatMul: y_scale");
  auto y_zp_l = zero_point_lanes(c.optional(7), "QLinearMatMul: y_zero_point");
  check_len(a, op, "a");
  check_len(b, op, "b");
  MatMulShape s = resolve_shapes(a, b, op);
  check_zero_point(a_zp, s.m, op, "a_zero_point");
  check_zero_point(b_zp, s.n, op, "b_zero_point");
  auto ai = tensor_to_i32(a, "QLinearMatMul: a");
  auto bi = tensor_to_i32(b, "QLinearMatMul: b");
  auto acc = integer_matmul(ai, bi, a_zp, b_zp, s);
  int32_t y_zp = y_zp_l.empty() ? 0 : y_zp_l[0];
  SatRange r = sat_range(c.optional(7), y_zp_l, a_zp);
  volatile float ab = a_scale * b_scale;
  float combined = ab / y_scale;
  alloc_out(c.out[0], s.out_shape);
  for (size_t i = 0; i < acc.size(); ++i) c.out[0].data[i] = requantize(acc[i], combined, y_zp, r);
}

// ---------------------------------------------------------------------------------------
// Convolution geometry: oxionnx-ops/src/conv/spatial.rs:36-50, 88-160, 204-260, 272-345,
// 413-455.
// ---------------------------------------------------------------------------------------
struct ConvGeo {
  int rank;
  std::vector<int64_t> strides, pads, dilations, out_shape;
  int64_t group;
};

std::vector<int64_t> read_positive_spatial(const std::vector<int64_t>& v, int rank, const char* name, const char* op) {
  std::vector<int64_t> out((size_t)rank, 1);
  for (int a = 0; a < rank; ++a)
    if ((size_t)a < v.size()) {
      if (v[(size_t)a] < 1) fail(OXO_ERR_SHAPE_MISMATCH, "%s: %s[%d] must be >= 1, got %lld", op, name, a, (long long)v[(size_t)a]);
      out[(size_t)a] = v[(size_t)a];
    }
  return out;
}

std::vector<int64_t> read_pads(const std::vector<int64_t>& v, int rank, const char* op) {
  std::vector<int64_t> out((size_t)(2 * rank), 0);
  for (int i = 0; i < 2 * rank; ++i)
    if ((size_t)i < v.size()) {
      if (v[(size_t)i] < 0) fail(OXO_ERR_SHAPE_MISMATCH, "%s: pads[%d] must be >= 0, got %lld", op, i, (long long)v[(size_t)i]);
      out[(size_t)i] = v[(size_t)i];
    }
  return out;
}

enum AutoPad { NOTSET, SAME_UPPER, SAME_LOWER, VALID };
AutoPad parse_auto_pad(const std::string& raw, const char* op) {
  if (raw.empty() || raw == "NOTSET") return NOTSET;
  if (raw == "SAME_UPPER") return SAME_UPPER;
  if (raw == "SAME_LOWER") return SAME_LOWER;
  if (raw == "VALID") return VALID;
  fail(OXO_ERR_UNSUPPORTED, "%s: unknown auto_pad value '%s' (expected NOTSET, SAME_UPPER, SAME_LOWER or VALID)", op, raw.c_str());
}

std::vector<int64_t> resolve_pads(AutoPad ap, const int64_t* in_sp, const int64_t* kernel, const std::vector<int64_t>& strides,
                                  const std::vector<int64_t>& dil, const std::vector<int64_t>& explicit_pads, int rank) {
  if (ap == NOTSET) return explicit_pads;
  std::vector<int64_t> out((size_t)(2 * rank), 0);
  if (ap == VALID) return out;
  bool lower = ap == SAME_LOWER;
  for (int a = 0; a < rank; ++a) {
    int64_t stride = std::max<int64_t>(strides[(size_t)a], 1);
    int64_t out_dim = (in_sp[a] + stride - 1) / stride;
    int64_t eff_k = std::max<int64_t>(kernel[a] - 1, 0) * dil[(size_t)a] + 1;
    int64_t needed = std::max<int64_t>(std::max<int64_t>(out_dim - 1, 0) * strides[(size_t)a] + eff_k - in_sp[a], 0);
    int64_t half = needed / 2;
    out[(size_t)a] = lower ? needed - half : half;
    out[(size_t)(a + rank)] = lower ? half : needed - half;
  }
  return out;
}

int64_t pool_out_dim(const char* op, int axis, int64_t in_dim, int64_t pb, int64_t pe, int64_t kernel, int64_t dil, int64_t stride, bool ceil_mode) {
  if (stride == 0) fail(OXO_ERR_SHAPE_MISMATCH, "%s: strides[%d] must be >= 1, got 0", op, axis);
  if (kernel == 0 || dil == 0) fail(OXO_ERR_SHAPE_MISMATCH, "%s: invalid kernel/dilation on axis %d", op, axis);
  int64_t eff_k = (kernel - 1) * dil + 1;
  int64_t padded = in_dim + pb + pe;
  if (padded < eff_k)
    fail(OXO_ERR_SHAPE_MISMATCH, "%s: padded input extent %lld on axis %d is smaller than the dilated kernel extent %lld", op, (long long)padded, axis,
         (long long)eff_k);
  int64_t span = padded - eff_k;
  int64_t out = ceil_mode ? (span + stride - 1) / stride + 1 : span / stride + 1;
  if (ceil_mode && out > 1 && (out - 1) * stride >= in_dim + pb) out -= 1;
  return out;
}

ConvGeo conv_geometry(const Attrs& at, const oxo_tensor& x, const oxo_tensor& w, const char* op, bool check_kernel_shape) {
  if (x.rank < 3) fail(OXO_ERR_SHAPE_MISMATCH, "%s: input must have rank >= 3 ([N, C, d_0, ...]), got rank %d", op, x.rank);
  int rank = x.rank - 2;
  if (w.rank != x.rank) fail(OXO_ERR_SHAPE_MISMATCH, "%s: weight rank %d must equal input rank %d", op, w.rank, x.rank);
  ConvGeo g;
  g.rank = rank;
  g.strides = read_positive_spatial(at.ints("strides"), rank, "strides", op);
  g.dilations = read_positive_spatial(at.ints("dilations"), rank, "dilations", op);
  g.group = at.i("group", 1);
  if (g.group < 1) fail(OXO_ERR_SHAPE_MISMATCH, "%s: group must be >= 1, got %lld", op, (long long)g.group);
  if (check_kernel_shape) {  // float Conv only: registry/conv_ops/conv.rs:66-77
    auto ks = at.ints("kernel_shape");
    if (!ks.empty()) {
      if ((int)ks.size() < rank) fail(OXO_ERR_SHAPE_MISMATCH, "%s: kernel_shape requires %d spatial dims, got %zu", op, rank, ks.size());
      for (int a = 0; a < rank; ++a) {
        if (ks[(size_t)a] < 1) fail(OXO_ERR_SHAPE_MISMATCH, "%s: kernel_shape[%d] must be >= 1", op, a);
        if (ks[(size_t)a] != w.shape[a + 2]) fail(OXO_ERR_SHAPE_MISMATCH, "%s: kernel_shape disagrees with weight spatial dims", op);
      }
    }
  }
  int64_t c_in = x.shape[1], cpg = w.shape[1];
  if (cpg * g.group != c_in)
    fail(OXO_ERR_SHAPE_MISMATCH, "%s: input channels %lld != weight input channels %lld * group %lld", op, (long long)c_in, (long long)cpg, (long long)g.group);
  if (w.shape[0] % g.group != 0) fail(OXO_ERR_SHAPE_MISMATCH, "%s: output channels %lld not divisible by group %lld", op, (long long)w.shape[0], (long long)g.group);
  auto explicit_pads = read_pads(at.ints("pads"), rank, op);
  AutoPad ap = parse_auto_pad(at.s("auto_pad"), op);
  g.pads = resolve_pads(ap, x.shape + 2, w.shape + 2, g.strides, g.dilations, explicit_pads, rank);
  g.out_shape = {x.shape[0], w.shape[0]};
  for (int a = 0; a < rank; ++a)
    g.out_shape.push_back(pool_out_dim(op, a, x.shape[a + 2], g.pads[(size_t)a], g.pads[(size_t)(a + rank)], w.shape[a + 2], g.dilations[(size_t)a],
                                       g.strides[(size_t)a], false));
  return g;
}

// Visit every (output position, kernel tap) pair of a rank-generic convolution and hand
// the caller the input spatial offset of in-bounds taps.  Mirrors the odometer loops of
// quant_ops/conv_kernel.rs:205-249.
struct TapTable {
  // for each output flat index: list of (k_flat, in_off) for in-bounds taps
  std::vector<int64_t> start;           // size out_plane+1
  std::vector<int32_t> k_flat, in_off;  // concatenated
};

TapTable build_taps(const ConvGeo& g, const int64_t* in_sp, const int64_t* kernel) {
  int rank = g.rank;
  const int64_t* out_sp = g.out_shape.data() + 2;
  int64_t out_plane = 1, k_volume = 1;
  for (int d = 0; d < rank; ++d) {
    out_plane *= out_sp[d];
    k_volume *= kernel[d];
  }
  std::vector<int64_t> in_stride((size_t)rank, 1);
  for (int d = rank - 2; d >= 0; --d) in_stride[(size_t)d] = in_stride[(size_t)d + 1] * in_sp[d + 1];
  TapTable t;
  t.start.resize((size_t)out_plane + 1);
  std::vector<int64_t> oidx((size_t)rank, 0), kidx((size_t)rank, 0);
  for (int64_t o = 0; o < out_plane; ++o) {
    t.start[(size_t)o] = (int64_t)t.k_flat.size();
    std::fill(kidx.begin(), kidx.end(), 0);
    for (int64_t kf = 0; kf < k_volume; ++kf) {
      int64_t off = 0;
      bool inside = true;
      for (int d = 0; d < rank; ++d) {
        int64_t pos = oidx[(size_t)d] * g.strides[(size_t)d] + kidx[(size_t)d] * g.dilations[(size_t)d];
        int64_t ip = pos - g.pads[(size_t)d];
        if (ip < 0 || ip >= in_sp[d]) {
          inside = false;
          break;
        }
        off += ip * in_stride[(size_t)d];
      }
      if (inside) {
        t.k_flat.push_back((int32_t)kf);
        t.in_off.push_back((int32_t)off);
      }
      for (int d = rank - 1; d >= 0; --d) {
        if (++kidx[(size_t)d] < kernel[d]) break;
        kidx[(size_t)d] = 0;
      }
    }
    for (int d = rank - 1; d >= 0; --d) {
      if (++oidx[(size_t)d] < out_sp[d]) break;
      oidx[(size_t)d] = 0;
    }
  }
  t.start[(size_t)out_plane] = (int64_t)t.k_flat.size();
  return t;
}

// integer_conv: quant_ops/conv_kernel.rs:134-254.  acc starts at the int32 bias; taps in
// the padding are skipped.
std::vector<int64_t> integer_conv(const oxo_tensor& x, const oxo_tensor& w, int32_t x_zp, const std::vector<int32_t>& w_zp, const oxo_tensor* bias,
                                  const ConvGeo& g, const char* op) {
  int64_t batch = x.shape[0], c_in = x.shape[1], c_out = w.shape[0], cpg = w.shape[1];
  if (w_zp.size() != 1 && (int64_t)w_zp.size() != c_out)
    fail(OXO_ERR_SHAPE_MISMATCH, "%s: w_zero_point has %zu entries, expected 1 or %lld (per output channel)", op, w_zp.size(), (long long)c_out);
  if (x.len != numel(x)) fail(OXO_ERR_SHAPE_MISMATCH, "%s: input data length %lld does not match shape", op, (long long)x.len);
  if (w.len != numel(w)) fail(OXO_ERR_SHAPE_MISMATCH, "%s: weight data length %lld does not match shape", op, (long long)w.len);
  std::vector<int64_t> bias64;
  if (bias) {
    if (bias->len != c_out) fail(OXO_ERR_SHAPE_MISMATCH, "%s: bias has %lld entries, expected %lld", op, (long long)bias->len, (long long)c_out);
    std::string label = std::string(op) + ": bias";
    for (int64_t i = 0; i < c_out; ++i) bias64.push_back(lane_to_i32(bias->data[i], label.c_str()));
  }
  std::string li = std::string(op) + ": input", lw = std::string(op) + ": weight";
  auto xi = tensor_to_i32(x, li.c_str());
  auto wi = tensor_to_i32(w, lw.c_str());
  int rank = g.rank;
  int64_t in_plane = 1, out_plane = 1, k_volume = 1;
  for (int d = 0; d < rank; ++d) {
    in_plane *= x.shape[d + 2];
    out_plane *= g.out_shape[(size_t)d + 2];
    k_volume *= w.shape[d + 2];
  }
  int64_t copg = c_out / g.group;
  TapTable taps = build_taps(g, x.shape + 2, w.shape + 2);
  std::vector<int64_t> acc((size_t)(batch * c_out * out_plane), 0);
  int64_t jobs = batch * c_out;
#pragma omp parallel for if (g_threads > 1) num_threads(g_threads) schedule(dynamic, 1)
  for (int64_t job = 0; job < jobs; ++job) {
    int64_t n = job / c_out, oc = job % c_out;
    int64_t grp = oc / copg;
    int64_t wz = w_zp.size() == 1 ? w_zp[0] : w_zp[(size_t)oc];
    int64_t w_base = oc * cpg * k_volume;
    int64_t out_base = (n * c_out + oc) * out_plane;
    int64_t bias_term = bias64.empty() ? 0 : bias64[(size_t)oc];
    for (int64_t o = 0; o < out_plane; ++o) {
      int64_t sum = bias_term;
      for (int64_t t = taps.start[(size_t)o]; t < taps.start[(size_t)o + 1]; ++t) {
        int64_t kf = taps.k_flat[(size_t)t], off = taps.in_off[(size_t)t];
        for (int64_t ic = 0; ic < cpg; ++ic) {
          int64_t plane = (n * c_in + grp * cpg + ic) * in_plane;
          int64_t xv = xi[(size_t)(plane + off)];
          int64_t wv = wi[(size_t)(w_base + ic * k_volume + kf)];
          sum += (xv - x_zp) * (wv - wz);
        }
      }
      acc[(size_t)(out_base + o)] = sum;
    }
  }
  return acc;
}

// QLinearConv: quant_ops/qlinear_conv.rs:34-103
void op_qlinear_conv(Ctx& c) {
  const char* op = "QLinearConv";
  const oxo_tensor& x = c.input(0);
  float x_scale = scale_input(c.input(1), "QLinearConv: x_scale");
  auto x_zp_l = zero_point_lanes(c.optional(2), "QLinearConv: x_zero_point");
  const oxo_tensor& w = c.input(3);
  const oxo_tensor& w_scale = c.input(4);
  auto w_zp_l = zero_point_lanes(c.optional(5), "QLinearConv: w_zero_point");
  float y_scale = scale_input(c.input(6), "QLinearConv: y_scale");
  auto y_zp_l = zero_point_lanes(c.optional(7), "QLinearConv: y_zero_point");
  const oxo_tensor* bias = c.optional(8);
  if (bias && bias->len == 0) bias = nullptr;
  if (w_scale.len == 0) fail(OXO_ERR_INVALID_MODEL, "QLinearConv: w_scale is empty");
  int32_t x_zp = x_zp_l.empty() ? 0 : x_zp_l[0];
  int32_t y_zp = y_zp_l.empty() ? 0 : y_zp_l[0];
  ConvGeo g = conv_geometry(c.attrs, x, w, op, false);
  auto acc = integer_conv(x, w, x_zp, w_zp_l, bias, g, op);
  int64_t c_out = w.shape[0];
  bool per_channel = w_scale.len > 1;
  if (per_channel && w_scale.len != c_out)
    fail(OXO_ERR_SHAPE_MISMATCH, "QLinearConv: w_scale has %lld entries, expected 1 or %lld (per output channel)", (long long)w_scale.len, (long long)c_out);
  for (int64_t i = 0; i < w_scale.len; ++i)
    if (!std::isfinite(w_scale.data[i])) fail(OXO_ERR_INVALID_MODEL, "QLinearConv: w_scale[%lld] must be finite", (long long)i);
  SatRange r = sat_range(c.optional(7), y_zp_l, {x_zp});
  int64_t spatial = 1;
  for (size_t d = 2; d < g.out_shape.size(); ++d) spatial *= g.out_shape[d];
  alloc_out(c.out[0], g.out_shape);
  float* y = c.out[0].data;
#pragma omp parallel for if (g_threads > 1) num_threads(g_threads)
  for (int64_t flat = 0; flat < (int64_t)acc.size(); ++flat) {
    int64_t oc = (flat / spatial) % c_out;
    float ws = per_channel ? w_scale.data[oc] : w_scale.data[0];
    volatile float xw = x_scale * ws;
    float combined = xw / y_scale;
    y[flat] = requantize(acc[(size_t)flat], combined, y_zp, r);
  }
}

// ConvInteger: quant_ops/qlinear_conv.rs:173-203
void op_conv_integer(Ctx& c) {
  const char* op = "ConvInteger";
  const oxo_tensor& x = c.input(0);
  const oxo_tensor& w = c.input(1);
  auto x_zp_l = zero_point_lanes(c.optional(2), "ConvInteger: x_zero_point");
  auto w_zp_l = zero_point_lanes(c.optional(3), "ConvInteger: w_zero_point");
  int32_t x_zp = x_zp_l.empty() ? 0 : x_zp_l[0];
  ConvGeo g = conv_geometry(c.attrs, x, w, op, false);
  auto acc = integer_conv(x, w, x_zp, w_zp_l, nullptr, g, op);
  alloc_out(c.out[0], g.out_shape);
  for (size_t i = 0; i < acc.size(); ++i) c.out[0].data[i] = saturate_i32(acc[i]);
}

// ---------------------------------------------------------------------------------------
// Float Conv: oxionnx-ops/src/registry/conv_ops/conv.rs:40-156 (geometry + fused
// activation) over the definition implemented by oxionnx-ops/src/conv/conv2d.rs.
// ---------------------------------------------------------------------------------------
void apply_fused_activation(const Attrs& at, float* data, int64_t n) {
  std::string act = at.s("activation");
  if (act == "relu") {
    for (int64_t i = 0; i < n; ++i) data[i] = std::max(data[i], 0.0f);  // f32::max: NaN -> 0
  } else if (act == "clip") {
    float mn = at.f("activation_min", -std::numeric_limits<float>::infinity());
    float mx = at.f("activation_max", std::numeric_limits<float>::infinity());
    float lo = std::isnan(mn) ? -std::numeric_limits<float>::infinity() : mn;
    float hi = std::isnan(mx) ? std::numeric_limits<float>::infinity() : mx;
    if (lo <= hi)
      for (int64_t i = 0; i < n; ++i) {
        float v = data[i];
        if (v < lo) v = lo;
        if (v > hi) v = hi;
        data[i] = v;
      }
  }
}

// ---------------------------------------------------------------------------------------
// The reference's float contraction ALGORITHM (float mode 2): what the timed CPU baseline runs.
//
// Conv: oxionnx-ops/src/conv/conv2d.rs:246-546 -- a 1x1 / stride-1 / unpadded convolution is one
// sgemm per (batch, group) over the input viewed as [C, H*W] (conv2d_1x1_into, :1071); every other
// shape gathers an im2col column matrix [C/g*kH*kW, OH*OW] in blocks of at most 64 MiB
// (IM2COL_WORKSPACE_MAX_BYTES :119, im2col_block_cols :135) and multiplies the filter matrix into
// it; with more than one (batch, group) job the jobs run in parallel, each with a sequential
// sgemm (:468-546), otherwise the one job's sgemm is split by rows of the filter matrix
// (parallel_sgemm :1132, taken when m*k*n >= 64^3 and m >= 2 * threads, :896).  Bias is a separate
// pass (:441-449), the fused activation another (registry/conv_ops/conv.rs:124-156).  The
// Winograd branch (:325-346) only takes layers below 4096 work units and is not restated.
// MatMul / Gemm: one sgemm per batch item, items in parallel from four on (math_typed.rs:334-420).
//
// sgemm itself is the third-party crate matrixmultiply 0.3 (Cargo.toml:43, not vendored).  Its
// published algorithm is restated here: Goto-style blocking (kc = 256, mc = 64, nc = 1024), both
// operands packed into panels, an 8 x 8 register tile updated with fused multiply-adds (AVX2 + FMA,
// which that crate selects at run time on x86-64), the K blocks of an output element added in
// order.  The summation order inside a tile is this file's own, so the result agrees with the
// reference's to rounding (about 1e-6 relative), not bit for bit.
// ---------------------------------------------------------------------------------------
constexpr int64_t kGemmMR = 8, kGemmNR = 8, kGemmKC = 256, kGemmMC = 64, kGemmNC = 1024;

// acc[8][8] += sum_p ap[p][0..8] (x) bp[p][0..8]; ap and bp are packed panels of kc steps.
inline void gemm_micro_8x8(int64_t kc, const float* ap, const float* bp, float* acc /* 64 */) {
#if defined(__AVX2__) && defined(__FMA__)
  __m256 r0 = _mm256_setzero_ps(), r1 = r0, r2 = r0, r3 = r0, r4 = r0, r5 = r0, r6 = r0, r7 = r0;
  for (int64_t p = 0; p < kc; ++p) {
    const __m256 b = _mm256_loadu_ps(bp + p * 8);
    const float* a = ap + p * 8;
    r0 = _mm256_fmadd_ps(_mm256_broadcast_ss(a + 0), b, r0);
    r1 = _mm256_fmadd_ps(_mm256_broadcast_ss(a + 1), b, r1);
    r2 = _mm256_fmadd_ps(_mm256_broadcast_ss(a + 2), b, r2);
    r3 = _mm256_fmadd_ps(_mm256_broadcast_ss(a + 3), b, r3);
    r4 = _mm256_fmadd_ps(_mm256_broadcast_ss(a + 4), b, r4);
    r5 = _mm256_fmadd_ps(_mm256_broadcast_ss(a + 5), b, r5);
    r6 = _mm256_fmadd_ps(_mm256_broadcast_ss(a + 6), b, r6);
    r7 = _mm256_fmadd_ps(_mm256_broadcast_ss(a + 7), b, r7);
  }
  _mm256_storeu_ps(acc + 0, r0);
  _mm256_storeu_ps(acc + 8, r1);
  _mm256_storeu_ps(acc + 16, r2);
  _mm256_storeu_ps(acc + 24, r3);
  _mm256_storeu_ps(acc + 32, r4);
  _mm256_storeu_ps(acc + 40, r5);
  _mm256_storeu_ps(acc + 48, r6);
  _mm256_storeu_ps(acc + 56, r7);
#else
  for (int i = 0; i < 64; ++i) acc[i] = 0.f;
  for (int64_t p = 0; p < kc; ++p)
    for (int i = 0; i < 8; ++i)
      for (int j = 0; j < 8; ++j) acc[i * 8 + j] = std::fma(ap[p * 8 + i], bp[p * 8 + j], acc[i * 8 + j]);
#endif
}

// C[m, n] (row stride ldc) = A[m, k] * B[k, n], general strides for A and B, beta = 0, one thread.
void sgemm_sequential(int64_t m, int64_t k, int64_t n, const float* a, int64_t rsa, int64_t csa, const float* b, int64_t rsb, int64_t csb, float* c,
                      int64_t ldc) {
  if (m <= 0 || n <= 0) return;
  if (k <= 0) {
    for (int64_t i = 0; i < m; ++i) std::fill(c + i * ldc, c + i * ldc + n, 0.f);
    return;
  }
  std::vector<float> bpack((size_t)(kGemmKC * ((std::min(n, kGemmNC) + kGemmNR - 1) / kGemmNR) * kGemmNR));
  std::vector<float> apack((size_t)(kGemmKC * kGemmMC));
  float acc[64];
  for (int64_t jc = 0; jc < n; jc += kGemmNC) {
    const int64_t nc = std::min(kGemmNC, n - jc);
    for (int64_t pc = 0; pc < k; pc += kGemmKC) {
      const int64_t kc = std::min(kGemmKC, k - pc);
      // pack B[pc..pc+kc, jc..jc+nc] into panels of 8 columns: panel-major, then k, then the 8 columns
      for (int64_t jr = 0; jr < nc; jr += kGemmNR) {
        float* dst = bpack.data() + (jr / kGemmNR) * kc * kGemmNR;
        const int64_t w = std::min(kGemmNR, nc - jr);
        for (int64_t p = 0; p < kc; ++p) {
          const float* src = b + (pc + p) * rsb + (jc + jr) * csb;
          for (int64_t j = 0; j < w; ++j) dst[p * kGemmNR + j] = src[j * csb];
          for (int64_t j = w; j < kGemmNR; ++j) dst[p * kGemmNR + j] = 0.f;
        }
      }
      for (int64_t ic = 0; ic < m; ic += kGemmMC) {
        const int64_t mc = std::min(kGemmMC, m - ic);
        for (int64_t ir = 0; ir < mc; ir += kGemmMR) {
          float* dst = apack.data() + (ir / kGemmMR) * kc * kGemmMR;
          const int64_t h = std::min(kGemmMR, mc - ir);
          for (int64_t p = 0; p < kc; ++p) {
            const float* src = a + (ic + ir) * rsa + (pc + p) * csa;
            for (int64_t i = 0; i < h; ++i) dst[p * kGemmMR + i] = src[i * rsa];
            for (int64_t i = h; i < kGemmMR; ++i) dst[p * kGemmMR + i] = 0.f;
          }
        }
        for (int64_t jr = 0; jr < nc; jr += kGemmNR) {
          const float* bp = bpack.data() + (jr / kGemmNR) * kc * kGemmNR;
          const int64_t w = std::min(kGemmNR, nc - jr);
          for (int64_t ir = 0; ir < mc; ir += kGemmMR) {
            const float* ap = apack.data() + (ir / kGemmMR) * kc * kGemmMR;
            const int64_t h = std::min(kGemmMR, mc - ir);
            gemm_micro_8x8(kc, ap, bp, acc);
            float* ct = c + (ic + ir) * ldc + jc + jr;
            if (pc == 0) {
              for (int64_t i = 0; i < h; ++i)
                for (int64_t j = 0; j < w; ++j) ct[i * ldc + j] = acc[i * 8 + j];
            } else {
              for (int64_t i = 0; i < h; ++i)
                for (int64_t j = 0; j < w; ++j) ct[i * ldc + j] += acc[i * 8 + j];
            }
          }
        }
      }
    }
  }
}

// sgemm_maybe_parallel_ldc (conv2d.rs:884-903): row bands of A over the threads when the product is large.
void sgemm_maybe_parallel(int64_t m, int64_t k, int64_t n, const float* a, const float* b, float* c, int64_t ldc) {
  const int threads = g_threads;
  if (threads > 1 && m * k * n >= 64LL * 64 * 64 && m >= 2 * threads) {
    const int64_t chunk = std::max<int64_t>((m + threads - 1) / threads, 1);
#pragma omp parallel for num_threads(threads) schedule(static, 1)
    for (int64_t t = 0; t < threads; ++t) {
      const int64_t r0 = t * chunk;
      if (r0 < m) sgemm_sequential(std::min(chunk, m - r0), k, n, a + r0 * k, k, 1, b, n, 1, c + r0 * ldc, ldc);
    }
    return;
  }
  sgemm_sequential(m, k, n, a, k, 1, b, n, 1, c, ldc);
}

// im2col_block_cols (conv2d.rs:135-166)
int64_t im2col_block_cols(int64_t col_rows, int64_t col_cols, int64_t ow, int64_t cap_bytes) {
  const int64_t bytes_per_col = col_rows * 4;
  if (bytes_per_col == 0 || col_cols == 0) return col_cols;
  if (bytes_per_col * col_cols <= cap_bytes) return col_cols;
  const int64_t cap_cols = std::max<int64_t>(cap_bytes / bytes_per_col, 1);
  const int64_t blocks = (col_cols + cap_cols - 1) / cap_cols;
  const int64_t even = std::min(std::max<int64_t>((col_cols + blocks - 1) / std::max<int64_t>(blocks, 1), 1), cap_cols);
  if (ow > 0 && even >= ow) {
    const int64_t up = (even + ow - 1) / ow * ow;
    if (up <= cap_cols) return std::min(up, col_cols);
    const int64_t down = (even / ow) * ow;
    if (down >= 1) return std::min(down, col_cols);
  }
  return even;
}

// Columns [col0, col1) of the im2col matrix of one (batch, group): row (ic, r, s), column (oh, ow).
void im2col_block(const float* x, int64_t h, int64_t w, int64_t cpg, int64_t kh, int64_t kw, const ConvGeo& g, int64_t ow, int64_t col0, int64_t col1,
                  float* col) {
  const int64_t bw = col1 - col0;
  const int64_t sh = g.strides[0], sw = g.strides[1], dh = g.dilations[0], dw = g.dilations[1], pt = g.pads[0], pl = g.pads[1];
  for (int64_t ic = 0; ic < cpg; ++ic)
    for (int64_t r = 0; r < kh; ++r)
      for (int64_t s = 0; s < kw; ++s) {
        float* dst = col + ((ic * kh + r) * kw + s) * bw;
        const float* plane = x + ic * h * w;
        for (int64_t j = col0; j < col1; ++j) {
          const int64_t oy = j / ow, ox = j % ow;
          const int64_t iy = oy * sh - pt + r * dh, ix = ox * sw - pl + s * dw;
          dst[j - col0] = (iy >= 0 && iy < h && ix >= 0 && ix < w) ? plane[iy * w + ix] : 0.f;
        }
      }
}

void conv2d_reference_algorithm(const oxo_tensor& x, const oxo_tensor& w, const oxo_tensor* bias, const ConvGeo& g, float* y) {
  const int64_t n = x.shape[0], c_in = x.shape[1], h = x.shape[2], wd = x.shape[3];
  const int64_t c_out = w.shape[0], cpg = w.shape[1], kh = w.shape[2], kw = w.shape[3];
  const int64_t oh = g.out_shape[2], ow = g.out_shape[3];
  const int64_t group = g.group, copg = c_out / group;
  const int64_t col_rows = cpg * kh * kw, col_cols = oh * ow;
  const bool no_pad = g.pads[0] == 0 && g.pads[1] == 0 && g.pads[2] == 0 && g.pads[3] == 0;
  auto add_bias = [&](int64_t batch, int64_t grp) {
    if (!bias) return;
    for (int64_t oc = 0; oc < copg; ++oc) {
      const float bv = bias->data[grp * copg + oc];
      float* row = y + ((batch * c_out + grp * copg + oc) * col_cols);
      for (int64_t j = 0; j < col_cols; ++j) row[j] += bv;
    }
  };
  if (kh == 1 && kw == 1 && g.strides[0] == 1 && g.strides[1] == 1 && no_pad && g.dilations[0] == 1 && g.dilations[1] == 1) {
    const int64_t spatial = h * wd;
    for (int64_t batch = 0; batch < n; ++batch)
      for (int64_t grp = 0; grp < group; ++grp) {
        sgemm_maybe_parallel(copg, cpg, spatial, w.data + grp * copg * cpg, x.data + (batch * c_in + grp * cpg) * spatial,
                             y + (batch * c_out + grp * copg) * spatial, spatial);
        add_bias(batch, grp);
      }
    return;
  }
  const int64_t block_cols = im2col_block_cols(col_rows, col_cols, ow, 64LL * 1024 * 1024);
  const int64_t jobs = n * group;
  auto run_job = [&](int64_t batch, int64_t grp, std::vector<float>& col, bool parallel_gemm) {
    const float* xin = x.data + (batch * c_in + grp * cpg) * h * wd;
    const float* wm = w.data + grp * copg * col_rows;
    float* out = y + (batch * c_out + grp * copg) * col_cols;
    for (int64_t c0 = 0; c0 < col_cols; c0 += block_cols) {
      const int64_t c1 = std::min(c0 + block_cols, col_cols);
      im2col_block(xin, h, wd, cpg, kh, kw, g, ow, c0, c1, col.data());
      if (parallel_gemm) sgemm_maybe_parallel(copg, col_rows, c1 - c0, wm, col.data(), out + c0, col_cols);
      else sgemm_sequential(copg, col_rows, c1 - c0, wm, col_rows, 1, col.data(), c1 - c0, 1, out + c0, col_cols);
    }
    add_bias(batch, grp);
  };
  if (jobs <= 1 || g_threads <= 1) {
    std::vector<float> col((size_t)(col_rows * block_cols));
    for (int64_t job = 0; job < jobs; ++job) run_job(job / group, job % group, col, jobs <= 1);
    return;
  }
#pragma omp parallel num_threads(g_threads)
  {
    std::vector<float> col((size_t)(col_rows * block_cols));  // one workspace per worker (for_each_init, :506)
#pragma omp for schedule(dynamic, 1)
    for (int64_t job = 0; job < jobs; ++job) run_job(job / group, job % group, col, false);
  }
}

void op_conv(Ctx& c) {
  const char* op = "Conv";
  const oxo_tensor& x = c.input(0);
  const oxo_tensor& w = c.input(1);
  const oxo_tensor* bias = c.optional(2);
  ConvGeo g = conv_geometry(c.attrs, x, w, op, true);
  if (x.len != numel(x) || w.len != numel(w)) fail(OXO_ERR_SHAPE_MISMATCH, "Conv: data length does not match shape");
  int64_t batch = x.shape[0], c_in = x.shape[1], c_out = w.shape[0], cpg = w.shape[1];
  if (bias && bias->len != c_out) fail(OXO_ERR_SHAPE_MISMATCH, "Conv: bias has %lld entries, expected %lld", (long long)bias->len, (long long)c_out);
  int rank = g.rank;
  int64_t in_plane = 1, out_plane = 1, k_volume = 1;
  for (int d = 0; d < rank; ++d) {
    in_plane *= x.shape[d + 2];
    out_plane *= g.out_shape[(size_t)d + 2];
    k_volume *= w.shape[d + 2];
  }
  int64_t copg = c_out / g.group;
  alloc_out(c.out[0], g.out_shape);
  float* y = c.out[0].data;
  if (g_float_accum == 2 && rank == 2) {  // the reference's algorithm (im2col + blocked sgemm), for the timed baseline
    conv2d_reference_algorithm(x, w, bias, g, y);
    apply_fused_activation(c.attrs, y, c.out[0].len);
    return;
  }
  TapTable taps = build_taps(g, x.shape + 2, w.shape + 2);
  int64_t jobs = batch * c_out;
  const int accum = g_float_accum;
#pragma omp parallel for if (g_threads > 1) num_threads(g_threads) schedule(dynamic, 1)
  for (int64_t job = 0; job < jobs; ++job) {
    int64_t n = job / c_out, oc = job % c_out;
    int64_t grp = oc / copg;
    int64_t w_base = oc * cpg * k_volume;
    int64_t out_base = (n * c_out + oc) * out_plane;
    float b = bias ? bias->data[oc] : 0.0f;
    for (int64_t o = 0; o < out_plane; ++o) {
      double sum64 = 0.0;
      float sum32 = 0.0f;
      for (int64_t ic = 0; ic < cpg; ++ic) {
        int64_t plane = (n * c_in + grp * cpg + ic) * in_plane;
        for (int64_t t = taps.start[(size_t)o]; t < taps.start[(size_t)o + 1]; ++t) {
          float xv = x.data[plane + taps.in_off[(size_t)t]];
          float wv = w.data[w_base + ic * k_volume + taps.k_flat[(size_t)t]];
          if (accum == 0) sum64 += (double)xv * (double)wv;
          else sum32 += xv * wv;
        }
      }
      float r = accum == 0 ? (float)sum64 : sum32;
      y[out_base + o] = r + b;
    }
  }
  apply_fused_activation(c.attrs, y, c.out[0].len);
}

// ---------------------------------------------------------------------------------------
// MatMul / Gemm: oxionnx-ops/src/math/matmul.rs:53-190 (alpha and beta*C applied as
// separate passes after the raw product).
// ---------------------------------------------------------------------------------------
void raw_matmul(const float* a, int64_t rsa, int64_t csa, const float* b, int64_t rsb, int64_t csb, float* out, int64_t m, int64_t k, int64_t n) {
  const int accum = g_float_accum;
  if (accum == 2) {  // sgemm_strided (math_typed.rs:45): one sequential blocked sgemm
    sgemm_sequential(m, k, n, a, rsa, csa, b, rsb, csb, out, n);
    return;
  }
#pragma omp parallel for if (g_threads > 1) num_threads(g_threads)
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      double s64 = 0.0;
      float s32 = 0.0f;
      for (int64_t p = 0; p < k; ++p) {
        float av = a[i * rsa + p * csa], bv = b[p * rsb + j * csb];
        if (accum == 0) s64 += (double)av * (double)bv;
        else s32 += av * bv;
      }
      out[i * n + j] = accum == 0 ? (float)s64 : s32;
    }
  }
}

void op_matmul(Ctx& c) {
  const oxo_tensor& a = c.input(0);
  const oxo_tensor& b = c.input(1);
  if (a.len != numel(a) || b.len != numel(b)) fail(OXO_ERR_SHAPE_MISMATCH, "MatMul: data length does not match shape");
  MatMulShape s = resolve_shapes(a, b, "MatMul");
  alloc_out(c.out[0], s.out_shape);
  // batch items in parallel from four on (matmul_f32_into, math_typed.rs:355); only the timed mode threads here,
  // the other modes thread inside raw_matmul
#pragma omp parallel for if (g_float_accum == 2 && g_threads > 1 && s.batch >= 4) num_threads(g_threads)
  for (int64_t bi = 0; bi < s.batch; ++bi) {
    const float* ap = a.data + (s.a_broadcast ? 0 : bi * s.m * s.k);
    const float* bp = b.data + (s.b_broadcast ? 0 : bi * s.k * s.n);
    raw_matmul(ap, s.k, 1, bp, s.n, 1, c.out[0].data + bi * s.m * s.n, s.m, s.k, s.n);
  }
}

// unidirectional broadcast of C to [m,n] (numpy rules, right-aligned)
float bcast2(const oxo_tensor& t, int64_t i, int64_t j, int64_t m, int64_t n) {
  (void)m;
  (void)n;
  if (t.rank == 0 || t.len == 1) return t.data[0];
  if (t.rank == 1) return t.data[t.shape[0] == 1 ? 0 : j];
  int64_t r = t.shape[t.rank - 2], cc = t.shape[t.rank - 1];
  return t.data[(r == 1 ? 0 : i) * cc + (cc == 1 ? 0 : j)];
}

void op_gemm(Ctx& c) {
  const oxo_tensor& a = c.input(0);
  const oxo_tensor& b = c.input(1);
  const oxo_tensor* cc = c.optional(2);
  float alpha = c.attrs.f("alpha", 1.0f), beta = c.attrs.f("beta", 1.0f);
  bool ta = c.attrs.i("transA", 0) != 0, tb = c.attrs.i("transB", 0) != 0;
  if (a.rank != 2 || b.rank != 2) fail(OXO_ERR_UNSUPPORTED, "Gemm: oracle covers rank-2 operands only");
  int64_t m = ta ? a.shape[1] : a.shape[0], k = ta ? a.shape[0] : a.shape[1];
  int64_t k2 = tb ? b.shape[1] : b.shape[0], n = tb ? b.shape[0] : b.shape[1];
  if (k != k2) fail(OXO_ERR_SHAPE_MISMATCH, "gemm: inner dimensions mismatch %lld != %lld", (long long)k, (long long)k2);
  alloc_out(c.out[0], {m, n});
  float* y = c.out[0].data;
  raw_matmul(a.data, ta ? 1 : k, ta ? m : 1, b.data, tb ? 1 : n, tb ? k : 1, y, m, k, n);
  if (alpha != 1.0f)
    for (int64_t i = 0; i < m * n; ++i) y[i] *= alpha;
  if (cc) {
    if (cc->rank > 2) fail(OXO_ERR_UNSUPPORTED, "Gemm: C rank > 2");
    for (int64_t i = 0; i < m; ++i)
      for (int64_t j = 0; j < n; ++j) {
        volatile float bc = beta * bcast2(*cc, i, j, m, n);
        y[i * n + j] += bc;
      }
  }
}

// ---------------------------------------------------------------------------------------
// OxiInstanceNorm: oxionnx-ops/src/registry/oxi_instance_norm.rs:58-66, 153-160
// ---------------------------------------------------------------------------------------
void op_oxi_instance_norm(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  float eps = c.attrs.f("epsilon", 1e-5f);
  if (x.rank < 3) fail(OXO_ERR_SHAPE_MISMATCH, "OxiInstanceNorm: input must have rank >= 3 ([N, C, ...])");
  if (x.len != numel(x)) fail(OXO_ERR_SHAPE_MISMATCH, "OxiInstanceNorm: element count disagrees with shape");
  int64_t spatial = 1;
  for (int d = 2; d < x.rank; ++d) spatial *= x.shape[d];
  alloc_out(c.out[0], shape_of(x));
  float* y = c.out[0].data;
  if (spatial == 0 || x.len == 0) return;
  int64_t planes = x.len / spatial;
#pragma omp parallel for if (g_threads > 1) num_threads(g_threads)
  for (int64_t p = 0; p < planes; ++p) {
    const float* src = x.data + p * spatial;
    float* dst = y + p * spatial;
    float count = (float)spatial;
    float sum = 0.0f;
    for (int64_t i = 0; i < spatial; ++i) sum += src[i];
    float mean = sum / count;
    float vs = 0.0f;
    for (int64_t i = 0; i < spatial; ++i) {
      volatile float d = src[i] - mean;
      volatile float dd = d * d;
      vs += dd;
    }
    float var = vs / count;
    float inv_std = 1.0f / std::sqrt(var + eps);
    for (int64_t i = 0; i < spatial; ++i) {
      volatile float d = src[i] - mean;
      dst[i] = d * inv_std;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Element-wise glue: oxionnx-ops/src/math/broadcast.rs:219-249 (numpy broadcasting),
// oxionnx-ops/src/nn/activations.rs:5 (relu), :43 (tanh), :100 (prelu), :271 (silu).
// ---------------------------------------------------------------------------------------
std::vector<int64_t> broadcast_shape(const oxo_tensor& a, const oxo_tensor& b, const char* op) {
  int r = std::max(a.rank, b.rank);
  std::vector<int64_t> out((size_t)r);
  for (int i = 0; i < r; ++i) {
    int64_t da = i < r - a.rank ? 1 : a.shape[i - (r - a.rank)];
    int64_t db = i < r - b.rank ? 1 : b.shape[i - (r - b.rank)];
    if (da != db && da != 1 && db != 1) fail(OXO_ERR_SHAPE_MISMATCH, "%s: shapes are not broadcastable", op);
    out[(size_t)i] = std::max(da, db);
    if (da == 0 || db == 0) out[(size_t)i] = 0;
  }
  return out;
}

template <class F>
void binary_op(Ctx& c, F f) {
  const oxo_tensor& a = c.input(0);
  const oxo_tensor& b = c.input(1);
  auto os = broadcast_shape(a, b, c.op);
  alloc_out(c.out[0], os);
  int r = (int)os.size();
  std::vector<int64_t> sa((size_t)r, 0), sb((size_t)r, 0);
  int64_t st = 1;
  for (int i = a.rank - 1; i >= 0; --i) {
    sa[(size_t)(i + r - a.rank)] = a.shape[i] == 1 ? 0 : st;
    st *= a.shape[i];
  }
  st = 1;
  for (int i = b.rank - 1; i >= 0; --i) {
    sb[(size_t)(i + r - b.rank)] = b.shape[i] == 1 ? 0 : st;
    st *= b.shape[i];
  }
  float* y = c.out[0].data;
  int64_t n = c.out[0].len;
  if (a.len == n && b.len == n) {  // same shape: one straight pass (the reference's simd_add / simd_mul path, math/broadcast.rs:219-249)
    const float* pa = a.data;
    const float* pb = b.data;
    for (int64_t i = 0; i < n; ++i) y[i] = f(pa[i], pb[i]);
    return;
  }
#pragma omp parallel for if (g_threads > 1) num_threads(g_threads)
  for (int64_t flat = 0; flat < n; ++flat) {
    int64_t rem = flat, ia = 0, ib = 0;
    for (int d = r - 1; d >= 0; --d) {
      int64_t idx = rem % os[(size_t)d];
      rem /= os[(size_t)d];
      ia += idx * sa[(size_t)d];
      ib += idx * sb[(size_t)d];
    }
    y[flat] = f(a.data[ia], b.data[ib]);
  }
}

template <class F>
void unary_op(Ctx& c, F f) {
  const oxo_tensor& x = c.input(0);
  alloc_out(c.out[0], shape_of(x));
  for (int64_t i = 0; i < x.len; ++i) c.out[0].data[i] = f(x.data[i]);
}

void op_prelu(Ctx& c) {
  // slope broadcasts unidirectionally to x (per-channel [C,1,1] or scalar)
  binary_op(c, [](float x, float s) { return x >= 0.0f ? x : x * s; });
}

// ---------------------------------------------------------------------------------------
// Pooling: oxionnx-ops/src/conv/pooling.rs:166-260 (max_pool_into), :462-480
// (global_avg_pool: sequential f32 sum, then divide by the count).
// ---------------------------------------------------------------------------------------
void op_max_pool(Ctx& c) {
  const char* op = "MaxPool";
  const oxo_tensor& x = c.input(0);
  if (x.rank < 3) fail(OXO_ERR_SHAPE_MISMATCH, "MaxPool: input must have rank >= 3");
  int rank = x.rank - 2;
  auto ks = c.attrs.ints("kernel_shape");
  if ((int)ks.size() < rank) fail(OXO_ERR_SHAPE_MISMATCH, "MaxPool: kernel_shape requires %d spatial dims, got %zu", rank, ks.size());
  for (int a = 0; a < rank; ++a)
    if (ks[(size_t)a] < 1) fail(OXO_ERR_SHAPE_MISMATCH, "MaxPool: kernel_shape[%d] must be >= 1", a);
  ConvGeo g;
  g.rank = rank;
  g.strides = read_positive_spatial(c.attrs.ints("strides"), rank, "strides", op);
  g.dilations = read_positive_spatial(c.attrs.ints("dilations"), rank, "dilations", op);
  auto explicit_pads = read_pads(c.attrs.ints("pads"), rank, op);
  AutoPad ap = parse_auto_pad(c.attrs.s("auto_pad"), op);
  g.pads = resolve_pads(ap, x.shape + 2, ks.data(), g.strides, g.dilations, explicit_pads, rank);
  bool ceil_mode = c.attrs.i("ceil_mode", 0) != 0;
  g.out_shape = {x.shape[0], x.shape[1]};
  for (int a = 0; a < rank; ++a)
    g.out_shape.push_back(
        pool_out_dim(op, a, x.shape[a + 2], g.pads[(size_t)a], g.pads[(size_t)(a + rank)], ks[(size_t)a], g.dilations[(size_t)a], g.strides[(size_t)a], ceil_mode));
  TapTable taps = build_taps(g, x.shape + 2, ks.data());
  int64_t in_plane = 1, out_plane = 1;
  for (int d = 0; d < rank; ++d) {
    in_plane *= x.shape[d + 2];
    out_plane *= g.out_shape[(size_t)d + 2];
  }
  alloc_out(c.out[0], g.out_shape);
  float* y = c.out[0].data;
  int64_t planes = x.shape[0] * x.shape[1];
#pragma omp parallel for if (g_threads > 1) num_threads(g_threads)
  for (int64_t p = 0; p < planes; ++p)
    for (int64_t o = 0; o < out_plane; ++o) {
      float mx = -std::numeric_limits<float>::infinity();
      for (int64_t t = taps.start[(size_t)o]; t < taps.start[(size_t)o + 1]; ++t) {
        float v = x.data[p * in_plane + taps.in_off[(size_t)t]];
        if (v > mx) mx = v;
      }
      y[p * out_plane + o] = mx;
    }
}

void op_global_average_pool(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  if (x.rank < 3) {
    alloc_out(c.out[0], shape_of(x));
    std::copy(x.data, x.data + x.len, c.out[0].data);
    return;
  }
  int64_t n = x.shape[0], ch = x.shape[1], spatial = 1;
  for (int d = 2; d < x.rank; ++d) spatial *= x.shape[d];
  std::vector<int64_t> os = {n, ch};
  for (int d = 2; d < x.rank; ++d) os.push_back(1);
  alloc_out(c.out[0], os);
  for (int64_t p = 0; p < n * ch; ++p) {
    float sum = 0.0f;
    for (int64_t i = 0; i < spatial; ++i) sum += x.data[p * spatial + i];
    c.out[0].data[p] = sum / (float)spatial;
  }
}

// ---------------------------------------------------------------------------------------
// Shape glue: Flatten / Reshape (row-major reinterpretation), Concat
// (oxionnx-ops/src/shape/sequence.rs:8), Pad constant/reflect (:356), Cast (f32 lanes are
// already the value representation, so a cast between the lane types used here copies).
// ---------------------------------------------------------------------------------------
void op_flatten(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  int64_t axis = c.attrs.i("axis", 1);
  if (axis < 0) axis += x.rank;
  if (axis < 0 || axis > x.rank) fail(OXO_ERR_INVALID_MODEL, "Flatten: axis out of range");
  int64_t outer = 1, inner = 1;
  for (int d = 0; d < x.rank; ++d) (d < axis ? outer : inner) *= x.shape[d];
  alloc_out(c.out[0], {outer, inner});
  std::copy(x.data, x.data + x.len, c.out[0].data);
}

void op_reshape(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  const oxo_tensor& sh = c.input(1);
  bool allowzero = c.attrs.i("allowzero", 0) != 0;
  std::vector<int64_t> os;
  int64_t known = 1;
  int infer = -1;
  for (int64_t i = 0; i < sh.len; ++i) {
    int64_t d = (int64_t)sh.data[i];
    if (d == -1) {
      if (infer >= 0) fail(OXO_ERR_INVALID_MODEL, "Reshape: more than one -1");
      infer = (int)i;
      os.push_back(1);
      continue;
    }
    if (d == 0 && !allowzero) {
      if (i >= x.rank) fail(OXO_ERR_INVALID_MODEL, "Reshape: 0 dim out of range");
      d = x.shape[i];
    }
    os.push_back(d);
    known *= d;
  }
  if (infer >= 0) {
    if (known == 0 || x.len % known != 0) fail(OXO_ERR_SHAPE_MISMATCH, "Reshape: cannot infer dimension");
    os[(size_t)infer] = x.len / known;
    known *= os[(size_t)infer];
  }
  if (known != x.len) fail(OXO_ERR_SHAPE_MISMATCH, "Reshape: element count changes");
  alloc_out(c.out[0], os);
  std::copy(x.data, x.data + x.len, c.out[0].data);
}

void op_concat(Ctx& c) {
  const oxo_tensor& first = c.input(0);
  int64_t axis = c.attrs.i("axis", 0);
  if (axis < 0) axis += first.rank;
  if (axis < 0 || axis >= first.rank) fail(OXO_ERR_INVALID_MODEL, "Concat: axis out of range");
  std::vector<int64_t> os = shape_of(first);
  os[(size_t)axis] = 0;
  for (int i = 0; i < c.n_in; ++i) {
    const oxo_tensor& t = c.input(i);
    if (t.rank != first.rank) fail(OXO_ERR_SHAPE_MISMATCH, "Concat: rank mismatch");
    for (int d = 0; d < t.rank; ++d)
      if (d != axis && t.shape[d] != first.shape[d]) fail(OXO_ERR_SHAPE_MISMATCH, "Concat: non-axis dims disagree");
    os[(size_t)axis] += t.shape[axis];
  }
  alloc_out(c.out[0], os);
  int64_t outer = 1, inner = 1;
  for (int d = 0; d < axis; ++d) outer *= os[(size_t)d];
  for (int d = (int)axis + 1; d < first.rank; ++d) inner *= os[(size_t)d];
  int64_t off = 0;
  for (int i = 0; i < c.n_in; ++i) {
    const oxo_tensor& t = c.in[i];
    int64_t chunk = t.shape[axis] * inner;
    for (int64_t o = 0; o < outer; ++o) std::copy(t.data + o * chunk, t.data + (o + 1) * chunk, c.out[0].data + o * os[(size_t)axis] * inner + off);
    off += chunk;
  }
}

// Slice (oxionnx-ops src/registry/shape_ops/concat_slice_ops.rs:27-53, src/shape/sequence.rs:52-150):
// starts/ends/axes/steps arrive as f32 lanes cast to i64 (saturating); negative start/end count
// from the end of the axis, then clamp to [0, dim] (positive step) or [-1, dim-1] (negative
// step); axes not named pass through whole.
int64_t lane_as_i64(float v) {
  if (std::isnan(v)) return 0;
  if (v >= 9.2233720368547758e18f) return INT64_MAX;
  if (v <= -9.2233720368547758e18f) return INT64_MIN;
  return (int64_t)v;
}

void op_slice(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  const oxo_tensor& st = c.input(1);
  const oxo_tensor& en = c.input(2);
  const oxo_tensor* ax = c.optional(3);
  const oxo_tensor* sp = c.optional(4);
  const int64_t n = st.len;
  if (en.len != n || (ax && ax->len != n) || (sp && sp->len != n)) fail(OXO_ERR_SHAPE_MISMATCH, "slice: starts/ends/axes/steps length mismatch");
  const int rank = x.rank;
  std::vector<int64_t> ds(rank, 0), de(rank), dp(rank, 1);
  for (int d = 0; d < rank; ++d) de[d] = x.shape[d];
  for (int64_t i = 0; i < n; ++i) {
    int64_t a = ax ? lane_as_i64(ax->data[i]) : i;
    if (a < 0) a += rank;
    if (a < 0 || a >= rank) fail(OXO_ERR_INVALID_MODEL, "slice: axis out of range");
    const int64_t dim = x.shape[a];
    const int64_t step = sp ? lane_as_i64(sp->data[i]) : 1;
    if (step == 0) fail(OXO_ERR_INVALID_MODEL, "slice: steps must not be 0");
    if (step == INT64_MIN) fail(OXO_ERR_INVALID_MODEL, "slice: steps out of range");
    int64_t s0 = lane_as_i64(st.data[i]), e0 = lane_as_i64(en.data[i]);
    if (s0 < 0) s0 += dim;  // a negative value plus a dimension cannot overflow
    if (e0 < 0) e0 += dim;
    if (step > 0) {
      s0 = std::min(std::max<int64_t>(s0, 0), dim);
      e0 = std::min(std::max<int64_t>(e0, 0), dim);
    } else {
      s0 = std::min(std::max<int64_t>(s0, -1), dim - 1);
      e0 = std::min(std::max<int64_t>(e0, -1), dim - 1);
    }
    ds[a] = s0, de[a] = e0, dp[a] = step;
  }
  std::vector<int64_t> os(rank);
  for (int d = 0; d < rank; ++d) {
    if (dp[d] > 0) os[d] = de[d] <= ds[d] ? 0 : (de[d] - ds[d] + dp[d] - 1) / dp[d];
    else os[d] = ds[d] <= de[d] ? 0 : (ds[d] - de[d] + (-dp[d]) - 1) / (-dp[d]);
  }
  alloc_out(c.out[0], os);
  const int64_t total = c.out[0].len;
  std::vector<int64_t> xs(rank, 1);
  for (int d = rank - 2; d >= 0; --d) xs[d] = xs[d + 1] * x.shape[d + 1];
  std::vector<int64_t> idx(rank, 0);
  for (int64_t o = 0; o < total; ++o) {
    int64_t src = 0;
    for (int d = 0; d < rank; ++d) src += (ds[d] + idx[d] * dp[d]) * xs[d];
    c.out[0].data[o] = x.data[src];
    for (int d = rank - 1; d >= 0; --d) {
      if (++idx[d] < os[d]) break;
      idx[d] = 0;
    }
  }
}

// ---------------------------------------------------------------------------------------
// Transformer glue for the dynamic-INT8 encoder (float, tolerance-checked).
// Gather: oxionnx-ops/src/indexing/gather.rs:12-44 (negative indices wrap, out of range is an error).
// Transpose: src/shape/basic.rs:146-230 (empty perm reverses; perm must be a permutation).
// Softmax: src/nn/normalization.rs:300-360 (max, exp(v - max) summed in order, multiply by 1/sum).
// LayerNormalization: src/nn/normalization.rs layer_norm_into (mean and variance as sequential f32
//   sums over the normalised group, inv_std = 1/sqrt(var + eps), (x - mean) * inv_std * scale, + bias).
// Gelu: src/registry/nn_ops/activations.rs:357-386 (approximate="tanh" -> 0.5 x (1 + tanh(0.7978846 (x +
//   0.044715 x^3))); otherwise x * 0.5 * (1 + erf(x / sqrt 2)) with the Abramowitz-Stegun 7.1.26
//   polynomial of erf_approx :578-586).  Erf uses the same polynomial.
// ---------------------------------------------------------------------------------------
float erf_poly(float x) {
  const float sign = x >= 0.0f ? 1.0f : -1.0f;
  x = std::fabs(x);
  const float t = 1.0f / (1.0f + 0.3275911f * x);
  const float poly = t * (0.2548296f + t * (-0.28449672f + t * (1.4214138f + t * (-1.4531521f + t * 1.0614054f))));
  return sign * (1.0f - poly * std::exp(-x * x));
}

void op_gelu(Ctx& c) {
  if (c.attrs.s("approximate") == "tanh") {
    unary_op(c, [](float x) {
      const float inner = 0.7978846f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.0f + std::tanh(inner));
    });
  } else {
    unary_op(c, [](float x) { return x * 0.5f * (1.0f + erf_poly(x * 0.70710678118654752440f)); });
  }
}

void op_gather(Ctx& c) {
  const oxo_tensor& data = c.input(0);
  const oxo_tensor& idx = c.input(1);
  int64_t axis = c.attrs.i("axis", 0);
  if (axis < 0) axis += data.rank;
  if (axis < 0 || axis >= data.rank) fail(OXO_ERR_INVALID_MODEL, "gather: axis out of range");
  std::vector<int64_t> os;
  for (int d = 0; d < axis; ++d) os.push_back(data.shape[d]);
  for (int d = 0; d < idx.rank; ++d) os.push_back(idx.shape[d]);
  for (int d = (int)axis + 1; d < data.rank; ++d) os.push_back(data.shape[d]);
  int64_t outer = 1, inner = 1;
  for (int d = 0; d < axis; ++d) outer *= data.shape[d];
  for (int d = (int)axis + 1; d < data.rank; ++d) inner *= data.shape[d];
  const int64_t axis_size = data.shape[axis], idx_n = idx.len;
  alloc_out(c.out[0], os);
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t ii = 0; ii < idx_n; ++ii) {
      int64_t iv = (int64_t)idx.data[ii];
      if (iv < 0) iv += axis_size;
      if (iv < 0 || iv >= axis_size) fail(OXO_ERR_INVALID_MODEL, "gather: index out of range");
      std::copy(data.data + (o * axis_size + iv) * inner, data.data + (o * axis_size + iv + 1) * inner, c.out[0].data + (o * idx_n + ii) * inner);
    }
}

void op_transpose(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  const int rank = x.rank;
  std::vector<int64_t> perm = c.attrs.ints("perm");
  if (perm.empty())
    for (int d = rank - 1; d >= 0; --d) perm.push_back(d);
  if ((int)perm.size() != rank) fail(OXO_ERR_INVALID_MODEL, "transpose: perm length differs from the rank");
  std::vector<char> seen(rank, 0);
  for (int64_t pv : perm) {
    if (pv < 0 || pv >= rank) fail(OXO_ERR_INVALID_MODEL, "transpose: perm entry out of range");
    if (seen[pv]) fail(OXO_ERR_INVALID_MODEL, "transpose: perm entry repeated");
    seen[pv] = 1;
  }
  std::vector<int64_t> os(rank), xs(rank, 1);
  for (int d = rank - 2; d >= 0; --d) xs[d] = xs[d + 1] * x.shape[d + 1];
  for (int d = 0; d < rank; ++d) os[d] = x.shape[perm[d]];
  alloc_out(c.out[0], os);
  std::vector<int64_t> idx(rank, 0);
  for (int64_t o = 0; o < c.out[0].len; ++o) {
    int64_t src = 0;
    for (int d = 0; d < rank; ++d) src += idx[d] * xs[perm[d]];
    c.out[0].data[o] = x.data[src];
    for (int d = rank - 1; d >= 0; --d) {
      if (++idx[d] < os[d]) break;
      idx[d] = 0;
    }
  }
}

void op_softmax(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  int64_t axis = c.attrs.i("axis", -1);
  if (axis < 0) axis += x.rank;
  if (axis < 0 || axis >= x.rank) fail(OXO_ERR_INVALID_MODEL, "softmax: axis out of range");
  int64_t outer = 1, inner = 1;
  for (int d = 0; d < axis; ++d) outer *= x.shape[d];
  for (int d = (int)axis + 1; d < x.rank; ++d) inner *= x.shape[d];
  const int64_t n = x.shape[axis];
  alloc_out(c.out[0], shape_of(x));
  float* out = c.out[0].data;
#pragma omp parallel for collapse(2) schedule(static) if (outer * inner * n > 65536)
  for (int64_t o = 0; o < outer; ++o)
    for (int64_t i = 0; i < inner; ++i) {
      const float* px = x.data + o * n * inner + i;
      float* py = out + o * n * inner + i;
      float mx = -INFINITY;
      for (int64_t k = 0; k < n; ++k) mx = px[k * inner] > mx ? px[k * inner] : mx;
      float sum = 0.0f;
      for (int64_t k = 0; k < n; ++k) {
        const float e = std::exp(px[k * inner] - mx);
        py[k * inner] = e;
        sum += e;
      }
      const float inv = 1.0f / sum;
      for (int64_t k = 0; k < n; ++k) py[k * inner] *= inv;
    }
}

void op_layer_norm(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  const oxo_tensor& scale = c.input(1);
  const oxo_tensor* bias = c.optional(2);
  int64_t axis = c.attrs.i("axis", -1);
  const float eps = c.attrs.f("epsilon", 1e-5f);
  if (axis < 0) axis += x.rank;
  if (axis < 0 || axis >= x.rank) fail(OXO_ERR_INVALID_MODEL, "layer_norm: axis out of range");
  int64_t outer = 1, norm = 1;
  for (int d = 0; d < axis; ++d) outer *= x.shape[d];
  for (int d = (int)axis; d < x.rank; ++d) norm *= x.shape[d];
  if (norm == 0 || scale.len == 0 || (bias && bias->len == 0)) fail(OXO_ERR_SHAPE_MISMATCH, "layer_norm: empty operand");
  alloc_out(c.out[0], shape_of(x));
  float* out = c.out[0].data;
#pragma omp parallel for schedule(static) if (outer * norm > 65536)
  for (int64_t o = 0; o < outer; ++o) {
    const float* in = x.data + o * norm;
    float* dst = out + o * norm;
    float sum = 0.0f;
    for (int64_t j = 0; j < norm; ++j) sum += in[j];
    const float mean = sum / (float)norm;
    float vs = 0.0f;
    for (int64_t j = 0; j < norm; ++j) {
      const float d = in[j] - mean;
      vs += d * d;
    }
    const float var = vs / (float)norm;
    const float inv_std = 1.0f / std::sqrt(var + eps);
    for (int64_t j = 0; j < norm; ++j) dst[j] = (in[j] - mean) * inv_std * scale.data[j % scale.len];
    if (bias)
      for (int64_t j = 0; j < norm; ++j) dst[j] += bias->data[j % bias->len];
  }
}

void op_pad(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  std::vector<int64_t> pads;
  if (const oxo_tensor* p = c.optional(1)) {
    for (int64_t i = 0; i < p->len; ++i) pads.push_back((int64_t)p->data[i]);
  } else {
    pads = c.attrs.ints("pads");
  }
  if ((int)pads.size() != 2 * x.rank) fail(OXO_ERR_SHAPE_MISMATCH, "Pad: pads must have 2*rank entries");
  float cval = 0.0f;
  if (const oxo_tensor* v = c.optional(2)) {
    if (v->len > 0) cval = v->data[0];
  } else {
    cval = c.attrs.f("value", 0.0f);
  }
  std::string mode = c.attrs.s("mode");
  if (mode.empty()) mode = "constant";
  if (mode != "constant" && mode != "reflect" && mode != "edge") fail(OXO_ERR_UNSUPPORTED, "Pad: unsupported mode '%s'", mode.c_str());
  std::vector<int64_t> os = shape_of(x);
  for (int d = 0; d < x.rank; ++d) {
    if (pads[(size_t)d] < 0 || pads[(size_t)(d + x.rank)] < 0) fail(OXO_ERR_UNSUPPORTED, "Pad: negative pads not covered by the oracle");
    os[(size_t)d] += pads[(size_t)d] + pads[(size_t)(d + x.rank)];
    if (mode == "reflect" && (pads[(size_t)d] >= x.shape[d] || pads[(size_t)(d + x.rank)] >= x.shape[d]) && x.shape[d] > 0 &&
        (pads[(size_t)d] > 0 || pads[(size_t)(d + x.rank)] > 0))
      fail(OXO_ERR_INVALID_MODEL, "Pad: reflect pad must be smaller than the axis extent");
  }
  alloc_out(c.out[0], os);
  std::vector<int64_t> xs((size_t)x.rank, 1);
  for (int d = x.rank - 2; d >= 0; --d) xs[(size_t)d] = xs[(size_t)d + 1] * x.shape[d + 1];
  for (int64_t flat = 0; flat < c.out[0].len; ++flat) {
    int64_t rem = flat, src = 0;
    bool outside = false;
    for (int d = x.rank - 1; d >= 0; --d) {
      int64_t idx = rem % os[(size_t)d] - pads[(size_t)d];
      rem /= os[(size_t)d];
      int64_t ext = x.shape[d];
      if (idx < 0 || idx >= ext) {
        if (mode == "constant") outside = true;
        else if (mode == "edge") idx = idx < 0 ? 0 : ext - 1;
        else idx = idx < 0 ? -idx : 2 * (ext - 1) - idx;
      }
      if (!outside) src += idx * xs[(size_t)d];
    }
    c.out[0].data[flat] = outside ? cval : x.data[src];
  }
}

void op_identity(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  alloc_out(c.out[0], shape_of(x));
  std::copy(x.data, x.data + x.len, c.out[0].data);
}

// Resize, nearest and linear, for the 4-D NCHW upsampling the face-swap decoder uses:
// oxionnx-ops/src/resize.rs (coordinate transforms half_pixel / pytorch_half_pixel /
// asymmetric / align_corners; nearest_mode round_prefer_floor / floor / ceil /
// round_prefer_ceil).  Only scale factors on the two spatial axes are covered.
float resize_src_coord(const std::string& mode, int64_t o, float scale, int64_t in_size, int64_t out_size) {
  if (mode == "asymmetric") return (float)o / scale;
  if (mode == "align_corners") return out_size <= 1 ? 0.0f : (float)o * (float)(in_size - 1) / (float)(out_size - 1);
  if (mode == "pytorch_half_pixel") return out_size > 1 ? ((float)o + 0.5f) / scale - 0.5f : 0.0f;
  return ((float)o + 0.5f) / scale - 0.5f;  // half_pixel
}

void op_resize(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  if (x.rank != 4) fail(OXO_ERR_UNSUPPORTED, "Resize: oracle covers NCHW rank-4 input only");
  const oxo_tensor* scales = c.optional(2);
  const oxo_tensor* sizes = c.optional(3);
  std::string mode = c.attrs.s("mode");
  if (mode.empty()) mode = "nearest";
  std::string coord = c.attrs.s("coordinate_transformation_mode");
  if (coord.empty()) coord = "half_pixel";
  std::string nearest = c.attrs.s("nearest_mode");
  if (nearest.empty()) nearest = "round_prefer_floor";
  if (c.attrs.i("antialias", 0) != 0) fail(OXO_ERR_UNSUPPORTED, "Resize: antialias not covered by the oracle");
  if (coord != "half_pixel" && coord != "pytorch_half_pixel" && coord != "asymmetric" && coord != "align_corners")
    fail(OXO_ERR_UNSUPPORTED, "Resize: coordinate mode '%s' not covered by the oracle", coord.c_str());
  std::vector<int64_t> os = shape_of(x);
  float sc[4] = {1, 1, 1, 1};
  if (scales && scales->len == 4) {
    for (int d = 0; d < 4; ++d) {
      sc[d] = scales->data[d];
      os[(size_t)d] = (int64_t)std::floor((float)x.shape[d] * sc[d]);
    }
  } else if (sizes && sizes->len == 4) {
    for (int d = 0; d < 4; ++d) {
      os[(size_t)d] = (int64_t)sizes->data[d];
      sc[d] = (float)os[(size_t)d] / (float)x.shape[d];
    }
  } else {
    fail(OXO_ERR_INVALID_MODEL, "Resize: needs scales or sizes with 4 entries");
  }
  if (os[0] != x.shape[0] || os[1] != x.shape[1]) fail(OXO_ERR_UNSUPPORTED, "Resize: only spatial axes may change in the oracle");
  alloc_out(c.out[0], os);
  int64_t H = x.shape[2], W = x.shape[3], OH = os[2], OW = os[3];
  bool lin = mode == "linear" || mode == "bilinear";
  if (!lin && mode != "nearest") fail(OXO_ERR_UNSUPPORTED, "Resize: mode '%s' not covered by the oracle", mode.c_str());
  auto nearest_idx = [&](float s, int64_t in_size) {
    float r;
    if (nearest == "floor") r = std::floor(s);
    else if (nearest == "ceil") r = std::ceil(s);
    else if (nearest == "round_prefer_ceil") r = std::floor(s + 0.5f);
    else r = std::ceil(s - 0.5f);  // round_prefer_floor
    int64_t i = (int64_t)r;
    return std::min<int64_t>(std::max<int64_t>(i, 0), in_size - 1);
  };
  for (int64_t p = 0; p < x.shape[0] * x.shape[1]; ++p) {
    const float* src = x.data + p * H * W;
    float* dst = c.out[0].data + p * OH * OW;
    for (int64_t oy = 0; oy < OH; ++oy) {
      float sy = resize_src_coord(coord, oy, sc[2], H, OH);
      for (int64_t ox = 0; ox < OW; ++ox) {
        float sx = resize_src_coord(coord, ox, sc[3], W, OW);
        if (!lin) {
          dst[oy * OW + ox] = src[nearest_idx(sy, H) * W + nearest_idx(sx, W)];
        } else {
          float cy = std::min(std::max(sy, 0.0f), (float)(H - 1)), cx = std::min(std::max(sx, 0.0f), (float)(W - 1));
          int64_t y0 = (int64_t)std::floor(cy), x0 = (int64_t)std::floor(cx);
          int64_t y1 = std::min(y0 + 1, H - 1), x1 = std::min(x0 + 1, W - 1);
          float fy = cy - (float)y0, fx = cx - (float)x0;
          float top = src[y0 * W + x0] * (1.0f - fx) + src[y0 * W + x1] * fx;
          float bot = src[y1 * W + x0] * (1.0f - fx) + src[y1 * W + x1] * fx;
          dst[oy * OW + ox] = top * (1.0f - fy) + bot * fy;
        }
      }
    }
  }
}

// BatchNormalization, inference form: oxionnx-ops/src/nn/normalization.rs:132-166 --
// out = (x - mean) * (1 / sqrt(var + eps)) * scale + bias, each step rounded to f32 in that order.
void op_batch_norm(Ctx& c) {
  const oxo_tensor& x = c.input(0);
  if (x.rank < 2) fail(OXO_ERR_SHAPE_MISMATCH, "batch_norm: need at least 2D");
  const oxo_tensor &scale = c.input(1), &bias = c.input(2), &mean = c.input(3), &var = c.input(4);
  const int64_t n = x.shape[0], ch = x.shape[1];
  for (const oxo_tensor* t : {&scale, &bias, &mean, &var})
    if (t->len < ch) fail(OXO_ERR_SHAPE_MISMATCH, "batch_norm: a parameter has %lld entries, expected %lld", (long long)t->len, (long long)ch);
  int64_t spatial = 1;
  for (int d = 2; d < x.rank; ++d) spatial *= x.shape[d];
  const float eps = c.attrs.f("epsilon", 1e-5f);
  alloc_out(c.out[0], std::vector<int64_t>(x.shape, x.shape + x.rank));
  float* y = c.out[0].data;
  for (int64_t ni = 0; ni < n; ++ni)
    for (int64_t ci = 0; ci < ch; ++ci) {
      const float inv_std = 1.0f / std::sqrt(var.data[ci] + eps);
      const float s = scale.data[ci], b = bias.data[ci], m = mean.data[ci];
      const int64_t base = (ni * ch + ci) * spatial;
      for (int64_t si = 0; si < spatial; ++si) {
        volatile float d = x.data[base + si] - m;
        volatile float t = d * inv_std;
        volatile float u = t * s;
        y[base + si] = u + b;
      }
    }
}

// ConvAddRelu, the node fuse_conv_add_relu emits (src/optimizer/fusion/conv/add_relu.rs:27-156): inputs
// (x, w, bias or "", residual) and the Conv's attributes; its value is the unfused chain's,
// relu(conv(x, w, bias) + residual), every step rounded to f32.
void op_conv_add_relu(Ctx& c) {
  if (c.n_in < 4) fail(OXO_ERR_SHAPE_MISMATCH, "ConvAddRelu: expected inputs (x, w, bias, residual)");
  Ctx conv{c.op, c.in, 3, c.attrs, c.out, c.n_out};
  op_conv(conv);
  const oxo_tensor& r = c.input(3);
  oxo_tensor& y = c.out[0];
  if (r.len != y.len) fail(OXO_ERR_SHAPE_MISMATCH, "ConvAddRelu: residual has %lld entries, the convolution %lld", (long long)r.len, (long long)y.len);
  for (int64_t i = 0; i < y.len; ++i) y.data[i] = std::max(y.data[i] + r.data[i], 0.0f);
}

struct OpEntry {
  const char* name;
  void (*fn)(Ctx&);
  int min_out;
};

const OpEntry kOps[] = {
    {"QuantizeLinear", op_quantize_linear, 1},
    {"DequantizeLinear", op_dequantize_linear, 1},
    {"DynamicQuantizeLinear", op_dynamic_quantize_linear, 1},
    {"MatMulInteger", op_matmul_integer, 1},
    {"QLinearMatMul", op_qlinear_matmul, 1},
    {"QLinearConv", op_qlinear_conv, 1},
    {"ConvInteger", op_conv_integer, 1},
    {"Conv", op_conv, 1},
    {"MatMul", op_matmul, 1},
    {"Gemm", op_gemm, 1},
    {"OxiInstanceNorm", op_oxi_instance_norm, 1},
    {"Add", [](Ctx& c) { binary_op(c, [](float a, float b) { return a + b; }); }, 1},
    {"Sub", [](Ctx& c) { binary_op(c, [](float a, float b) { return a - b; }); }, 1},
    {"Mul", [](Ctx& c) { binary_op(c, [](float a, float b) { return a * b; }); }, 1},
    {"Div", [](Ctx& c) { binary_op(c, [](float a, float b) { return a / b; }); }, 1},
    {"Relu", [](Ctx& c) { unary_op(c, [](float v) { return std::max(v, 0.0f); }); }, 1},
    {"Tanh", [](Ctx& c) { unary_op(c, [](float v) { return std::tanh(v); }); }, 1},
    {"Sigmoid", [](Ctx& c) { unary_op(c, [](float v) { return 1.0f / (1.0f + std::exp(-v)); }); }, 1},
    {"Silu", [](Ctx& c) { unary_op(c, [](float v) { return v / (1.0f + std::exp(-v)); }); }, 1},
    {"SiLU", [](Ctx& c) { unary_op(c, [](float v) { return v / (1.0f + std::exp(-v)); }); }, 1},
    {"PRelu", op_prelu, 1},
    {"BatchNormalization", op_batch_norm, 1},
    {"ConvAddRelu", op_conv_add_relu, 1},
    {"MaxPool", op_max_pool, 1},
    {"GlobalAveragePool", op_global_average_pool, 1},
    {"Flatten", op_flatten, 1},
    {"Reshape", op_reshape, 1},
    {"Concat", op_concat, 1},
    {"Pad", op_pad, 1},
    {"Slice", op_slice, 1},
    {"Gather", op_gather, 1},
    {"Transpose", op_transpose, 1},
    {"Softmax", op_softmax, 1},
    {"LayerNormalization", op_layer_norm, 1},
    {"LayerNorm", op_layer_norm, 1},
    {"Gelu", op_gelu, 1},
    {"Erf", [](Ctx& c) { unary_op(c, [](float v) { return erf_poly(v); }); }, 1},
    {"Resize", op_resize, 1},
    {"Cast", op_identity, 1},
    {"Identity", op_identity, 1},
};

}  // namespace

extern "C" {

int oxo_run_node(const char* op_type, const oxo_tensor* inputs, int32_t n_inputs, const oxo_attr* attrs, int32_t n_attrs, oxo_tensor* outputs,
                 int32_t n_outputs) {
  for (int i = 0; i < n_outputs; ++i) std::memset(&outputs[i], 0, sizeof(oxo_tensor));
  try {
    for (const OpEntry& e : kOps) {
      if (std::strcmp(e.name, op_type) == 0) {
        if (n_outputs < e.min_out) fail(OXO_ERR_INTERNAL, "%s: expected at least %d output slot(s)", op_type, e.min_out);
        Ctx c{op_type, inputs, n_inputs, Attrs{attrs, n_attrs}, outputs, n_outputs};
        e.fn(c);
        return OXO_OK;
      }
    }
    fail(OXO_ERR_UNSUPPORTED, "operator '%s' is not covered by the oracle", op_type);
  } catch (const Fail& f) {
    for (int i = 0; i < n_outputs; ++i) oxo_free_tensor(&outputs[i]);
    return f.code;
  } catch (const std::exception& e) {
    g_err = e.what();
    for (int i = 0; i < n_outputs; ++i) oxo_free_tensor(&outputs[i]);
    return OXO_ERR_INTERNAL;
  }
}

void oxo_free_tensor(oxo_tensor* t) {
  if (t && t->data) {
    std::free(t->data);
    t->data = nullptr;
  }
}

const char* oxo_last_error(void) { return g_err.c_str(); }
void oxo_set_threads(int32_t threads) { g_threads = threads < 1 ? 1 : threads; }
int32_t oxo_get_threads(void) { return g_threads; }
void oxo_set_float_accum(int32_t mode) { g_float_accum = (mode == 1 || mode == 2) ? mode : 0; }
double oxo_round_ties_even_f64(double v) { return round_ties_even_f64(v); }
float oxo_round_ties_even_f32(float v) { return round_ties_even_f32_native(v); }
float oxo_requantize(int64_t acc, float combined, int32_t zero_point, int64_t lo, int64_t hi) {
  return requantize(acc, combined, zero_point, SatRange{lo, hi});
}

}  // extern "C"
