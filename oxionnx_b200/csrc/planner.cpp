// Planning: from a topologically sorted node list to device steps.
//
// For every node the planner resolves shapes and device storage types (the reference has no
// shape rules for the INT8 family, so they are supplied here), validates the node the way the
// reference's CPU operator does (a malformed node DECLINES so the CPU operator can raise its own
// typed error), packs and uploads weights once per context, chooses the tensor-core or the
// direct kernel, fuses what the provider may fuse on its own (a Relu behind a quantised
// contraction or an Add, the DequantizeLinear -> Add -> Relu -> QuantizeLinear residual chain)
// and finally lays every intermediate out in one device arena by lifetime
// (MemoryPlan::compute, root crate src/memory/types.rs:347-452, in bytes instead of elements).
#include <algorithm>
#include <cmath>
#include <cstring>
#include <deque>
#include <functional>
#include <limits>
#include <memory>

#include "runtime.hpp"

namespace oxb {

namespace {

using k::Dims4;
using k::TensorRef;

const char* kSupportedOps[] = {"Conv",       "Gemm",     "MatMul",  "QLinearConv", "QLinearMatMul", "MatMulInteger",     "ConvInteger",
                               "QuantizeLinear", "DequantizeLinear", "DynamicQuantizeLinear", "Relu", "Tanh", "Sigmoid",    "PRelu",
                               "Add",        "Sub",      "Mul",     "Div",         "MaxPool",       "GlobalAveragePool", "OxiInstanceNorm",
                               "Resize",     "Pad",      "Concat",  "Flatten",     "Reshape",       "Identity",          "Cast",
                               "Slice",      "Gather",   "Transpose", "Softmax",   "LayerNormalization", "LayerNorm",    "Gelu",
                               "Erf",        "ConvAddRelu", "Silu",  "SiLU"};

// ---- scalar helpers that must agree with the reference bit for bit -----------------------
double round_ties_even(double v) { return std::nearbyint(v); }  // default rounding mode: ties to even

// lane_to_i32 (quant_ops/mod.rs:79-92): non-finite or out-of-range lanes are malformed.
bool lane_to_i32(float v, int32_t* out) {
  if (!std::isfinite(v)) return false;
  double r = round_ties_even((double)v);
  if (r < -2147483648.0 || r > 2147483647.0) return false;
  *out = (int32_t)r;
  return true;
}

bool lanes_to_i32(const HostTensor& t, std::vector<int32_t>* out) {
  out->resize(t.data.size());
  for (size_t i = 0; i < t.data.size(); ++i)
    if (!lane_to_i32(t.data[i], &(*out)[i])) return false;
  return true;
}

struct Range {
  int lo, hi;
};
// SatRange::infer (quant_ops/mod.rs:190-200)
Range sat_infer(const std::vector<int32_t>& y_zp, const std::vector<int32_t>& x_zp) {
  const std::vector<int32_t>* l[2] = {&y_zp, &x_zp};
  for (auto* lanes : l) {
    for (int32_t v : *lanes)
      if (v > 127) return {0, 255};
    for (int32_t v : *lanes)
      if (v < 0) return {-128, 127};
  }
  return {-128, 255};
}

// SatRange::for_dtype (quant_ops/mod.rs:216-222) where the zero point kept its declared type, else SatRange::infer.
Range sat_range(const HostTensor* y_zp_tensor, const std::vector<int32_t>& y_zp, const std::vector<int32_t>& x_zp) {
  if (y_zp_tensor && y_zp_tensor->declared == DT::U8) return {0, 255};
  if (y_zp_tensor && y_zp_tensor->declared == DT::I8) return {-128, 127};
  return sat_infer(y_zp, x_zp);
}

DT narrowest_int(int64_t lo, int64_t hi) {
  if (lo >= 0 && hi <= 255) return DT::U8;
  if (lo >= -128 && hi <= 127) return DT::I8;
  if (lo >= -32768 && hi <= 32767) return DT::I16;
  return DT::I32;
}

// f32 -> IEEE binary16 bits, round to nearest even (overflow to infinity, subnormals kept, NaN quiet).
uint16_t f32_to_f16_bits(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  const uint32_t mag = x & 0x7fffffffu;
  if (mag >= 0x7f800000u) return (uint16_t)(sign | (mag > 0x7f800000u ? 0x7e00u : 0x7c00u));
  if (mag >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);  // rounds to 65520 or above: infinity
  if (mag < 0x33000001u) return (uint16_t)sign;              // below half of the smallest subnormal
  const int e = (int)(mag >> 23) - 127;
  uint32_t man = (mag & 0x7fffffu) | 0x800000u;
  uint32_t shift, base;
  if (e < -14) {  // subnormal half: value = man * 2^(e-23), unit 2^-24
    shift = (uint32_t)(-e - 1);  // 13 + (-14 - e)
    base = 0;
  } else {
    shift = 13;
    base = ((uint32_t)(e + 15) << 10) - 0x400u;  // the implicit bit of man adds the last exponent step
  }
  const uint32_t q = man >> shift, rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
  uint32_t r = base + q;
  if (rem > half || (rem == half && (q & 1u))) r += 1;
  return (uint16_t)(sign | r);
}
// f32 -> bfloat16 bits, round to nearest even.
uint16_t f32_to_bf16_bits(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((x >> 16) | 0x40u);
  x += 0x7fffu + ((x >> 16) & 1u);
  return (uint16_t)(x >> 16);
}

float round_to_tf32(float v) {
  if (!std::isfinite(v)) return v;
  uint32_t u;
  std::memcpy(&u, &v, 4);
  u += 0x1000u;  // round to nearest, ties away from zero in magnitude (cvt.rna)
  u &= 0xffffe000u;
  float r;
  std::memcpy(&r, &u, 4);
  return r;
}

// ---- convolution geometry (oxionnx-ops src/conv/spatial.rs) --------------------------------
struct Geo {
  std::vector<int64_t> strides, pads, dilations, out_spatial;
  int64_t group = 1;
};

int64_t out_dim(const char* op, int64_t in, int64_t pb, int64_t pe, int64_t kernel, int64_t dil, int64_t stride, bool ceil_mode) {
  int64_t eff = (kernel - 1) * dil + 1;
  int64_t padded = in + pb + pe;
  if (padded < eff) OXB_DECLINE("%s: padded input extent %lld is smaller than the dilated kernel extent %lld", op, (long long)padded, (long long)eff);
  int64_t span = padded - eff;
  int64_t out = ceil_mode ? ceil_div(span, stride) + 1 : span / stride + 1;
  if (ceil_mode && out > 1 && (out - 1) * stride >= in + pb) out -= 1;
  return out;
}

Geo resolve_geometry(const char* op, const AttrMap& at, const int64_t* in_sp, const int64_t* kernel, int rank, bool ceil_mode) {
  Geo g;
  auto st = at.int_list("strides"), dl = at.int_list("dilations"), pd = at.int_list("pads");
  g.strides.assign(rank, 1);
  g.dilations.assign(rank, 1);
  for (int a = 0; a < rank; ++a) {
    if ((size_t)a < st.size()) {
      if (st[a] < 1) OXB_DECLINE("%s: strides[%d] must be >= 1", op, a);
      g.strides[a] = st[a];
    }
    if ((size_t)a < dl.size()) {
      if (dl[a] < 1) OXB_DECLINE("%s: dilations[%d] must be >= 1", op, a);
      g.dilations[a] = dl[a];
    }
  }
  std::vector<int64_t> expl(2 * rank, 0);
  for (int i = 0; i < 2 * rank; ++i)
    if ((size_t)i < pd.size()) {
      if (pd[i] < 0) OXB_DECLINE("%s: pads[%d] must be >= 0", op, i);
      expl[i] = pd[i];
    }
  std::string ap = at.s("auto_pad");
  if (ap.empty() || ap == "NOTSET") {
    g.pads = expl;
  } else if (ap == "VALID") {
    g.pads.assign(2 * rank, 0);
  } else if (ap == "SAME_UPPER" || ap == "SAME_LOWER") {
    bool lower = ap == "SAME_LOWER";
    g.pads.assign(2 * rank, 0);
    for (int a = 0; a < rank; ++a) {
      int64_t od = ceil_div(in_sp[a], g.strides[a]);
      int64_t eff = (kernel[a] - 1) * g.dilations[a] + 1;
      int64_t needed = std::max<int64_t>((od - 1) * g.strides[a] + eff - in_sp[a], 0);
      int64_t half = needed / 2;
      g.pads[a] = lower ? needed - half : half;
      g.pads[a + rank] = lower ? half : needed - half;
    }
  } else {
    OXB_DECLINE("%s: unknown auto_pad value '%s'", op, ap.c_str());
  }
  for (int a = 0; a < rank; ++a)
    g.out_spatial.push_back(out_dim(op, in_sp[a], g.pads[a], g.pads[a + rank], kernel[a], g.dilations[a], g.strides[a], ceil_mode));
  return g;
}

}  // namespace

bool is_supported_op(const std::string& op) {
  for (const char* s : kSupportedOps)
    if (op == s) return true;
  return false;
}

// Which operand slots may bind a device-resident activation in place (the data operands);
// parameter slots (scales, zero points, weights, shape vectors) must come from the host.
bool accepts_resident_slot(const std::string& op, uint32_t slot) {
  if (!is_supported_op(op)) return false;
  if (op == "QLinearConv") return slot == 0;
  if (op == "QLinearMatMul") return slot == 0;
  if (op == "MatMulInteger") return slot == 0 || slot == 2;  // A and the dynamic a_zero_point
  if (op == "ConvInteger" || op == "Conv") return slot == 0;
  if (op == "ConvAddRelu") return slot == 0 || slot == 3;  // the activation and the residual
  if (op == "Gemm") return slot == 0;
  if (op == "MatMul" || op == "Add" || op == "Sub" || op == "Mul" || op == "Div") return slot <= 1;
  if (op == "Concat") return true;
  if (op == "QuantizeLinear" || op == "DequantizeLinear" || op == "PRelu" || op == "Reshape" || op == "Resize" || op == "Pad") return slot == 0;
  return slot == 0;
}

// =========================================================================================
class Planner {
 public:
  Planner(Session& s, Context& c, const std::vector<NodeDef>& nodes, const std::map<std::string, const HostTensor*>& vconsts)
      : S(s), C(c), nodes_(nodes), vconsts_(vconsts) {}

  void run(const std::vector<std::pair<std::string, std::vector<int64_t>>>& inputs, const std::vector<std::string>& outputs);

 private:
  Session& S;
  Context& C;
  const std::vector<NodeDef> nodes_;  // copies: the step closures outlive the caller's arguments
  const std::map<std::string, const HostTensor*> vconsts_;
  std::unordered_map<std::string, std::vector<std::pair<int, int>>> consumers_;
  std::vector<char> skipped_;
  std::set<std::string> graph_outputs_;
  std::map<std::pair<int, int>, int> layout_memo_;
  std::set<std::string> tf32_rounded_names_;
  int cur_node_ = -1;

  // ---- value bookkeeping ----
  int add_value(const std::string& name, const std::vector<int64_t>& shape, DT dt, Layout layout) {
    auto it = S.index_.find(name);
    if (it != S.index_.end()) OXB_FAIL("value '%s' is produced twice", name.c_str());
    Value v;
    v.name = name;
    v.shape = shape;
    v.dt = dt;
    v.layout = layout;
    v.bytes = (size_t)std::max<int64_t>(prod(shape), 0) * dt_size(dt);
    S.values_.push_back(v);
    int idx = (int)S.values_.size() - 1;
    S.index_[name] = idx;
    return idx;
  }
  Value& V(int i) { return S.values_[i]; }

  const HostTensor* const_of(const std::string& name) const {
    if (name.empty()) return nullptr;
    auto it = vconsts_.find(name);
    if (it != vconsts_.end()) return it->second;
    return C.weight(name);
  }
  bool cacheable_const(const std::string& name) const { return vconsts_.find(name) == vconsts_.end(); }

  // Value index of a node input; initializers that are consumed as data get a device value on demand.
  int value_of(const std::string& name) {
    auto it = S.index_.find(name);
    if (it != S.index_.end()) return it->second;
    const HostTensor* h = const_of(name);
    if (!h) OXB_FAIL("value '%s' is neither produced by a node, fed, nor an initializer", name.c_str());
    // constant consumed as a data operand: upload as f32 lanes in logical order
    int idx = add_value(name, h->shape, DT::F32, Layout::PLAIN);
    V(idx).host = h;
    V(idx).external = true;
    size_t bytes = std::max<size_t>(h->data.size() * 4, 4);
    V(idx).ptr = C.resident_form(name, "raw_f32", bytes, [h](void* dst) { std::memcpy(dst, h->data.data(), h->data.size() * 4); },
                                 cacheable_const(name));
    return idx;
  }

  const std::string& in_name(const NodeDef& n, size_t i) const {
    static const std::string empty;
    return i < n.inputs.size() ? n.inputs[i] : empty;
  }
  const HostTensor* const_in(const NodeDef& n, size_t i) const { return const_of(in_name(n, i)); }
  bool has_in(const NodeDef& n, size_t i) const { return i < n.inputs.size() && !n.inputs[i].empty(); }

  void check_attrs(const NodeDef& n, std::initializer_list<const char*> known) {
    for (const std::string& a : n.attrs.names()) {
      bool ok = false;
      for (const char* kname : known)
        if (a == kname) ok = true;
      if (!ok) OXB_DECLINE("%s '%s': attribute '%s' is not handled by this provider", n.op.c_str(), n.name.c_str(), a.c_str());
    }
  }

  // ---- device parameter buffers owned by the session ----
  template <typename T>
  T* upload_vec(const std::vector<T>& v) {
    size_t bytes = std::max<size_t>(v.size() * sizeof(T), 16);
    void* p = C.alloc_device(bytes);
    S.owned_.push_back(DeviceBuffer{p, bytes});
    if (!v.empty()) OXB_CUDA(cudaMemcpyAsync(p, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice, C.stream()));
    OXB_CUDA(cudaStreamSynchronize(C.stream()));
    return (T*)p;
  }
  void* owned_buffer(size_t bytes) {
    void* p = C.alloc_device(bytes);
    S.owned_.push_back(DeviceBuffer{p, std::max<size_t>(bytes, 256)});
    return p;
  }

  // ---- steps ----
  Step& add_step(const NodeDef& n, const char* kernel, int family, std::vector<int> reads, std::vector<int> writes) {
    Step st;
    st.node_name = n.name;
    st.op_type = n.op;
    st.kernel = kernel;
    st.family = family;
    st.reads = std::move(reads);
    st.writes = std::move(writes);
    S.steps_.push_back(std::move(st));
    int idx = (int)S.steps_.size() - 1;
    // a value written by several steps (Concat) is born at the first of them
    for (int w : S.steps_[idx].writes)
      if (V(w).producer < 0) V(w).producer = idx;
    return S.steps_[idx];
  }

  static Dims4 dims_of(const Value& v) {
    if (v.shape.size() == 4) return Dims4{v.shape[0], v.shape[1], v.shape[2], v.shape[3]};
    if (v.shape.size() == 2) return Dims4{v.shape[0], v.shape[1], 1, 1};
    return Dims4{std::max<int64_t>(prod(v.shape), 0), 1, 1, 1};
  }
  static bool order_free(const Value& v) {  // PLAIN and NHWC coincide
    if (v.shape.size() != 4) return true;
    return v.shape[1] == 1 || v.shape[2] * v.shape[3] == 1;
  }
  Layout effective_layout(const Value& v) const { return v.shape.size() == 4 ? v.layout : Layout::PLAIN; }

  TensorRef ref_of(int vi, const Dims4* override_dims = nullptr) {
    Value& v = V(vi);
    return TensorRef{nullptr, v.dt, effective_layout(v), override_dims ? *override_dims : dims_of(v)};
  }
  // Resolve pointers at launch time (after the arena is laid out).
  TensorRef bound(const TensorRef& proto, int vi) {
    TensorRef r = proto;
    r.ptr = V(vi).ptr;
    return r;
  }

  // A copy of value `vi` in memory order `want` (memoised; rank-4 only).
  int ensure_layout(const NodeDef& n, int vi, Layout want) {
    if (V(vi).shape.size() != 4 || V(vi).layout == want) return vi;
    if (order_free(V(vi))) return vi;  // same bytes either way: kernels take the layout they need
    auto key = std::make_pair(vi, (int)want);
    auto it = layout_memo_.find(key);
    if (it != layout_memo_.end()) return it->second;
    Value src = V(vi);
    int out = add_value(src.name + (want == Layout::NHWC ? "@nhwc" : "@nchw"), src.shape, src.dt, want);
    TensorRef a = ref_of(vi), b = ref_of(out);
    Step& st = add_step(n, "convert_layout", 2, {vi}, {out});
    st.work = 2.0 * (double)src.bytes;
    st.launch = [this, a, b, vi, out](cudaStream_t s) {
      k::convert(bound(a, vi), bound(b, out), s);
      C.counters.glue_launches++;
      C.counters.kernel_launches++;
    };
    layout_memo_[key] = out;
    return out;
  }
  // The 16-bit float copy of an f32 value in the same memory order: the A operand of a kind::f16 contraction
  // (context option float_precision).  One copy per value, shared by its consumers.
  int half_copy(const NodeDef& n, int vi, DT dt16) {
    auto key = std::make_pair(vi, 100 + (int)dt16);
    auto it = layout_memo_.find(key);
    if (it != layout_memo_.end()) return it->second;
    Value src = V(vi);
    int out = add_value(src.name + (dt16 == DT::F16 ? "@f16" : "@bf16"), src.shape, dt16, src.layout);
    V(out).bytes = src.bytes / 2;  // padded layouts (the stem's row windows) keep their padding
    const int64_t lanes = (int64_t)(src.bytes / 4);
    Step& st = add_step(n, dt16 == DT::F16 ? "convert_f32_to_f16" : "convert_f32_to_bf16", 2, {vi}, {out});
    st.work = 1.5 * (double)src.bytes;
    st.launch = [this, vi, out, dt16, lanes](cudaStream_t s) {
      k::convert_f32_to_half((const float*)V(vi).ptr, V(out).ptr, dt16, lanes, s);
      C.counters.glue_launches++;
      C.counters.kernel_launches++;
    };
    layout_memo_[key] = out;
    return out;
  }
  // For order-free rank-4 values any kernel may treat the bytes as NHWC.
  Layout layout_for_kernel(const Value& v, Layout want) const { return (v.shape.size() == 4 && order_free(v)) ? want : effective_layout(v); }

  // Sole consumer of `name` if it is op `op` at slot 0 and the value is not a graph output.
  int sole_consumer(const std::string& name, const char* op) {
    if (graph_outputs_.count(name)) return -1;
    auto it = consumers_.find(name);
    if (it == consumers_.end() || it->second.size() != 1) return -1;
    int ni = it->second[0].first;
    if (it->second[0].second != 0 || nodes_[ni].op != op || skipped_[ni]) return -1;
    if (!nodes_[ni].attrs.names().empty()) return -1;
    return ni;
  }

  // Every producer decides whether to round its output to TF32 by asking this about its output's name; a "yes"
  // is remembered, so that a contraction can tell whether its operand arrives rounded (tf32_ready).
  bool feeds_contraction(const std::string& name) {
    const bool yes = feeds_contraction_impl(name);
    if (yes) tf32_rounded_names_.insert(name);
    return yes;
  }
  // Does the value hold TF32-rounded lanes?  Either its producer rounded it, or it was moved / selected (layout
  // conversion, pooling by maximum, padding, slicing, concatenation, transposition, the stem's packing) out of
  // values that were.  A graph input never is: the tensor pipe would truncate its low mantissa bits instead of
  // rounding them, which doubles the operand error and biases it.
  bool tf32_ready(int vi, int depth = 0) {
    while (V(vi).alias_of >= 0) vi = V(vi).alias_of;
    if (tf32_rounded_names_.count(V(vi).name)) return true;
    if (V(vi).is_graph_input || V(vi).producer < 0 || depth > 12) return false;
    const Step& ps = S.steps_[V(vi).producer];
    static const char* movers[] = {"convert_layout", "max_pool", "pad", "slice", "concat", "transpose_perm", "transpose_a", "s2d_pack", "window_pack",
                                   "resize_nearest"};
    bool mover = false;
    for (const char* m : movers) mover = mover || ps.kernel.rfind(m, 0) == 0;
    if (!mover || ps.reads.empty()) return false;
    for (int r : ps.reads)
      if (V(r).dt == DT::F32 && !tf32_ready(r, depth + 1)) return false;
    return true;
  }
  // A TF32-rounded copy of an f32 value in the same memory order (round to nearest, ties away: cvt.rna), made once
  // per value for the contractions that read it.
  int tf32_copy(const NodeDef& n, int vi) {
    auto key = std::make_pair(vi, 200);
    auto it = layout_memo_.find(key);
    if (it != layout_memo_.end()) return it->second;
    Value src = V(vi);
    int out = add_value(src.name + "@tf32", src.shape, DT::F32, src.layout);
    V(out).bytes = src.bytes;
    const int64_t lanes = (int64_t)(src.bytes / 4);
    Step& st = add_step(n, "round_to_tf32", 2, {vi}, {out});
    st.work = 2.0 * (double)src.bytes;
    st.launch = [this, vi, out, lanes](cudaStream_t s) {
      k::round_to_tf32_copy((const float*)V(vi).ptr, (float*)V(out).ptr, lanes, s);
      C.counters.glue_launches++;
      C.counters.kernel_launches++;
    };
    layout_memo_[key] = out;
    return out;
  }
  bool feeds_contraction_impl(const std::string& name) {
    auto it = consumers_.find(name);
    if (it == consumers_.end()) return false;
    for (auto& c : it->second) {
      const std::string& op = nodes_[c.first].op;
      if (op == "Conv" || op == "Gemm" || op == "MatMul") return true;
      // look through nodes that only move or select values
      if (op == "MaxPool" || op == "Flatten" || op == "Reshape" || op == "Identity" || op == "Relu" || op == "Pad" || op == "Resize" ||
          op == "Concat" || op == "Transpose")
        if (!nodes_[c.first].outputs.empty() && feeds_contraction_impl(nodes_[c.first].outputs[0])) return true;
    }
    return false;
  }

  // ---- operator rules ----
  void plan_node(int ni);
  void plan_quantize(const NodeDef& n);
  void plan_dequantize(const NodeDef& n);
  void plan_dynamic_quantize(const NodeDef& n);
  void plan_conv_family(const NodeDef& n, int ni);
  void plan_matmul_family(const NodeDef& n, int ni);
  void plan_unary(const NodeDef& n);
  void plan_binary(const NodeDef& n, int ni);
  void plan_prelu(const NodeDef& n);
  void plan_max_pool(const NodeDef& n);
  void plan_global_avg_pool(const NodeDef& n);
  void plan_instance_norm(const NodeDef& n);
  void plan_resize(const NodeDef& n);
  void plan_pad(const NodeDef& n);
  void plan_concat(const NodeDef& n);
  void plan_slice(const NodeDef& n);
  void plan_gather(const NodeDef& n);
  void plan_transpose(const NodeDef& n);
  void emit_transpose(const NodeDef& n, int xi, const std::vector<int64_t>& perm, int yi);
  // A head split Transpose(Reshape(x2d [B*S, H*D] -> [B,S,H,D])) whose only reader is a MatMul is not run when
  // planned: the tensor-core product reads the heads straight out of x2d through strided tensor maps.
  struct LazyHeads {
    int src_vi, root_vi;
    int64_t B, S, H, D;
    int kind;  // 0: [B,H,S,D] (perm 0,2,1,3), 1: [B,H,D,S] (perm 0,2,3,1)
    int node;
    std::vector<int64_t> perm;
    bool materialised;
  };
  std::map<int, LazyHeads> lazy_heads_;
  void materialise_heads(int yi);
  bool try_plan_attention_product(const NodeDef& n, int ai, int bi);
  void plan_softmax(const NodeDef& n);
  bool try_plan_scaled_masked_softmax(const NodeDef& n);
  bool try_plan_fused_attention(const NodeDef& n, int qi, int ki);
  void plan_layer_norm(const NodeDef& n);
  void plan_alias(const NodeDef& n);
  bool try_plan_residual_chain(const NodeDef& n, int ni);

  struct Contraction {
    k::ConvShape cs;
    int x_vi, out_vi;
    bool x_plain_nchw = false;
    // weights in ONNX order [OC][C/g][R][S] as exact values
    const HostTensor* w = nullptr;
    std::string w_name;
    bool w_is_kn = false;  // matmul B stored [K][N]
    bool is_int = false;
    DT w_dt = DT::F32;
    k::Epilogue epi;
    std::vector<int32_t> w_zp;   // per-oc or single
    bool x_zp_static = true;
    int x_zp = 0;
    int x_zp_vi = -1;            // device lane (dynamic)
    int res_vi = -1;             // f32 residual added in the epilogue (a fused Add), or -1
    int dq_xs_vi = -1;           // dequantising epilogue: the device lane holding the activation scale
    std::vector<float> dq_w_scale, dq_bias;  // ... and its per-channel weight scales and bias
    std::vector<int32_t> x_zp_rows;
    std::vector<int32_t> bias_i;  // empty or OC
    std::vector<float> bias_f;    // empty or OC
    std::vector<float> slope;     // PRelu epilogue: OC slopes
    std::vector<float> combined;  // OC
    float w_scale_mul = 1.0f;     // Gemm alpha folded into the packed weights
    double algorithmic_ops = 0;   // ops of the node as written (a rewritten stem pads its reduction)
    int w_cacheable = -1;         // whether the packed weights may stay resident (-1: decide from the name)
  };
  void emit_contraction(const NodeDef& n, Contraction& c);

  void finalize_lifetimes_and_arena();
  struct LastAdd {
    int step = -1, a = -1, b = -1, y = -1;
  };
  LastAdd last_add_;
  struct ChainLink {
    int step = -1, rows = 0, x_vi = -1, out_vi = -1;
    k::UmmaChainLayer layer;
  };
  std::vector<ChainLink> chain_links_;
  void link_chains();
  bool try_s2d_stem(const NodeDef& n, Contraction& c, int src_vi);
  bool try_window_stem(const NodeDef& n, Contraction& c, int src_vi);
  std::deque<HostTensor> made_consts_;  // weights rewritten by the planner (space-to-depth stems)
};

// -----------------------------------------------------------------------------------------
void Planner::run(const std::vector<std::pair<std::string, std::vector<int64_t>>>& inputs, const std::vector<std::string>& outputs) {
  for (auto& o : outputs) graph_outputs_.insert(o);
  S.outputs_ = outputs;
  skipped_.assign(nodes_.size(), 0);
  for (size_t ni = 0; ni < nodes_.size(); ++ni)
    for (size_t s = 0; s < nodes_[ni].inputs.size(); ++s)
      if (!nodes_[ni].inputs[s].empty()) consumers_[nodes_[ni].inputs[s]].push_back({(int)ni, (int)s});

  OXB_CUDA(cudaMalloc(&S.err_flag_, 256));
  OXB_CUDA(cudaMemset(S.err_flag_, 0, 256));

  // graph inputs: raw f32 lanes in logical order, uploaded into persistent staging
  for (auto& in : inputs) {
    // declared element type (TensorInfo): 8-bit inputs are stored, fed and bound as 8-bit lanes
    auto declared = S.input_types_.find(in.first);
    const DT in_dt = declared == S.input_types_.end() ? DT::F32 : declared->second;
    if (!(in_dt == DT::F32 || in_dt == DT::U8 || in_dt == DT::I8)) OXB_DECLINE("graph input '%s': declared element type %s is not one this provider takes at the boundary", in.first.c_str(), dt_name(in_dt));
    int vi = add_value(in.first, in.second, in_dt, Layout::PLAIN);
    V(vi).is_graph_input = true;
    V(vi).external = true;
    auto vc = vconsts_.find(in.first);
    if (vc != vconsts_.end()) V(vi).host = vc->second;
    auto eb = S.external_bind_.find(in.first);
    if (eb != S.external_bind_.end()) {
      V(vi).ptr = eb->second.first;
      V(vi).dt = eb->second.second.first;
      V(vi).layout = eb->second.second.second;
      V(vi).bytes = (size_t)V(vi).numel() * dt_size(V(vi).dt);
    } else {
      V(vi).ptr = owned_buffer(std::max<size_t>(V(vi).bytes, 256));
    }
    S.input_staging_.push_back({in.first, vi});
  }

  for (size_t ni = 0; ni < nodes_.size(); ++ni) {
    if (skipped_[ni]) continue;
    cur_node_ = (int)ni;
    plan_node((int)ni);
  }

  // graph outputs: f32 lanes in logical order in persistent staging
  NodeDef out_node;
  out_node.op = "(output)";
  for (auto& o : outputs) {
    auto it = S.index_.find(o);
    if (it == S.index_.end()) OXB_FAIL("graph output '%s' is not produced by any planned node", o.c_str());
    int vi = it->second;
    V(vi).is_graph_output = true;
    out_node.name = o;
    bool direct = V(vi).dt == DT::F32 && (effective_layout(V(vi)) == Layout::PLAIN || order_free(V(vi))) && V(vi).alias_of < 0 &&
                  !V(vi).is_graph_input && V(vi).host == nullptr;
    if (direct) {
      // give the value its own persistent storage instead of an arena slot
      V(vi).external = true;
      V(vi).ptr = owned_buffer(std::max<size_t>(V(vi).bytes, 256));
      S.output_staging_.push_back({o, vi});
      continue;
    }
    int so = add_value(o + "@host", V(vi).shape, DT::F32, Layout::PLAIN);
    V(so).external = true;
    V(so).ptr = owned_buffer(std::max<size_t>(V(so).bytes, 256));
    Dims4 d = V(vi).shape.size() == 4 ? dims_of(V(vi)) : Dims4{std::max<int64_t>(V(vi).numel(), 0), 1, 1, 1};
    TensorRef a{nullptr, V(vi).dt, effective_layout(V(vi)), d}, b{nullptr, DT::F32, Layout::PLAIN, d};
    Step& st = add_step(out_node, "convert_output", 2, {vi}, {so});
    st.work = (double)V(vi).bytes + (double)V(so).bytes;
    st.launch = [this, a, b, vi, so](cudaStream_t s) {
      k::convert(bound(a, vi), bound(b, so), s);
      C.counters.glue_launches++;
      C.counters.kernel_launches++;
    };
    S.output_staging_.push_back({o, so});
  }

  finalize_lifetimes_and_arena();
  for (auto& st : S.steps_)
    if (st.finalize) st.finalize();
  link_chains();
}

// Consecutive steps that are quantised linear layers over the same few rows, each reading what the one before
// wrote, run as one cooperative kernel launched by the first of them; the others keep their place in the plan
// (values, lifetimes, profile rows) and launch nothing.  Every intermediate row is still written to its own
// value, so other readers and kept intermediates see what the separate kernels would have produced.
void Planner::link_chains() {
  size_t i = 0;
  while (i < chain_links_.size()) {
    size_t j = i + 1;
    while (j < chain_links_.size() && j - i < 4 && chain_links_[j].step == chain_links_[j - 1].step + 1 && chain_links_[j].rows == chain_links_[i].rows &&
           chain_links_[j].layer.x == chain_links_[j - 1].layer.out && chain_links_[j].layer.K == chain_links_[j - 1].layer.N)
      ++j;
    if (j - i >= 2) {
      std::vector<k::UmmaChainLayer> layers;
      for (size_t t = i; t < j; ++t) layers.push_back(chain_links_[t].layer);
      // A per-tensor QuantizeLinear right in front of the chain whose only reader is the first layer is done by
      // that layer while it stages its activation blocks; a per-tensor DequantizeLinear right behind the chain is
      // written by the last layer beside its 8-bit rows.  Both steps then launch nothing.  The f32 rows must
      // outlive the quantising step, and the dequantised value must not share memory with what the last layer
      // still reads (earlier layers' values are dead by then: a grid barrier lies in between).
      k::UmmaChainEnds ends;
      int head_step = -1, tail_step = -1;
      const int first_step = chain_links_[i].step, last_step = chain_links_[j - 1].step;
      auto overlaps = [&](const Value& a, const Value& b) {
        const uint8_t *a0 = (const uint8_t*)a.ptr, *b0 = (const uint8_t*)b.ptr;
        return a0 < b0 + std::max<size_t>(b.bytes, 1) && b0 < a0 + std::max<size_t>(a.bytes, 1);
      };
      if (!C.cfg().keep_intermediates) {
        const Value& xv = V(chain_links_[i].x_vi);
        if (xv.q_src >= 0 && xv.q_step == first_step - 1 && !graph_outputs_.count(xv.name)) {
          auto it = consumers_.find(xv.name);
          int root = xv.q_src;
          while (V(root).alias_of >= 0) root = V(root).alias_of;
          const Value& sv = V(xv.q_src);
          const bool lives = V(root).external || V(root).is_graph_output || V(root).last_use >= first_step;
          if (it != consumers_.end() && it->second.size() == 1 && lives && sv.dt == DT::F32 && (sv.shape.size() != 4 || order_free(sv)) &&
              sv.numel() == (int64_t)chain_links_[i].rows * chain_links_[i].layer.K && ((uintptr_t)sv.ptr & 15) == 0) {
            ends.head_x = (const float*)sv.ptr;
            ends.head_scale = xv.q_scale, ends.head_zp = xv.q_zp, ends.head_lo = xv.q_lo, ends.head_hi = xv.q_hi;
            head_step = xv.q_step;
          }
        }
        const int last_out = chain_links_[j - 1].out_vi;
        for (int vi = 0; vi < (int)S.values_.size() && tail_step < 0; ++vi) {
          const Value& dv = V(vi);
          if (dv.dq_src != last_out || dv.dq_step != last_step + 1 || dv.alias_of >= 0 || dv.dt != DT::F32) continue;
          if ((dv.shape.size() == 4 && !order_free(dv)) || overlaps(dv, V(chain_links_[j - 1].x_vi)) || overlaps(dv, V(last_out))) continue;
          ends.tail_out = (float*)dv.ptr;
          ends.tail_scale = dv.dq_scale, ends.tail_zp = dv.dq_zp;
          ends.tail_signed = V(last_out).dt == DT::I8 ? 1 : 0;
          tail_step = dv.dq_step;
        }
      }
      std::string why;
      k::UmmaChain* chain = k::umma_chain_create(layers.data(), (int)layers.size(), chain_links_[i].rows, ends, &why);
      if (chain) {
        S.umma_chains_.push_back(chain);
        Step& first = S.steps_[chain_links_[i].step];
        first.kernel = k::umma_chain_desc(chain);
        int* err = S.err_flag_;
        // the layers' own launches stay behind the chain: a cooperative launch the driver refuses (the grid cannot
        // be co-resident right now, e.g. under a profiler) turns the chain off for this session
        auto own = std::make_shared<std::vector<std::function<void(cudaStream_t)>>>();
        if (head_step >= 0) own->push_back(S.steps_[head_step].launch);
        for (size_t t = i; t < j; ++t) own->push_back(S.steps_[chain_links_[t].step].launch);
        if (tail_step >= 0) own->push_back(S.steps_[tail_step].launch);
        for (int extra : {head_step, tail_step})
          if (extra >= 0) {
            S.steps_[extra].kernel = "umma_i8_chain (inside the launch of '" + first.node_name + "')";
            S.steps_[extra].launch = [](cudaStream_t) {};
          }
        auto off = std::make_shared<bool>(false);
        const int head_vi = ends.head_x ? V(chain_links_[i].x_vi).q_src : -1;
        first.launch = [this, chain, err, own, off, head_vi](cudaStream_t s) {
          // a cooperative kernel node makes a replayed CUDA graph several times slower than the separate kernels
          // (measured: 232 us against 61 us per pass of the 64-row MLP), so a capture records the layers' own launches
          cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
          if (cudaStreamIsCapturing(s, &capturing) != cudaSuccess) (void)cudaGetLastError();
          if (!*off && capturing == cudaStreamCaptureStatusNone) {
            if (k::umma_chain_launch(chain, err, head_vi >= 0 ? (const float*)V(head_vi).ptr : nullptr, s)) {
              C.counters.umma_launches++;
              C.counters.kernel_launches++;
              return;
            }
            *off = true;
          }
          for (auto& f : *own) f(s);
        };
        for (size_t t = i + 1; t < j; ++t) {
          Step& st = S.steps_[chain_links_[t].step];
          st.kernel = "umma_i8_chain (inside the launch of '" + first.node_name + "')";
          st.launch = [](cudaStream_t) {};
        }
      }
    }
    i = j;
  }
}

void Planner::finalize_lifetimes_and_arena() {
  const int n_steps = (int)S.steps_.size();
  for (int si = 0; si < n_steps; ++si)
  {
    Step& st = S.steps_[si];
    st.bytes = st.param_bytes;
    for (int r : st.reads) {
      V(r).last_use = std::max(V(r).last_use, si);
      st.bytes += (double)V(r).bytes;
    }
    for (int w : st.writes) {
      V(w).last_use = std::max(V(w).last_use, si);
      st.bytes += (double)V(w).bytes;
    }
  }
  // aliases extend the life of the storage they share
  for (int i = (int)S.values_.size() - 1; i >= 0; --i) {
    Value& v = V(i);
    if (v.alias_of >= 0) {
      Value& root = V(v.alias_of);
      root.last_use = std::max(root.last_use, std::max(v.last_use, v.is_graph_output ? n_steps : -1));
      if (v.is_graph_output) root.is_graph_output = true;
    }
  }
  // The dequantised copy of a few 8-bit rows may be written by the kernel that produces those rows, and that kernel
  // may be launched up to three steps earlier (a chain of quantised linear layers, link_chains): its storage is
  // reserved from there on, so that it never shares memory with what the chain still reads.
  for (Value& v : S.values_) {
    if (v.dq_src < 0 || v.dq_step < 0 || v.producer < 0) continue;
    const Value& src = V(v.dq_src);
    if (src.producer < 0 || src.shape.size() != 4 || src.shape[0] * src.shape[2] * src.shape[3] > 64) continue;
    v.producer = std::max(0, std::min(v.producer, src.producer - 3));
  }
  struct Slot {
    size_t bytes;
    int free_after;
  };
  std::vector<Slot> slots;
  std::vector<int> order;
  for (int i = 0; i < (int)S.values_.size(); ++i) {
    Value& v = V(i);
    if (v.external || v.alias_of >= 0 || v.producer < 0) continue;
    order.push_back(i);
  }
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return V(a).producer < V(b).producer; });
  const bool keep_all = C.cfg().keep_intermediates != 0;
  for (int i : order) {
    Value& v = V(i);
    int last = v.is_graph_output ? n_steps : std::max(v.last_use, v.producer);
    size_t need = align_up(std::max<size_t>(v.bytes, 1), 1024);
    int best = -1;
    if (!keep_all) {
      // smallest free slot that already fits, else the smallest free slot (grown)
      for (int s = 0; s < (int)slots.size(); ++s)
        if (slots[s].free_after < v.producer && slots[s].bytes >= need && (best < 0 || slots[s].bytes < slots[best].bytes)) best = s;
      if (best < 0)
        for (int s = 0; s < (int)slots.size(); ++s)
          if (slots[s].free_after < v.producer && (best < 0 || slots[s].bytes < slots[best].bytes)) best = s;
    }
    if (best < 0) {
      slots.push_back(Slot{need, last});
      best = (int)slots.size() - 1;
    } else {
      slots[best].bytes = std::max(slots[best].bytes, need);
      slots[best].free_after = last;
    }
    v.slot = best;
  }
  size_t total = 0;
  std::vector<size_t> offs(slots.size());
  for (size_t s = 0; s < slots.size(); ++s) {
    offs[s] = total;
    total += slots[s].bytes;
  }
  S.n_slots_ = slots.size();
  S.arena_.bytes = total;
  if (total > 0) {
    OXB_CUDA(cudaMalloc(&S.arena_.ptr, total));
  }
  for (int i : order) V(i).ptr = (uint8_t*)S.arena_.ptr + offs[V(i).slot];
  for (int i = 0; i < (int)S.values_.size(); ++i)
    if (V(i).alias_of >= 0) {
      int r = V(i).alias_of;
      while (V(r).alias_of >= 0) r = V(r).alias_of;
      V(i).ptr = V(r).ptr;
    }
  C.counters.arena_bytes = total;
  C.counters.arena_peak_bytes = std::max<uint64_t>(C.counters.arena_peak_bytes, total);
  C.counters.arena_slots = slots.size();
}

// -----------------------------------------------------------------------------------------
void Planner::plan_node(int ni) {
  const NodeDef& n = nodes_[ni];
  const std::string& op = n.op;
  if (!is_supported_op(op)) OXB_DECLINE("operator '%s' (node '%s') is not claimed by this provider", op.c_str(), n.name.c_str());
  if (op == "Slice") return plan_slice(n);
  if (op == "Gather") return plan_gather(n);
  if (op == "Transpose") return plan_transpose(n);
  if (op == "Softmax") return plan_softmax(n);
  if (op == "LayerNormalization" || op == "LayerNorm") return plan_layer_norm(n);
  if (op == "Gelu" || op == "Erf") return plan_unary(n);
  if (op == "QuantizeLinear") return plan_quantize(n);
  if (op == "DequantizeLinear") {
    if (try_plan_residual_chain(n, ni)) return;
    return plan_dequantize(n);
  }
  if (op == "DynamicQuantizeLinear") return plan_dynamic_quantize(n);
  if (op == "Conv" || op == "QLinearConv" || op == "ConvInteger" || op == "ConvAddRelu") return plan_conv_family(n, ni);
  if (op == "Gemm" || op == "MatMul" || op == "QLinearMatMul" || op == "MatMulInteger") return plan_matmul_family(n, ni);
  if (op == "Relu" || op == "Tanh" || op == "Sigmoid" || op == "Silu" || op == "SiLU") return plan_unary(n);
  if (op == "Add" || op == "Sub" || op == "Mul" || op == "Div") return plan_binary(n, ni);
  if (op == "PRelu") return plan_prelu(n);
  if (op == "MaxPool") return plan_max_pool(n);
  if (op == "GlobalAveragePool") return plan_global_avg_pool(n);
  if (op == "OxiInstanceNorm") return plan_instance_norm(n);
  if (op == "Resize") return plan_resize(n);
  if (op == "Pad") return plan_pad(n);
  if (op == "Concat") return plan_concat(n);
  if (op == "Flatten" || op == "Reshape" || op == "Identity" || op == "Cast") return plan_alias(n);
  OXB_DECLINE("operator '%s' has no planning rule", op.c_str());
}

// ---- QuantizeLinear / DequantizeLinear (oxionnx-ops src/indexing/quantize.rs:58-193) -------
static void quant_axis_view(const Value& x, int64_t axis_raw, int64_t plen, const char* op, Dims4* d, bool* use_native4) {
  int64_t rank = (int64_t)x.shape.size();
  *use_native4 = false;
  if (plen <= 1) {
    if (rank == 4) {
      *d = Dims4{x.shape[0], x.shape[1], x.shape[2], x.shape[3]};
      *use_native4 = true;
    } else {
      *d = Dims4{std::max<int64_t>(prod(x.shape), 0), 1, 1, 1};
    }
    return;
  }
  int64_t axis = axis_raw < 0 ? axis_raw + rank : axis_raw;
  if (axis < 0 || axis >= rank) OXB_DECLINE("%s: axis %lld out of range for rank %lld", op, (long long)axis_raw, (long long)rank);
  if (x.shape[axis] != plen) OXB_DECLINE("%s: %lld quantisation parameters for an axis of extent %lld", op, (long long)plen, (long long)x.shape[axis]);
  if (rank == 4 && axis == 1) {
    *d = Dims4{x.shape[0], x.shape[1], x.shape[2], x.shape[3]};
    *use_native4 = true;
    return;
  }
  if (rank == 4 && x.layout == Layout::NHWC && !(x.shape[1] == 1 || x.shape[2] * x.shape[3] == 1))
    OXB_DECLINE("%s: per-axis parameters on axis %lld of a channels-last activation", op, (long long)axis);
  int64_t outer = 1, inner = 1;
  for (int64_t i = 0; i < axis; ++i) outer *= x.shape[i];
  for (int64_t i = axis + 1; i < rank; ++i) inner *= x.shape[i];
  *d = Dims4{outer, x.shape[axis], inner, 1};
}

void Planner::plan_quantize(const NodeDef& n) {
  check_attrs(n, {"axis"});
  if (n.attrs.has("saturate") || n.attrs.has("block_size")) OXB_DECLINE("QuantizeLinear: blocked / non-saturating forms");
  const HostTensor* scale = const_in(n, 1);
  const HostTensor* zp = has_in(n, 2) ? const_in(n, 2) : nullptr;
  if (!scale || (has_in(n, 2) && !zp)) OXB_DECLINE("QuantizeLinear '%s': scale / zero point are not initializers", n.name.c_str());
  if (scale->data.empty()) OXB_DECLINE("quantize_linear: y_scale must have at least one element");
  if (zp && zp->data.empty()) OXB_DECLINE("quantize_linear: y_zero_point must have at least one element when provided");
  int xi = value_of(in_name(n, 0));
  if (V(xi).dt != DT::F32) OXB_DECLINE("QuantizeLinear '%s': input is not a float tensor", n.name.c_str());
  // saturation_range (quantize.rs:58-64): absent -> u8; any lane > 127 -> u8; otherwise i8
  float lo = 0.f, hi = 255.f;
  if (zp) {
    bool any_gt = false;
    for (float z : zp->data) any_gt |= z > 127.0f;
    if (!any_gt) {
      lo = -128.f;
      hi = 127.f;
    }
    for (float z : zp->data)
      if (!std::isfinite(z) || z != std::nearbyint(z)) OXB_DECLINE("QuantizeLinear '%s': non-integral zero point", n.name.c_str());
  }
  for (float sc : scale->data)
    if (!std::isfinite(sc) || sc == 0.f) OXB_DECLINE("QuantizeLinear '%s': zero or non-finite scale", n.name.c_str());
  int64_t ns = (int64_t)scale->data.size(), nz = zp ? (int64_t)zp->data.size() : 0;
  int64_t plen = std::max(ns, nz);
  Dims4 d;
  bool native4;
  quant_axis_view(V(xi), n.attrs.i("axis", 1), plen, "QuantizeLinear", &d, &native4);
  if ((ns > 1 && ns != d.C) || (nz > 1 && nz != d.C)) OXB_DECLINE("QuantizeLinear '%s': parameter length disagrees with the axis", n.name.c_str());
  DT odt = lo < 0 ? DT::I8 : DT::U8;
  Layout ol = V(xi).shape.size() == 4 ? Layout::NHWC : Layout::PLAIN;
  if (!native4 && V(xi).shape.size() == 4) ol = V(xi).layout;
  int yi = add_value(n.outputs[0], V(xi).shape, odt, ol);
  TensorRef xr{nullptr, DT::F32, native4 ? layout_for_kernel(V(xi), ol) : Layout::PLAIN, d};
  TensorRef yr{nullptr, odt, native4 ? ol : Layout::PLAIN, d};
  const float* dscale = (const float*)C.resident_form(in_name(n, 1), "raw_f32", scale->data.size() * 4,
                                                      [scale](void* p) { std::memcpy(p, scale->data.data(), scale->data.size() * 4); },
                                                      cacheable_const(in_name(n, 1)));
  const float* dzp = nullptr;
  if (zp)
    dzp = (const float*)C.resident_form(in_name(n, 2), "raw_f32", zp->data.size() * 4, [zp](void* p) { std::memcpy(p, zp->data.data(), zp->data.size() * 4); },
                                        cacheable_const(in_name(n, 2)));
  float s0 = scale->data[0], z0 = zp ? zp->data[0] : 0.f;
  bool scalar = ns == 1 && nz <= 1;
  Step& st = add_step(n, "quantize_linear", 2, {xi}, {yi});
  if (scalar) {
    Value& yv = V(yi);
    yv.q_src = xi;
    yv.q_step = (int)S.steps_.size() - 1;
    yv.q_scale = s0, yv.q_zp = z0, yv.q_lo = lo, yv.q_hi = hi;
  }
  st.work = (double)V(xi).bytes + (double)V(yi).bytes;
  st.launch = [this, xr, yr, xi, yi, dscale, ns, dzp, nz, lo, hi, scalar, s0, z0](cudaStream_t s) {
    TensorRef a = bound(xr, xi), b = bound(yr, yi);
    if (scalar && k::quantize_linear_scalar_ok(a, b)) k::quantize_linear_scalar(a, b, s0, z0, lo, hi, s);
    else k::quantize_linear(a, b, dscale, ns, dzp, nz, lo, hi, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

void Planner::plan_dequantize(const NodeDef& n) {
  check_attrs(n, {"axis"});
  const HostTensor* scale = const_in(n, 1);
  const HostTensor* zp = has_in(n, 2) ? const_in(n, 2) : nullptr;
  if (!scale || (has_in(n, 2) && !zp)) OXB_DECLINE("DequantizeLinear '%s': scale / zero point are not initializers", n.name.c_str());
  if (scale->data.empty()) OXB_DECLINE("dequantize_linear: x_scale must have at least one element");
  if (zp && zp->data.empty()) OXB_DECLINE("dequantize_linear: x_zero_point must have at least one element when provided");
  int xi = value_of(in_name(n, 0));
  int64_t ns = (int64_t)scale->data.size(), nz = zp ? (int64_t)zp->data.size() : 0;
  Dims4 d;
  bool native4;
  quant_axis_view(V(xi), n.attrs.i("axis", 1), std::max(ns, nz), "DequantizeLinear", &d, &native4);
  if ((ns > 1 && ns != d.C) || (nz > 1 && nz != d.C)) OXB_DECLINE("DequantizeLinear '%s': parameter length disagrees with the axis", n.name.c_str());
  Layout l = V(xi).shape.size() == 4 ? V(xi).layout : Layout::PLAIN;
  int yi = add_value(n.outputs[0], V(xi).shape, DT::F32, l);
  TensorRef xr{nullptr, V(xi).dt, native4 ? effective_layout(V(xi)) : Layout::PLAIN, d};
  TensorRef yr{nullptr, DT::F32, native4 ? l : Layout::PLAIN, d};
  const float* dscale = (const float*)C.resident_form(in_name(n, 1), "raw_f32", scale->data.size() * 4,
                                                      [scale](void* p) { std::memcpy(p, scale->data.data(), scale->data.size() * 4); },
                                                      cacheable_const(in_name(n, 1)));
  const float* dzp = nullptr;
  if (zp)
    dzp = (const float*)C.resident_form(in_name(n, 2), "raw_f32", zp->data.size() * 4, [zp](void* p) { std::memcpy(p, zp->data.data(), zp->data.size() * 4); },
                                        cacheable_const(in_name(n, 2)));
  Step& st = add_step(n, "dequantize_linear", 2, {xi}, {yi});
  if (ns == 1 && nz <= 1 && native4 && V(xi).shape.size() == 4 && (V(xi).dt == DT::U8 || V(xi).dt == DT::I8)) {
    Value& yv = V(yi);
    yv.dq_src = xi;
    yv.dq_step = (int)S.steps_.size() - 1;
    yv.dq_scale = scale->data[0];
    yv.dq_zp = zp ? zp->data[0] : 0.f;
  }
  st.work = (double)V(xi).bytes + (double)V(yi).bytes;
  st.launch = [this, xr, yr, xi, yi, dscale, ns, dzp, nz](cudaStream_t s) {
    k::dequantize_linear(bound(xr, xi), bound(yr, yi), dscale, ns, dzp, nz, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

// DynamicQuantizeLinear (quant_ops/dynamic_quantize.rs:51-93): y plus rank-0 scale and zero point,
// both kept as device f32 lanes so a following MatMulInteger reads them without a host trip.
void Planner::plan_dynamic_quantize(const NodeDef& n) {
  check_attrs(n, {});
  int xi = value_of(in_name(n, 0));
  if (V(xi).dt != DT::F32) OXB_DECLINE("DynamicQuantizeLinear '%s': input is not a float tensor", n.name.c_str());
  if (V(xi).numel() == 0) OXB_DECLINE("DynamicQuantizeLinear: input is empty");
  if (V(xi).host)
    for (float f : V(xi).host->data)
      if (!std::isfinite(f)) OXB_DECLINE("DynamicQuantizeLinear: input contains a non-finite value");
  int yi = add_value(n.outputs[0], V(xi).shape, DT::U8, V(xi).shape.size() == 4 ? V(xi).layout : Layout::PLAIN);
  // scale and zero point live side by side in one 2-lane buffer; the two output values alias it
  int pi = add_value(n.outputs[0] + "@params", {2}, DT::F32, Layout::PLAIN);
  int si = -1, zi = -1;
  if (n.outputs.size() > 1 && !n.outputs[1].empty()) {
    si = add_value(n.outputs[1], {}, DT::F32, Layout::PLAIN);
    V(si).alias_of = pi;
  }
  if (n.outputs.size() > 2 && !n.outputs[2].empty()) {
    zi = add_value(n.outputs[2], {}, DT::F32, Layout::PLAIN);
    V(zi).alias_of = pi;
  }
  float* scratch = (float*)owned_buffer(256);
  k::dynamic_quantize_scratch_init(scratch);
  Dims4 d{V(xi).numel(), 1, 1, 1};
  TensorRef xr{nullptr, DT::F32, Layout::PLAIN, d}, yr{nullptr, DT::U8, Layout::PLAIN, d};
  std::vector<int> writes = {yi, pi};
  // A LayerNormalization that writes x can take x's extrema while it writes (one pass over the tensor saved):
  // it merges them into this node's keys, which the apply pass resets for the next run as always.
  bool have_minmax = false;
  // So can a tensor-core contraction that writes x as f32 lanes (its steps are still named "umma" here; the plan
  // is built when the arena is laid out and reads the value's keys then).
  if (!C.cfg().keep_intermediates && V(xi).alias_of < 0 && V(xi).producer >= 0 && V(xi).producer < (int)S.steps_.size() &&
      (S.steps_[V(xi).producer].kernel == "layer_norm_rows" || S.steps_[V(xi).producer].kernel == "add+layer_norm_rows" ||
       (S.steps_[V(xi).producer].kernel == "umma" && S.steps_[V(xi).producer].family == 0)) &&
      V(xi).minmax_keys == nullptr) {
    V(xi).minmax_keys = scratch;
    have_minmax = true;
  }
  Step& st = add_step(n, have_minmax ? "dynamic_quantize_linear (extrema from the producer)" : "dynamic_quantize_linear", 2, {xi}, writes);
  st.work = (have_minmax ? 1.0 : 2.0) * (double)V(xi).bytes + (double)V(yi).bytes;
  st.launch = [this, xr, yr, xi, yi, pi, scratch, have_minmax](cudaStream_t s) {
    k::dynamic_quantize_linear(bound(xr, xi), bound(yr, yi), (float*)V(pi).ptr, scratch, s, have_minmax);
    const uint64_t launched = have_minmax ? 1 : 2;
    C.counters.glue_launches += launched;
    C.counters.kernel_launches += launched;
  };
  // the zero-point alias points one lane further
  if (zi >= 0) {
    Step& st2 = S.steps_.back();
    auto prev = st2.finalize;
    st2.finalize = [this, zi, pi, prev]() {
      if (prev) prev();
      V(zi).ptr = (uint8_t*)V(pi).ptr + 4;
    };
  }
  (void)si;
}

// ---- contractions --------------------------------------------------------------------------
void Planner::emit_contraction(const NodeDef& n, Contraction& c) {
  const k::ConvShape& cs = c.cs;
  const int OC = cs.OC, cg = cs.C / cs.group;
  const int64_t taps = (int64_t)cs.R * cs.S;
  const HostTensor* w = c.w;
  const bool cache_w = c.w_cacheable >= 0 ? c.w_cacheable != 0 : cacheable_const(c.w_name);

  auto w_at = [&](int oc, int ic, int64_t tap) -> float {
    if (c.w_is_kn) return w->data[(size_t)ic * OC + oc];  // B[K][N]
    return w->data[((size_t)oc * cg + ic) * taps + tap];
  };

  // integer weights: exact values, narrowest storage
  std::vector<int32_t> wi;
  if (c.is_int) {
    if (!lanes_to_i32(*w, &wi)) OXB_DECLINE("%s '%s': weight holds a non-finite or out-of-range lane", n.op.c_str(), n.name.c_str());
    int32_t lo = 0, hi = 0;
    for (int32_t v : wi) {
      lo = std::min(lo, v);
      hi = std::max(hi, v);
    }
    c.w_dt = narrowest_int(lo, hi);
  }
  auto wi_at = [&](int oc, int ic, int64_t tap) -> int32_t {
    if (c.w_is_kn) return wi[(size_t)ic * OC + oc];
    return wi[((size_t)oc * cg + ic) * taps + tap];
  };

  // ---- can the tensor-core kernel take it? ----
  std::string why;
  bool want_umma = C.cfg().kernel_path == 0 && k::umma_available() && !c.x_plain_nchw;
  Value& xv = V(c.x_vi);
  if (want_umma && c.is_int) {
    bool w_zp_zero = true;
    for (int32_t z : c.w_zp) w_zp_zero &= z == 0;
    bool pads = cs.pt || cs.pl || cs.pb || cs.pr;
    if (!(xv.dt == DT::U8 || xv.dt == DT::I8)) want_umma = false, why = "activation is not stored as 8-bit";
    else if (!(c.w_dt == DT::I8 || c.w_dt == DT::U8)) want_umma = false, why = "weights do not fit 8 bits";
    else if (!w_zp_zero) want_umma = false, why = "non-zero weight zero point";
    else if (!c.x_zp_rows.empty()) want_umma = false, why = "per-row zero point";
    else if (pads && !(c.x_zp_static && c.x_zp == 0)) want_umma = false, why = "padding with a non-zero input zero point";
    else if ((double)cs.K() * 255.0 * 255.0 >= 2147483647.0) want_umma = false, why = "reduction too long for an s32 accumulator";
  } else if (want_umma && xv.dt != DT::F32) {
    want_umma = false;
  }
  // float contractions: TF32 operands unless the context asks for f16 / bf16 operands and the channel count fits
  // their 32-byte blocks (16 channels); accumulation is f32 either way
  // A weight the model declares as FLOAT16 / BFLOAT16 (the declared type survives loading beside the f32 lanes)
  // selects that kind for its contraction even without the context option: the graph's own tensors are 16-bit.
  int float_kind = 1;
  int want16 = C.cfg().float_precision == 1 ? 2 : (C.cfg().float_precision == 2 ? 3 : 0);
  if (want16 == 0 && w && w->declared == DT::F16) want16 = 2;
  if (want16 == 0 && w && w->declared == DT::BF16) want16 = 3;
  if (want_umma && !c.is_int && want16 != 0 && k::umma_channel_block(cs.C, want16) != 0) float_kind = want16;
  if (want_umma && k::umma_channel_block(cs.C, c.is_int ? 0 : float_kind) == 0) want_umma = false, why = "channel count not a multiple of the block";
  if (want_umma && cs.group != 1) want_umma = false, why = "grouped";

  // ---- epilogue parameter vectors ----
  k::Epilogue epi = c.epi;
  std::vector<int32_t> wsum(OC, 0);
  int64_t acc_abs_bound = 0;  // max over channels of 255 * sum|w| + |bias| + 255 * |sum w|
  if (c.is_int)
    for (int oc = 0; oc < OC; ++oc) {
      int64_t s = 0, sabs = 0;
      for (int ic = 0; ic < cg; ++ic)
        for (int64_t t = 0; t < taps; ++t) {
          const int64_t wv = wi_at(oc, ic, t);
          s += wv;
          sabs += wv < 0 ? -wv : wv;
        }
      wsum[oc] = (int32_t)s;
      const int64_t b = c.bias_i.empty() ? 0 : c.bias_i[oc];
      const int64_t bound = 255 * sabs + (b < 0 ? -b : b) + 255 * (s < 0 ? -s : s);
      acc_abs_bound = std::max(acc_abs_bound, bound);
    }
  epi.acc_abs_bound = acc_abs_bound;

  const int x_vi = c.x_vi, out_vi = c.out_vi, xzp_vi = c.x_zp_vi, res_vi = c.res_vi, dq_vi = c.dq_xs_vi;
  std::vector<int> reads = {x_vi};
  if (xzp_vi >= 0) reads.push_back(xzp_vi);
  if (res_vi >= 0) reads.push_back(res_vi);
  if (dq_vi >= 0) reads.push_back(dq_vi);
  if (epi.mode == k::EPI_DEQUANT) {
    const size_t padded = align_up((size_t)OC, 256);
    std::vector<float> ws = c.dq_w_scale, bs = c.dq_bias;
    ws.resize(padded, 0.f);
    bs.resize(padded, 0.f);
    epi.dq_w_scale = upload_vec(ws);
    epi.dq_bias = upload_vec(bs);
  }

  if (want_umma) {
    const int kind = c.is_int ? 0 : float_kind;
    const DT f_dt = float_kind == 2 ? DT::F16 : (float_kind == 3 ? DT::BF16 : DT::F32);
    const size_t es = c.is_int ? 1 : dt_size(f_dt);
    const int64_t ktot = cs.K();
    const size_t wbytes = (size_t)OC * ktot * es;
    char form[96];
    snprintf(form, sizeof form, "umma_%s_%dx%dx%dx%d_a%.9g%s", c.is_int ? dt_name(c.w_dt) : (float_kind == 1 ? "tf32" : dt_name(f_dt)), OC, cs.C, cs.R, cs.S,
             (double)c.w_scale_mul, c.w_is_kn ? "_kn" : "");
    const float wmul = c.w_scale_mul;
    void* wdev = C.resident_form(
        c.w_name, form, wbytes,
        [&](void* dst) {
          for (int oc = 0; oc < OC; ++oc)
            for (int64_t t = 0; t < taps; ++t)
              for (int ic = 0; ic < cs.C; ++ic) {
                size_t o = (size_t)oc * ktot + (size_t)t * cs.C + ic;
                if (c.is_int) {
                  ((uint8_t*)dst)[o] = (uint8_t)(wi_at(oc, ic, t) & 0xff);
                } else {
                  const float wv = wmul == 1.0f ? w_at(oc, ic, t) : w_at(oc, ic, t) * wmul;
                  if (float_kind == 1) ((float*)dst)[o] = round_to_tf32(wv);
                  else ((uint16_t*)dst)[o] = float_kind == 2 ? f32_to_f16_bits(wv) : f32_to_bf16_bits(wv);
                }
              }
        },
        cache_w);
    if (c.is_int) {
      std::vector<int32_t> bias_eff(OC, 0);
      for (int oc = 0; oc < OC; ++oc) {
        int64_t b = c.bias_i.empty() ? 0 : c.bias_i[oc];
        if (c.x_zp_static) b -= (int64_t)c.x_zp * wsum[oc];
        if (b < INT32_MIN || b > INT32_MAX) OXB_DECLINE("%s '%s': folded bias leaves the int32 range", n.op.c_str(), n.name.c_str());
        bias_eff[oc] = (int32_t)b;
      }
      // parameter vectors are padded to a multiple of 256 channels: the kernel reads them in
      // 16-byte pieces without bounds checks
      const size_t padded = align_up((size_t)OC, 256);
      bias_eff.resize(padded, 0);
      epi.bias_i = upload_vec(bias_eff);
      // the same bias as f32 lanes, exact below 2^24, for the epilogue variant that adds it after the conversion
      bool bias_fits = c.x_zp_static;
      for (int32_t b : bias_eff) bias_fits = bias_fits && b > -16777216 && b < 16777216;
      if (bias_fits && epi.mode == k::EPI_REQUANT) {
        std::vector<float> bias_as_f(bias_eff.begin(), bias_eff.end());
        epi.bias_if = upload_vec(bias_as_f);
      }
      if (c.x_zp_static) {
        epi.wsum = nullptr;
      } else {
        wsum.resize(padded, 0);
        epi.wsum = upload_vec(wsum);
      }
      if (epi.mode == k::EPI_REQUANT) {
        std::vector<float> comb = c.combined;
        epi.combined_fma_ok = 1;
        for (float v : comb) {
          const float a = std::fabs(v);
          if (!(a == 0.f || (a >= 4.76837158203125e-07f && a <= 1099511627776.0f))) epi.combined_fma_ok = 0;
        }
        double cmax = 0.0;
        for (float v : comb) cmax = std::max(cmax, (double)std::fabs(v));
        epi.q_abs_bound = (double)acc_abs_bound * cmax * 1.0001 + std::fabs((double)epi.y_zp) + 1.0;
        comb.resize(padded, 0.f);
        epi.combined = upload_vec(comb);
      }
    } else {
      std::vector<float> bias = c.bias_f;
      bias.resize(align_up((size_t)OC, 256), 0.f);
      epi.bias_f = upload_vec(bias);
      if (epi.act == 4) {
        std::vector<float> sl = c.slope;
        sl.resize(align_up((size_t)OC, 256), 0.f);
        epi.slope = upload_vec(sl);
      }
    }
    int x_op_vi = x_vi;  // the value the kernel reads as its A operand
    if (!c.is_int && float_kind != 1) {
      x_op_vi = half_copy(n, x_vi, f_dt);
      reads[0] = x_op_vi;
    } else if (!c.is_int && !tf32_ready(x_vi)) {
      x_op_vi = tf32_copy(n, x_vi);
      reads[0] = x_op_vi;
    }
    Step& st = add_step(n, "umma", 0, reads, {out_vi});
    st.work = c.algorithmic_ops > 0 ? c.algorithmic_ops : cs.ops();
    st.work_is_bytes = false;
    st.param_bytes = (double)wbytes;
    const DT xdt = V(x_op_vi).dt, wdt = c.is_int ? c.w_dt : f_dt;
    Step* stp = &st;
    const int step_index = (int)S.steps_.size() - 1;
    st.finalize = [this, step_index, x_vi = x_op_vi, out_vi, xzp_vi, res_vi, dq_vi, wdev, xdt, wdt, cs, epi, kind, n]() mutable {
      k::Epilogue e = epi;
      if (xzp_vi >= 0) e.x_zp_dev = (const float*)V(xzp_vi).ptr;
      if (res_vi >= 0) e.residual = (const float*)V(res_vi).ptr;
      if (dq_vi >= 0) e.dq_x_scale_dev = (const float*)V(dq_vi).ptr;
      e.minmax_keys = (unsigned int*)V(out_vi).minmax_keys;
      std::string why2;
      k::UmmaTuning tune;
      tune.requant_f64 = C.cfg().requant_f64;
      tune.split_k_max = C.cfg().split_k_max;
      tune.cta_pairs = C.cfg().cta_pairs;
      k::UmmaPlan* plan = k::umma_plan_create(V(x_vi).ptr, xdt, wdev, wdt, V(out_vi).ptr, cs, e, kind, tune, &why2);
      if (!plan) OXB_FAIL("%s '%s': tensor-core plan rejected after selection: %s", n.op.c_str(), n.name.c_str(), why2.c_str());
      S.umma_plans_.push_back(plan);
      Step& me = S.steps_[step_index];
      me.kernel = std::string(k::umma_plan_desc(plan)) + (res_vi >= 0 ? " +residual" : "") + (dq_vi >= 0 ? " +dequant" : "");
      // a quantised linear layer over few rows may become a link of a one-kernel chain (link_chains)
      if (kind == 0 && e.mode == k::EPI_REQUANT && xzp_vi < 0 && res_vi < 0 && dq_vi < 0 && cs.R == 1 && cs.S == 1 && cs.sh == 1 && cs.sw == 1 &&
          cs.pt == 0 && cs.pl == 0 && cs.pb == 0 && cs.pr == 0 && cs.group == 1 && cs.x_pixel_stride == 0 && cs.M() <= 64 && cs.C % 128 == 0 &&
          dt_size(e.out_dt) == 1 && C.cfg().split_k_max != 1) {
        ChainLink cl;
        cl.step = step_index;
        cl.rows = (int)cs.M();
        cl.x_vi = x_vi;
        cl.out_vi = out_vi;
        cl.layer.x = V(x_vi).ptr;
        cl.layer.x_dt = xdt;
        cl.layer.w = wdev;
        cl.layer.w_dt = wdt;
        cl.layer.out = V(out_vi).ptr;
        cl.layer.K = cs.C;
        cl.layer.N = cs.OC;
        cl.layer.bias_i = e.bias_i;
        cl.layer.combined = e.combined;
        cl.layer.y_zp = e.y_zp;
        cl.layer.lo = (e.relu_fused && e.lo < 0) ? 0 : e.lo;
        cl.layer.hi = e.hi;
        cl.layer.fma_exact = e.combined_fma_ok && C.cfg().requant_f64 != 1;
        chain_links_.push_back(cl);
      }
      int* err = S.err_flag_;
      me.launch = [this, plan, err](cudaStream_t s) {
        k::umma_launch(plan, err, s);
        C.counters.umma_launches++;
        C.counters.kernel_launches++;
      };
    };
    (void)stp;
    return;
  }

  // ---- direct kernel ----
  if (cs.x_pixel_stride != 0) OXB_DECLINE("%s '%s': the row-window stem layout needs the tensor-core kernel (%s)", n.op.c_str(), n.name.c_str(), why.c_str());
  {
    const size_t es = c.is_int ? dt_size(c.w_dt) : 4;
    const size_t wbytes = (size_t)taps * cg * OC * es;
    char form[96];
    snprintf(form, sizeof form, "direct_%s_%dx%dx%dx%d_a%.9g%s", c.is_int ? dt_name(c.w_dt) : "f32", OC, cg, cs.R, cs.S, (double)c.w_scale_mul,
             c.w_is_kn ? "_kn" : "");
    const float wmul = c.w_scale_mul;
    const DT wdt = c.is_int ? c.w_dt : DT::F32;
    void* wdev = C.resident_form(
        c.w_name, form, wbytes,
        [&](void* dst) {
          for (int64_t t = 0; t < taps; ++t)
            for (int ic = 0; ic < cg; ++ic)
              for (int oc = 0; oc < OC; ++oc) {
                size_t o = ((size_t)t * cg + ic) * OC + oc;
                if (!c.is_int) {
                  ((float*)dst)[o] = wmul == 1.0f ? w_at(oc, ic, t) : w_at(oc, ic, t) * wmul;
                } else {
                  int32_t v = wi_at(oc, ic, t);
                  switch (wdt) {
                    case DT::U8: ((uint8_t*)dst)[o] = (uint8_t)v; break;
                    case DT::I8: ((int8_t*)dst)[o] = (int8_t)v; break;
                    case DT::I16: ((int16_t*)dst)[o] = (int16_t)v; break;
                    default: ((int32_t*)dst)[o] = v; break;
                  }
                }
              }
        },
        cache_w);
    if (c.is_int) {
      epi.bias_i = c.bias_i.empty() ? nullptr : upload_vec(c.bias_i);
      epi.x_zp = c.x_zp;
      if (!c.x_zp_rows.empty()) epi.x_zp_rows = upload_vec(c.x_zp_rows);
      bool any_wzp = false;
      for (int32_t z : c.w_zp) any_wzp |= z != 0;
      if (any_wzp) {
        epi.w_zp = upload_vec(c.w_zp);
        epi.n_w_zp = (int)c.w_zp.size();
      }
      if (epi.mode == k::EPI_REQUANT) epi.combined = upload_vec(c.combined);
    } else {
      epi.bias_f = c.bias_f.empty() ? nullptr : upload_vec(c.bias_f);
      if (epi.act == 4) epi.slope = upload_vec(c.slope);
    }
    Step& st = add_step(n, "direct", 1, reads, {out_vi});
    st.kernel = std::string("direct_") + (c.is_int ? "int" : "f32") + (why.empty() ? "" : (" (" + why + ")"));
    st.work = cs.ops();
    st.work_is_bytes = false;
    const DT xdt = xv.dt;
    const int plain = c.x_plain_nchw ? 1 : 0;
    st.launch = [this, x_vi, out_vi, xzp_vi, res_vi, dq_vi, wdev, xdt, wdt, cs, epi, plain](cudaStream_t s) {
      k::Epilogue e = epi;
      if (xzp_vi >= 0) e.x_zp_dev = (const float*)V(xzp_vi).ptr;
      if (res_vi >= 0) e.residual = (const float*)V(res_vi).ptr;
      if (dq_vi >= 0) e.dq_x_scale_dev = (const float*)V(dq_vi).ptr;
      k::conv_direct(V(x_vi).ptr, xdt, plain, wdev, wdt, V(out_vi).ptr, cs, e, s);
      C.counters.simt_launches++;
      C.counters.kernel_launches++;
    };
  }
}

// Integer storage for a value that reaches an integer contraction as f32 lanes (a fed graph
// input, or an operand of a one-node dispatch whose lanes are known).
static DT int_storage_for(const Value& v, bool* ok) {
  *ok = true;
  if (v.dt != DT::F32) return v.dt;
  if (!v.host) return DT::I32;
  int64_t lo = 0, hi = 0;
  for (float f : v.host->data) {
    int32_t q;
    if (!lane_to_i32(f, &q)) {
      *ok = false;
      return DT::I32;
    }
    lo = std::min<int64_t>(lo, q);
    hi = std::max<int64_t>(hi, q);
  }
  return narrowest_int(lo, hi);
}

// A stride-2 convolution over very few channels (the 3-channel 7x7 stem) cannot feed the
// tensor cores directly: its channel rows are a few bytes long.  With ih = 2*oh - pt + r, shift
// the tap index by e = pt mod 2 so that ih = 2*(oh - (pt+e)/2 + a) + b with r + e = 2a + b: the
// same sums as a stride-1 convolution with ceil((R+e)/2) taps over the 2x2 space-to-depth copy
// P[n, y, x, (b_h, b_w, c)] = X[n, c, 2y+b_h, 2x+b_w], whose 4*C channels (padded) give rows of
// 32..128 bytes.  Taps that the shift invents carry zero weights; rows and columns outside P are
// exactly the original padding, so the tensor-map zero fill stays correct.  For integer inputs
// the copy stores x - x_zero_point, which makes the fill value equal to the zero point.
bool Planner::try_s2d_stem(const NodeDef& n, Contraction& c, int src_vi) {
  k::ConvShape& cs = c.cs;
  const Value xv = V(src_vi);
  if (cs.group != 1 || cs.sh != 2 || cs.sw != 2 || cs.dh != 1 || cs.dw != 1) return false;
  if (cs.C > 8 || (cs.H & 1) || (cs.W & 1) || xv.shape.size() != 4) return false;
  if (k::umma_channel_block(cs.C, c.is_int ? 0 : 1) != 0) return false;  // already eligible as it is
  int sub = 0;
  DT pdt = DT::F32;
  if (c.is_int) {
    if (!c.x_zp_static || !c.x_zp_rows.empty()) return false;
    for (int32_t z : c.w_zp)
      if (z != 0) return false;
    if (xv.dt == DT::U8 && c.x_zp == 128) sub = 128, pdt = DT::I8;
    else if ((xv.dt == DT::U8 || xv.dt == DT::I8) && c.x_zp == 0) pdt = xv.dt;
    else return false;
  } else if (xv.dt != DT::F32) {
    return false;
  }
  const int eh = cs.pt & 1, ew = cs.pl & 1;
  const int R2 = (cs.R + eh + 1) / 2, S2 = (cs.S + ew + 1) / 2;
  const int H2 = cs.H / 2, W2 = cs.W / 2;
  const int pt2 = (cs.pt + eh) / 2, pl2 = (cs.pl + ew) / 2;
  const int pb2 = cs.P - 1 + R2 - H2 - pt2, pr2 = cs.Q - 1 + S2 - W2 - pl2;
  if (pb2 < 0 || pr2 < 0) return false;
  const int c4 = 4 * cs.C;
  const int es = c.is_int ? 1 : 4;
  if (c4 <= 16 && S2 <= 8 && k::umma_overlapping_positions_ok()) {
    // Row-window layout: 16 lanes per packed pixel, a zero halo on both sides of every row, and
    // one filter-row tap = S2p neighbouring pixels = S2p * 16 contiguous lanes.  The convolution
    // the kernel sees has R2 taps of S2p * 16 "channels" each (positions overlap, 16 lanes apart).
    const int S2p = S2 <= 2 ? 2 : (S2 <= 4 ? 4 : 8);
    // Row pairs (8-bit stems with an even number of packed filter rows): a packed pixel carries the blocks of two
    // vertically adjacent rows, 32 lanes, so that one window of S2p pixels is 128 contiguous bytes covering two
    // filter rows -- half as many, twice as long rows for the TMA unit, whose cost is per row.  The vertical
    // padding becomes physical (rows of zeros written by the packing kernel) and the taps step two rows.
    const bool pairs = c.is_int && (R2 % 2 == 0) && S2p * 32 <= 128;
    const int CP = pairs ? 32 : 16, Cw = S2p * CP;
    const int RT = pairs ? R2 / 2 : R2;              // taps the kernel sees
    const int rows_phys = pairs ? cs.P - 2 + R2 : H2;  // stored rows per image
    const int wp = pl2 + W2 + pr2 + (S2p - S2);
    const HostTensor* w = c.w;
    made_consts_.emplace_back();
    HostTensor& w2 = made_consts_.back();
    w2.shape = {cs.OC, Cw, RT, 1};
    w2.data.assign((size_t)cs.OC * Cw * RT, 0.f);
    for (int oc = 0; oc < cs.OC; ++oc)
      for (int bh = 0; bh < 2; ++bh)
        for (int bw = 0; bw < 2; ++bw)
          for (int ch = 0; ch < cs.C; ++ch)
            for (int a = 0; a < R2; ++a)
              for (int b = 0; b < S2; ++b) {
                const int r = 2 * a + bh - eh, s = 2 * b + bw - ew;
                if (r < 0 || r >= cs.R || s < 0 || s >= cs.S) continue;
                const int lane = b * CP + (pairs ? (a % 2) * 16 : 0) + (bh * 2 + bw) * cs.C + ch;
                const int tap = pairs ? a / 2 : a;
                w2.data[((size_t)oc * Cw + lane) * RT + tap] = w->data[(((size_t)oc * cs.C + ch) * cs.R + r) * cs.S + s];
              }
    // quantise on the way when the activation is the sole product of the QuantizeLinear just planned
    k::S2dQuant q;
    int read_vi = src_vi;
    if (c.is_int && xv.q_src >= 0 && xv.q_step == (int)S.steps_.size() - 1 && !C.cfg().keep_intermediates && !graph_outputs_.count(xv.name) &&
        V(xv.q_src).shape.size() == 4) {
      auto it = consumers_.find(xv.name);
      if (it != consumers_.end() && it->second.size() == 1) {
        q.quantize = 1;
        q.scale = xv.q_scale, q.zp = xv.q_zp, q.lo = xv.q_lo, q.hi = xv.q_hi;
        read_vi = xv.q_src;
        S.steps_.pop_back();
        V(src_vi).producer = -1;
      }
    }
    const Value rv = V(read_vi);
    std::vector<int64_t> pshape = {cs.N, CP, rows_phys, wp};
    int pv = add_value(xv.name + "@s2dw", pshape, pdt, Layout::NHWC);
    k::TensorRef src{nullptr, rv.dt, effective_layout(rv), dims_of(rv)};
    if (order_free(rv)) src.layout = Layout::NHWC;
    Step& st = add_step(n, q.quantize ? "quantize+s2d_window_pack" : "s2d_window_pack", 2, {read_vi}, {pv});
    st.work = (double)rv.bytes + (double)V(pv).bytes;
    const DT pdt_c = pdt;
    const int pair_top = pairs ? pt2 : -1;
    st.launch = [this, src, read_vi, pv, pdt_c, pl2, wp, sub, q, pair_top, rows_phys](cudaStream_t s) {
      k::s2d_window_pack(bound(src, read_vi), V(pv).ptr, pdt_c, pl2, wp, sub, q, pair_top, rows_phys, s);
      C.counters.glue_launches++;
      C.counters.kernel_launches++;
    };
    c.algorithmic_ops = cs.ops();
    c.w_cacheable = cacheable_const(c.w_name) ? 1 : 0;
    c.w = &w2;
    c.w_name = c.w_name + "@s2dw";
    c.x_vi = pv;
    c.x_plain_nchw = false;
    c.x_zp = 0;
    cs.C = Cw;
    cs.H = rows_phys;
    cs.W = cs.Q;  // window start positions per row
    cs.R = RT;
    cs.S = 1;
    cs.sh = cs.sw = 1;
    cs.dh = pairs ? 2 : 1;
    cs.pt = pairs ? 0 : pt2;
    cs.pb = pairs ? 0 : pb2;
    cs.pl = cs.pr = 0;
    cs.x_pixel_stride = CP;
    cs.x_row_pixels = wp;
    return true;
  }
  int c_pad = 0;
  for (int bytes : {32, 64, 128})
    if (c4 * es <= bytes) {
      c_pad = bytes / es;
      break;
    }
  if (c_pad == 0) return false;
  // rewritten filter in ONNX order [OC, c_pad, R2, S2]
  const HostTensor* w = c.w;
  made_consts_.emplace_back();
  HostTensor& w2 = made_consts_.back();
  w2.shape = {cs.OC, c_pad, R2, S2};
  w2.data.assign((size_t)cs.OC * c_pad * R2 * S2, 0.f);
  for (int oc = 0; oc < cs.OC; ++oc)
    for (int bh = 0; bh < 2; ++bh)
      for (int bw = 0; bw < 2; ++bw)
        for (int ch = 0; ch < cs.C; ++ch)
          for (int a = 0; a < R2; ++a)
            for (int b = 0; b < S2; ++b) {
              const int r = 2 * a + bh - eh, s = 2 * b + bw - ew;
              if (r < 0 || r >= cs.R || s < 0 || s >= cs.S) continue;
              const int cp = (bh * 2 + bw) * cs.C + ch;
              w2.data[(((size_t)oc * c_pad + cp) * R2 + a) * S2 + b] = w->data[(((size_t)oc * cs.C + ch) * cs.R + r) * cs.S + s];
            }
  // the packed activation
  std::vector<int64_t> pshape = {cs.N, c_pad, H2, W2};
  int pv = add_value(xv.name + "@s2d", pshape, pdt, Layout::NHWC);
  k::TensorRef src{nullptr, xv.dt, effective_layout(xv), dims_of(xv)};
  if (order_free(xv)) src.layout = Layout::NHWC;
  Step& st = add_step(n, "s2d_pack", 2, {src_vi}, {pv});
  st.work = (double)xv.bytes + (double)V(pv).bytes;
  const DT pdt_c = pdt;
  st.launch = [this, src, src_vi, pv, pdt_c, c_pad, sub](cudaStream_t s) {
    k::s2d_pack(bound(src, src_vi), V(pv).ptr, pdt_c, c_pad, sub, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
  c.algorithmic_ops = cs.ops();
  c.w_cacheable = cacheable_const(c.w_name) ? 1 : 0;
  c.w = &w2;
  c.w_name = c.w_name + "@s2d";
  c.x_vi = pv;
  c.x_plain_nchw = false;
  c.x_zp = 0;
  cs.C = c_pad;
  cs.H = H2;
  cs.W = W2;
  cs.R = R2;
  cs.S = S2;
  cs.sh = cs.sw = 1;
  cs.pt = pt2;
  cs.pl = pl2;
  cs.pb = pb2;
  cs.pr = pr2;
  return true;
}

// A stride-1 float convolution over at most four channels (an image-space 7x7): four lanes per
// pixel, and one filter-row tap = the S (rounded up to 2, 4 or 8) neighbouring pixels of a row, read
// through a tensor map whose positions overlap, exactly as the space-to-depth stem does.
bool Planner::try_window_stem(const NodeDef& n, Contraction& c, int src_vi) {
  k::ConvShape& cs = c.cs;
  const Value xv = V(src_vi);
  if (c.is_int || xv.dt != DT::F32 || xv.shape.size() != 4) return false;
  if (cs.group != 1 || cs.sh != 1 || cs.sw != 1 || cs.dh != 1 || cs.dw != 1 || cs.C > 4 || cs.S > 8 || cs.S < 2) return false;
  if (!k::umma_overlapping_positions_ok()) return false;
  const int Sp = cs.S <= 2 ? 2 : (cs.S <= 4 ? 4 : 8);
  const int CP = 4, Cw = Sp * CP;
  if (k::umma_channel_block(Cw, 1) == 0) return false;
  const int wp = cs.pl + cs.W + cs.pr + (Sp - cs.S);
  const HostTensor* w = c.w;
  made_consts_.emplace_back();
  HostTensor& w2 = made_consts_.back();
  w2.shape = {cs.OC, Cw, cs.R, 1};
  w2.data.assign((size_t)cs.OC * Cw * cs.R, 0.f);
  for (int oc = 0; oc < cs.OC; ++oc)
    for (int ch = 0; ch < cs.C; ++ch)
      for (int r = 0; r < cs.R; ++r)
        for (int sx = 0; sx < cs.S; ++sx)
          w2.data[((size_t)oc * Cw + sx * CP + ch) * cs.R + r] = w->data[(((size_t)oc * cs.C + ch) * cs.R + r) * cs.S + sx];
  std::vector<int64_t> pshape = {cs.N, CP, cs.H, wp};
  int pv = add_value(xv.name + "@window", pshape, DT::F32, Layout::NHWC);
  k::TensorRef src{nullptr, xv.dt, effective_layout(xv), dims_of(xv)};
  if (order_free(xv)) src.layout = Layout::NHWC;
  Step& st = add_step(n, "window_pack", 2, {src_vi}, {pv});
  st.work = (double)xv.bytes + (double)V(pv).bytes;
  const int pl = cs.pl;
  st.launch = [this, src, src_vi, pv, pl, wp](cudaStream_t s) {
    k::window_pack_f32(bound(src, src_vi), V(pv).ptr, pl, wp, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
  c.algorithmic_ops = cs.ops();
  c.w_cacheable = cacheable_const(c.w_name) ? 1 : 0;
  c.w = &w2;
  c.w_name = c.w_name + "@window";
  c.x_vi = pv;
  c.x_plain_nchw = false;
  cs.C = Cw;
  cs.W = cs.Q;
  cs.S = 1;
  cs.pl = cs.pr = 0;
  cs.x_pixel_stride = CP;
  cs.x_row_pixels = wp;
  return true;
}

void Planner::plan_conv_family(const NodeDef& n, int ni) {
  (void)ni;
  const std::string& op = n.op;
  // ConvAddRelu (src/optimizer/fusion/conv/add_relu.rs:114-156): inputs (x, w, bias or "", residual), the Conv's
  // attributes plus fused_ops = "Add,Relu"; relu(conv(x, w, bias) + residual)
  const bool is_car = op == "ConvAddRelu";
  const bool is_q = op == "QLinearConv", is_ci = op == "ConvInteger", is_f = op == "Conv" || is_car;
  if (is_car) {
    check_attrs(n, {"strides", "pads", "dilations", "group", "auto_pad", "kernel_shape", "fused_ops"});
    if (n.attrs.s("fused_ops") != "Add,Relu") OXB_DECLINE("ConvAddRelu '%s': fused_ops is not \"Add,Relu\"", n.name.c_str());
    if (!has_in(n, 3)) OXB_DECLINE("ConvAddRelu '%s': no residual operand", n.name.c_str());
  } else if (is_f) check_attrs(n, {"strides", "pads", "dilations", "group", "auto_pad", "kernel_shape", "activation", "activation_min", "activation_max"});
  else check_attrs(n, {"strides", "pads", "dilations", "group", "auto_pad", "kernel_shape"});
  const size_t w_slot = is_q ? 3 : 1;
  const HostTensor* w = const_in(n, w_slot);
  if (!w) OXB_DECLINE("%s '%s': the filter is not an initializer", op.c_str(), n.name.c_str());
  int xi = value_of(in_name(n, 0));
  const Value xv = V(xi);
  if (xv.shape.size() != 4 || w->shape.size() != 4) OXB_DECLINE("%s '%s': only 2-D convolutions (rank-4 operands) are claimed", op.c_str(), n.name.c_str());
  if ((int64_t)w->data.size() != w->numel()) OXB_DECLINE("%s: weight data length does not match its shape", op.c_str());
  int64_t group = n.attrs.i("group", 1);
  if (group < 1) OXB_DECLINE("%s: group must be >= 1", op.c_str());
  if (w->shape[1] * group != xv.shape[1]) OXB_DECLINE("%s: input channels %lld != weight input channels %lld * group %lld", op.c_str(), (long long)xv.shape[1], (long long)w->shape[1], (long long)group);
  if (w->shape[0] % group != 0) OXB_DECLINE("%s: output channels not divisible by group", op.c_str());
  if (is_f) {
    auto ks = n.attrs.int_list("kernel_shape");
    if (!ks.empty()) {
      if (ks.size() < 2 || ks[0] != w->shape[2] || ks[1] != w->shape[3]) OXB_DECLINE("Conv: kernel_shape disagrees with weight spatial dims");
    }
  }
  Geo g = resolve_geometry(op.c_str(), n.attrs, xv.shape.data() + 2, w->shape.data() + 2, 2, false);
  Contraction c;
  k::ConvShape& cs = c.cs;
  cs.N = (int)xv.shape[0];
  cs.C = (int)xv.shape[1];
  cs.H = (int)xv.shape[2];
  cs.W = (int)xv.shape[3];
  cs.OC = (int)w->shape[0];
  cs.R = (int)w->shape[2];
  cs.S = (int)w->shape[3];
  cs.P = (int)g.out_spatial[0];
  cs.Q = (int)g.out_spatial[1];
  cs.sh = (int)g.strides[0];
  cs.sw = (int)g.strides[1];
  cs.pt = (int)g.pads[0];
  cs.pl = (int)g.pads[1];
  cs.pb = (int)g.pads[2];
  cs.pr = (int)g.pads[3];
  cs.dh = (int)g.dilations[0];
  cs.dw = (int)g.dilations[1];
  cs.group = (int)group;
  c.w = w;
  c.w_name = in_name(n, w_slot);
  c.is_int = !is_f;
  std::vector<int64_t> out_shape = {xv.shape[0], w->shape[0], g.out_spatial[0], g.out_spatial[1]};
  std::string out_name = n.outputs[0];

  if (is_f) {
    if (xv.dt != DT::F32) OXB_DECLINE("Conv '%s': input is not a float tensor", n.name.c_str());
    const HostTensor* b = has_in(n, 2) ? const_in(n, 2) : nullptr;
    if (has_in(n, 2) && !b) OXB_DECLINE("Conv '%s': bias is not an initializer", n.name.c_str());
    if (b) {
      if ((int64_t)b->data.size() != cs.OC) OXB_DECLINE("Conv: bias has %zu entries, expected %d", b->data.size(), cs.OC);
      c.bias_f = b->data;
    }
    c.epi.mode = k::EPI_F32;
    std::string act = n.attrs.s("activation");
    if (act == "relu") {
      c.epi.act = 1;
    } else if (act == "clip") {
      float mn = n.attrs.f("activation_min", -std::numeric_limits<float>::infinity());
      float mx = n.attrs.f("activation_max", std::numeric_limits<float>::infinity());
      float lo = std::isnan(mn) ? -std::numeric_limits<float>::infinity() : mn;
      float hi = std::isnan(mx) ? std::numeric_limits<float>::infinity() : mx;
      if (lo <= hi) {  // an inverted range passes the data through (conv_ops/conv.rs:150)
        c.epi.act = 2;
        c.epi.clip_lo = lo;
        c.epi.clip_hi = hi;
      }
    } else if (!act.empty()) {
      OXB_DECLINE("Conv '%s': fused activation '%s' is not one the optimizer emits", n.name.c_str(), act.c_str());
    }
    c.epi.out_dt = DT::F32;
    // a stem that reads a channels-first graph input directly skips the layout pass
    bool direct_nchw = xv.layout == Layout::PLAIN && !order_free(xv) && k::umma_channel_block(cs.C, 1) == 0;
    if (C.cfg().kernel_path == 0 && k::umma_available() && try_s2d_stem(n, c, xi)) {
      // the stride-2 few-channel stem became a stride-1 convolution over a space-to-depth copy
    } else if (C.cfg().kernel_path == 0 && k::umma_available() && try_window_stem(n, c, xi)) {
      // a stride-1 few-channel convolution reads row windows of a four-lane copy
    } else if (direct_nchw) {
      c.x_plain_nchw = true;
      c.x_vi = xi;
    } else {
      c.x_vi = ensure_layout(n, xi, Layout::NHWC);
    }
    if (is_car) {
      // the residual rides in the epilogue when it is a device-resident f32 tensor of the output's shape (brought
      // to channels-last first if need be); the sum and the Relu round as the separate nodes would
      int ri = value_of(in_name(n, 3));
      if (V(ri).dt != DT::F32 || V(ri).shape != out_shape) OXB_DECLINE("ConvAddRelu '%s': the residual is not an f32 tensor of the output's shape", n.name.c_str());
      ri = ensure_layout(n, ri, Layout::NHWC);
      c.res_vi = ri;
      c.epi.act = 1;
    }
    // Conv -> Add(other) [-> Relu] with `other` already on the device in the same layout: the
    // addition (and the Relu) move into this convolution's epilogue; the two float additions
    // round exactly as the separate nodes would.
    if (!is_car && c.epi.act == 0 && !C.cfg().keep_intermediates && cs.OC % 32 == 0 && !graph_outputs_.count(out_name)) {
      auto it = consumers_.find(out_name);
      if (it != consumers_.end() && it->second.size() == 1) {
        const int add_i = it->second[0].first, slot = it->second[0].second;
        const NodeDef& add = nodes_[add_i];
        if (!skipped_[add_i] && add.op == "Add" && add.inputs.size() == 2 && slot <= 1 && add.attrs.names().empty() && add.inputs[0] != add.inputs[1]) {
          auto other = S.index_.find(add.inputs[1 - slot]);
          if (other != S.index_.end()) {
            const Value& ov = V(other->second);
            if (ov.dt == DT::F32 && ov.shape == out_shape && ov.layout == Layout::NHWC && ov.host == nullptr) {
              c.res_vi = other->second;
              skipped_[add_i] = 1;
              out_name = add.outputs[0];
              const int relu_i = sole_consumer(out_name, "Relu");
              if (relu_i >= 0) {
                skipped_[relu_i] = 1;
                c.epi.act = 1;
                out_name = nodes_[relu_i].outputs[0];
              }
            }
          }
        }
      }
    }
    // Conv -> SiLU and Conv -> PRelu(constant slope, scalar or per channel): these activations have no fused-Conv
    // spelling in the reference's optimizer; they arrive as separate nodes and move into the epilogue here, the
    // value at the activation's output being what the separate node would give.
    if (c.epi.act == 0 && c.res_vi < 0 && !C.cfg().keep_intermediates && !graph_outputs_.count(out_name)) {
      int silu_i = sole_consumer(out_name, "Silu");
      if (silu_i < 0) silu_i = sole_consumer(out_name, "SiLU");
      if (silu_i >= 0 && nodes_[silu_i].inputs.size() == 1) {
        skipped_[silu_i] = 1;
        c.epi.act = 3;
        out_name = nodes_[silu_i].outputs[0];
      } else {
        auto it = consumers_.find(out_name);
        if (it != consumers_.end() && it->second.size() == 1 && it->second[0].second == 0) {
          const int pi = it->second[0].first;
          const NodeDef& pr = nodes_[pi];
          const HostTensor* slope = (pr.op == "PRelu" && !skipped_[pi] && pr.inputs.size() == 2 && pr.attrs.names().empty()) ? const_of(pr.inputs[1]) : nullptr;
          if (slope && S.index_.find(pr.inputs[1]) == S.index_.end()) {
            const int64_t ns = slope->numel();
            int64_t nontrivial = 0;
            for (int64_t d : slope->shape) nontrivial += d != 1;
            // scalar, or one value per channel shaped [C,1,1] / [1,C,1,1] (numpy broadcasting against [N,C,H,W])
            const bool per_channel = ns == cs.OC && ns > 1 && nontrivial == 1 && slope->shape.size() >= 3 && slope->shape[slope->shape.size() - 3] == ns;
            if (ns == 1 || per_channel) {
              c.slope.assign((size_t)cs.OC, slope->data[0]);
              if (per_channel) c.slope = slope->data;
              skipped_[pi] = 1;
              c.epi.act = 4;
              out_name = pr.outputs[0];
            }
          }
        }
      }
    }
    c.out_vi = add_value(out_name, out_shape, DT::F32, Layout::NHWC);
    c.epi.round_tf32 = feeds_contraction(out_name) ? 1 : 0;
    emit_contraction(n, c);
    return;
  }

  // ---- integer convolutions ----
  auto zp_lanes = [&](size_t slot, const char* what, std::vector<int32_t>* out) {
    out->assign(1, 0);
    if (!has_in(n, slot)) return;
    const HostTensor* t = const_in(n, slot);
    if (!t) OXB_DECLINE("%s '%s': %s is not an initializer", op.c_str(), n.name.c_str(), what);
    if (t->data.empty()) return;
    if (!lanes_to_i32(*t, out)) OXB_DECLINE("%s: %s holds a non-finite or out-of-range lane", op.c_str(), what);
  };
  auto scale_in = [&](size_t slot, const char* what) -> float {
    const HostTensor* t = const_in(n, slot);
    if (!t) OXB_DECLINE("%s '%s': %s is not an initializer", op.c_str(), n.name.c_str(), what);
    if (t->data.empty()) OXB_DECLINE("%s: %s is empty", op.c_str(), what);
    float v = t->data[0];
    if (!std::isfinite(v)) OXB_DECLINE("%s: %s must be finite", op.c_str(), what);
    if (v == 0.0f) OXB_DECLINE("%s: %s scale is zero", op.c_str(), what);
    return v;
  };
  std::vector<int32_t> x_zp_l, w_zp_l, y_zp_l;
  zp_lanes(is_q ? 2 : 2, "x_zero_point", &x_zp_l);
  zp_lanes(is_q ? 5 : 3, "w_zero_point", &w_zp_l);
  if (w_zp_l.size() != 1 && (int64_t)w_zp_l.size() != cs.OC) OXB_DECLINE("%s: w_zero_point has %zu entries, expected 1 or %d", op.c_str(), w_zp_l.size(), cs.OC);
  c.x_zp = x_zp_l.empty() ? 0 : x_zp_l[0];
  c.w_zp = w_zp_l;
  bool ok_lanes;
  DT want_x = int_storage_for(xv, &ok_lanes);
  if (!ok_lanes) OXB_DECLINE("%s: input holds a non-finite or out-of-range lane", op.c_str());
  int xq = xi;
  if (xv.dt == DT::F32) {
    // f32 lanes -> integer storage, channels-last
    xq = add_value(xv.name + "@int", xv.shape, want_x, Layout::NHWC);
    TensorRef a = ref_of(xi), b = ref_of(xq);
    a.layout = layout_for_kernel(xv, Layout::NHWC);
    Step& st = add_step(n, "lanes_to_int", 2, {xi}, {xq});
    st.work = (double)xv.bytes + (double)V(xq).bytes;
    st.launch = [this, a, b, xi, xq](cudaStream_t s) {
      k::convert(bound(a, xi), bound(b, xq), s);
      C.counters.glue_launches++;
      C.counters.kernel_launches++;
    };
  } else {
    xq = ensure_layout(n, xi, Layout::NHWC);
  }
  c.x_vi = xq;
  if (C.cfg().kernel_path == 0 && k::umma_available()) try_s2d_stem(n, c, xq);

  if (is_ci) {
    c.epi.mode = k::EPI_INT32;
    c.epi.out_dt = DT::I32;
    c.out_vi = add_value(out_name, out_shape, DT::I32, Layout::NHWC);
    emit_contraction(n, c);
    return;
  }
  float x_scale = scale_in(1, "x_scale");
  const HostTensor* w_scale = const_in(n, 4);
  if (!w_scale) OXB_DECLINE("QLinearConv '%s': w_scale is not an initializer", n.name.c_str());
  if (w_scale->data.empty()) OXB_DECLINE("QLinearConv: w_scale is empty");
  float y_scale = scale_in(6, "y_scale");
  zp_lanes(7, "y_zero_point", &y_zp_l);
  const HostTensor* bias = has_in(n, 8) ? const_in(n, 8) : nullptr;
  if (has_in(n, 8) && !bias) OXB_DECLINE("QLinearConv '%s': bias is not an initializer", n.name.c_str());
  if (bias && bias->data.empty()) bias = nullptr;
  if (bias) {
    if ((int64_t)bias->data.size() != cs.OC) OXB_DECLINE("QLinearConv: bias has %zu entries, expected %d", bias->data.size(), cs.OC);
    if (!lanes_to_i32(*bias, &c.bias_i)) OXB_DECLINE("QLinearConv: bias holds a non-finite or out-of-range lane");
  }
  bool per_channel = w_scale->data.size() > 1;
  if (per_channel && (int64_t)w_scale->data.size() != cs.OC) OXB_DECLINE("QLinearConv: w_scale has %zu entries, expected 1 or %d", w_scale->data.size(), cs.OC);
  c.combined.resize(cs.OC);
  for (int oc = 0; oc < cs.OC; ++oc) {
    float ws = per_channel ? w_scale->data[oc] : w_scale->data[0];
    if (!std::isfinite(ws)) OXB_DECLINE("QLinearConv: w_scale[%d] must be finite", oc);
    volatile float xw = x_scale * ws;  // f32 product, then f32 quotient (qlinear_conv.rs:99)
    volatile float comb = xw / y_scale;
    c.combined[oc] = comb;
    if (!std::isfinite(c.combined[oc])) OXB_DECLINE("QLinearConv: combined scale is not finite");
  }
  // the node's own zero point decides the range (a rewritten stem carries an effective zero point of 0)
  Range r = sat_range(has_in(n, 7) ? const_in(n, 7) : nullptr, y_zp_l, {x_zp_l.empty() ? 0 : x_zp_l[0]});
  c.epi.mode = k::EPI_REQUANT;
  c.epi.y_zp = y_zp_l.empty() ? 0 : y_zp_l[0];
  c.epi.lo = r.lo;
  c.epi.hi = r.hi;
  // a Relu behind the node clamps the same lanes at zero: fold it into the saturation
  int relu = sole_consumer(out_name, "Relu");
  if (relu >= 0) {
    skipped_[relu] = 1;
    c.epi.relu_fused = 1;
    out_name = nodes_[relu].outputs[0];
    r.lo = std::max(r.lo, 0);
  }
  c.epi.out_dt = narrowest_int(r.lo, r.hi);
  c.out_vi = add_value(out_name, out_shape, c.epi.out_dt, Layout::NHWC);
  emit_contraction(n, c);
}

// MatMul family as a 1x1 convolution over [rows, K] (oxionnx-ops quant_ops/qlinear_matmul.rs:30-254,
// src/math/matmul.rs:53-190).
void Planner::plan_matmul_family(const NodeDef& n, int ni) {
  (void)ni;
  const std::string& op = n.op;
  const bool is_qm = op == "QLinearMatMul", is_mi = op == "MatMulInteger", is_gemm = op == "Gemm";
  if (is_gemm) check_attrs(n, {"alpha", "beta", "transA", "transB"});
  else check_attrs(n, {});
  const size_t b_slot = is_qm ? 3 : 1;
  int ai = value_of(in_name(n, 0));
  if (is_gemm && n.attrs.i("transA", 0) != 0) {
    // A arrives as [K, M]: bring it to [M, K] once, as the channels-last view of a [1, K, M, 1] tensor
    const Value a0 = V(ai);
    if (a0.shape.size() != 2 || a0.dt != DT::F32) OXB_DECLINE("Gemm '%s': transA needs a rank-2 float A", n.name.c_str());
    int at = add_value(a0.name + "@t", {a0.shape[1], a0.shape[0]}, DT::F32, Layout::PLAIN);
    Dims4 d{1, a0.shape[0], a0.shape[1], 1};
    TensorRef src{nullptr, DT::F32, Layout::PLAIN, d}, dst{nullptr, DT::F32, Layout::NHWC, d};
    Step& st = add_step(n, "transpose_a", 2, {ai}, {at});
    st.work = 2.0 * (double)a0.bytes;
    const int a_src = ai;
    st.launch = [this, src, dst, a_src, at](cudaStream_t s) {
      k::convert(bound(src, a_src), bound(dst, at), s);
      C.counters.glue_launches++;
      C.counters.kernel_launches++;
    };
    ai = at;
  }
  const Value av = V(ai);
  const HostTensor* b = const_in(n, b_slot);
  // a stacked constant B of a float MatMul goes through the batched activation x activation product
  const bool b_is_const = b != nullptr && S.index_.find(in_name(n, b_slot)) == S.index_.end() && !(op == "MatMul" && b->shape.size() > 2);

  if (!b_is_const) {
    // activation x activation product: float MatMul only
    if (op != "MatMul") OXB_DECLINE("%s '%s': the B operand is not an initializer", op.c_str(), n.name.c_str());
    int bi = value_of(in_name(n, 1));
    if (try_plan_attention_product(n, ai, bi)) return;
    materialise_heads(ai);
    materialise_heads(bi);
    const Value bv = V(bi);
    if (av.dt != DT::F32 || bv.dt != DT::F32) OXB_DECLINE("MatMul '%s': operands are not float tensors", n.name.c_str());
    if (av.shape.size() < 2 || bv.shape.size() < 2) OXB_DECLINE("MatMul '%s': 1-D operands with a non-constant B", n.name.c_str());
    if ((av.shape.size() == 4 && av.layout == Layout::NHWC && !order_free(av)) || (bv.shape.size() == 4 && bv.layout == Layout::NHWC && !order_free(bv)))
      OXB_DECLINE("MatMul '%s': channels-last operand", n.name.c_str());
    int64_t M = av.shape[av.shape.size() - 2], K = av.shape.back(), K2 = bv.shape[bv.shape.size() - 2], N = bv.shape.back();
    if (K != K2) OXB_DECLINE("MatMul: inner dimensions disagree: %lld vs %lld", (long long)K, (long long)K2);
    int64_t ba = 1, bb = 1;
    for (size_t i = 0; i + 2 < av.shape.size(); ++i) ba *= av.shape[i];
    for (size_t i = 0; i + 2 < bv.shape.size(); ++i) bb *= bv.shape[i];
    int64_t batch;
    if (ba == bb) batch = ba;
    else if (ba == 1) batch = bb;
    else if (bb == 1) batch = ba;
    else OXB_DECLINE("MatMul: batch dimensions disagree (%lld vs %lld) and neither is 1", (long long)ba, (long long)bb);
    std::vector<int64_t> os;
    const std::vector<int64_t>& pre = ba >= bb ? av.shape : bv.shape;
    os.assign(pre.begin(), pre.end() - 2);
    os.push_back(M);
    os.push_back(N);
    int yi = add_value(n.outputs[0], os, DT::F32, Layout::PLAIN);
    Step& st = add_step(n, "matmul_f32_direct", 1, {ai, bi}, {yi});
    st.work = 2.0 * (double)batch * M * K * N;
    st.work_is_bytes = false;
    int64_t as = (ba == 1 && batch != 1) ? 0 : M * K, bs = (bb == 1 && batch != 1) ? 0 : K * N;
    st.launch = [this, ai, bi, yi, batch, M, K, N, as, bs](cudaStream_t s) {
      k::matmul_f32_direct((const float*)V(ai).ptr, (const float*)V(bi).ptr, (float*)V(yi).ptr, batch, M, K, N, as, bs, s);
      C.counters.simt_launches++;
      C.counters.kernel_launches++;
    };
    return;
  }

  if ((int64_t)b->data.size() != b->numel()) OXB_DECLINE("%s: B data length does not match its shape", op.c_str());
  if (av.shape.empty() || b->shape.empty()) OXB_DECLINE("%s: inputs must have rank >= 1", op.c_str());
  if (b->shape.size() > 2) OXB_DECLINE("%s '%s': stacked constant B", op.c_str(), n.name.c_str());
  if (av.shape.size() == 4 && av.layout == Layout::NHWC && !order_free(av)) OXB_DECLINE("%s '%s': channels-last A operand", op.c_str(), n.name.c_str());
  const bool trans_b = is_gemm && n.attrs.i("transB", 0) != 0;
  if (is_gemm && (av.shape.size() != 2 || b->shape.size() != 2)) OXB_DECLINE("Gemm '%s': operands are not rank 2", n.name.c_str());
  const bool a_1d = av.shape.size() == 1, b_1d = b->shape.size() == 1;
  int64_t K = av.shape.back();
  int64_t rows = a_1d ? 1 : prod(av.shape) / std::max<int64_t>(K, 1);
  int64_t Kb, N;
  if (b_1d) {
    Kb = b->shape[0];
    N = 1;
  } else if (trans_b) {
    Kb = b->shape[1];
    N = b->shape[0];
  } else {
    Kb = b->shape[0];
    N = b->shape[1];
  }
  if (K != Kb) OXB_DECLINE("%s: inner dimensions disagree: %lld vs %lld", op.c_str(), (long long)K, (long long)Kb);
  if (rows > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) OXB_DECLINE("%s: extents exceed 32 bits", op.c_str());
  std::vector<int64_t> os;
  if (!a_1d) os.assign(av.shape.begin(), av.shape.end() - 1);
  if (!b_1d) os.push_back(N);

  Contraction c;
  k::ConvShape& cs = c.cs;
  cs.N = (int)rows;
  cs.C = (int)K;
  cs.H = cs.W = 1;
  cs.OC = (int)N;
  cs.R = cs.S = 1;
  cs.P = cs.Q = 1;
  cs.sh = cs.sw = cs.dh = cs.dw = 1;
  cs.pt = cs.pl = cs.pb = cs.pr = 0;
  cs.group = 1;
  c.w = b;
  c.w_name = in_name(n, b_slot);
  c.w_is_kn = !trans_b;  // [K][N] unless Gemm stores B transposed, which is already [N][K] = [OC][C]
  c.is_int = is_qm || is_mi;
  const int64_t M_rows_per_batch = a_1d ? 1 : av.shape[av.shape.size() - 2];

  if (!c.is_int) {
    const HostTensor* full_c = nullptr;
    float full_c_beta = 1.0f;
    if (av.dt != DT::F32) OXB_DECLINE("%s '%s': A is not a float tensor", op.c_str(), n.name.c_str());
    c.epi.mode = k::EPI_F32;
    c.epi.out_dt = DT::F32;
    if (is_gemm) {
      float alpha = n.attrs.f("alpha", 1.0f), beta = n.attrs.f("beta", 1.0f);
      c.w_scale_mul = alpha;
      if (has_in(n, 2)) {
        const HostTensor* cc = const_in(n, 2);
        if (!cc) OXB_DECLINE("Gemm '%s': C is not an initializer", n.name.c_str());
        int64_t cn = cc->numel();
        bool row_like = cn == N && (cc->shape.empty() || cc->shape.back() == N) && (cc->shape.size() < 2 || cc->shape[cc->shape.size() - 2] == 1);
        if (cn == 1 || row_like) {
          c.bias_f.resize(N);
          for (int64_t j = 0; j < N; ++j) {
            volatile float bc = beta * cc->data[cn == 1 ? 0 : j];
            c.bias_f[j] = bc;
          }
        } else {
          // C varies along the rows ([M,N] or [M,1]): a separate add of beta*C after the product
          bool mn = cc->shape.size() == 2 && cc->shape[0] == rows && (cc->shape[1] == N || cc->shape[1] == 1);
          if (!mn) OXB_DECLINE("Gemm '%s': C is not broadcastable to the result", n.name.c_str());
          full_c = cc;
          full_c_beta = beta;
        }
      }
    }
    c.x_vi = ai;
    c.epi.round_tf32 = (!full_c && feeds_contraction(n.outputs[0])) ? 1 : 0;
    if (!full_c) {
      c.out_vi = add_value(n.outputs[0], os, DT::F32, Layout::PLAIN);
      emit_contraction(n, c);
      return;
    }
    int prod_vi = add_value(n.outputs[0] + "@product", os, DT::F32, Layout::PLAIN);
    c.out_vi = prod_vi;
    emit_contraction(n, c);
    const HostTensor* cc = full_c;
    const float beta = full_c_beta;
    char form[48];
    snprintf(form, sizeof form, "gemm_c_beta%.9g", (double)beta);
    const float* cdev = (const float*)C.resident_form(in_name(n, 2), form, cc->data.size() * 4,
                                                      [cc, beta](void* dst) {
                                                        for (size_t i = 0; i < cc->data.size(); ++i) {
                                                          volatile float v = beta * cc->data[i];
                                                          ((float*)dst)[i] = v;
                                                        }
                                                      },
                                                      cacheable_const(in_name(n, 2)));
    int yi = add_value(n.outputs[0], os, DT::F32, Layout::PLAIN);
    int rt = feeds_contraction(n.outputs[0]) ? 1 : 0;
    TensorRef ar{nullptr, DT::F32, Layout::PLAIN, Dims4{rows, N, 1, 1}}, br{(void*)cdev, DT::F32, Layout::PLAIN, Dims4{cc->shape[0], cc->shape[1], 1, 1}},
        yr{nullptr, DT::F32, Layout::PLAIN, Dims4{rows, N, 1, 1}};
    Step& st = add_step(n, "gemm_add_c", 2, {prod_vi}, {yi});
    st.work = 3.0 * (double)V(yi).bytes;
    st.launch = [this, ar, br, yr, prod_vi, yi, rt](cudaStream_t s) {
      k::binary(bound(ar, prod_vi), br, bound(yr, yi), k::BIN_ADD, 0, rt, s);
      C.counters.glue_launches++;
      C.counters.kernel_launches++;
    };
    return;
  }

  // ---- integer matmuls ----
  auto zp_const = [&](size_t slot, const char* what, std::vector<int32_t>* out, bool* is_const) {
    out->assign(1, 0);
    *is_const = true;
    if (!has_in(n, slot)) return;
    const HostTensor* t = const_in(n, slot);
    if (!t || S.index_.find(in_name(n, slot)) != S.index_.end()) {
      *is_const = false;
      return;
    }
    if (t->data.empty()) return;
    if (!lanes_to_i32(*t, out)) OXB_DECLINE("%s: %s holds a non-finite or out-of-range lane", op.c_str(), what);
  };
  std::vector<int32_t> a_zp, b_zp;
  bool a_zp_const, b_zp_const;
  zp_const(2, "a_zero_point", &a_zp, &a_zp_const);
  zp_const(is_qm ? 5 : 3, "b_zero_point", &b_zp, &b_zp_const);
  if (!b_zp_const) OXB_DECLINE("%s '%s': b_zero_point is not an initializer", op.c_str(), n.name.c_str());
  if (a_zp_const && a_zp.size() != 1 && (int64_t)a_zp.size() != M_rows_per_batch)
    OXB_DECLINE("%s: a_zero_point has %zu entries, expected 1 (per tensor) or %lld", op.c_str(), a_zp.size(), (long long)M_rows_per_batch);
  if (b_zp.size() != 1 && (int64_t)b_zp.size() != N)
    OXB_DECLINE("%s: b_zero_point has %zu entries, expected 1 (per tensor) or %lld", op.c_str(), b_zp.size(), (long long)N);
  c.w_zp = b_zp;
  if (a_zp_const) {
    if (a_zp.size() == 1) {
      c.x_zp = a_zp[0];
    } else {
      c.x_zp_rows.resize(rows);
      for (int64_t r = 0; r < rows; ++r) c.x_zp_rows[r] = a_zp[r % M_rows_per_batch];
    }
  } else {
    if (is_qm) OXB_DECLINE("QLinearMatMul '%s': a_zero_point is not an initializer", n.name.c_str());
    int zi = value_of(in_name(n, 2));
    if (V(zi).numel() != 1 || V(zi).dt != DT::F32) OXB_DECLINE("MatMulInteger '%s': dynamic a_zero_point must be one f32 lane", n.name.c_str());
    c.x_zp_static = false;
    c.x_zp_vi = zi;
  }
  bool ok_lanes;
  DT want_a = int_storage_for(av, &ok_lanes);
  if (!ok_lanes) OXB_DECLINE("%s: A holds a non-finite or out-of-range lane", op.c_str());
  int aq = ai;
  if (av.dt == DT::F32) {
    aq = add_value(av.name + "@int", av.shape, want_a, Layout::PLAIN);
    Dims4 d{std::max<int64_t>(av.numel(), 0), 1, 1, 1};
    TensorRef ta{nullptr, DT::F32, Layout::PLAIN, d}, tb{nullptr, want_a, Layout::PLAIN, d};
    Step& st = add_step(n, "lanes_to_int", 2, {ai}, {aq});
    st.work = (double)av.bytes + (double)V(aq).bytes;
    st.launch = [this, ta, tb, ai, aq](cudaStream_t s) {
      k::convert(bound(ta, ai), bound(tb, aq), s);
      C.counters.glue_launches++;
      C.counters.kernel_launches++;
    };
  }
  c.x_vi = aq;
  if (is_mi) {
    c.epi.mode = k::EPI_INT32;
    c.epi.out_dt = DT::I32;
    // The chain a dynamically quantised linear is exported as,
    //   MatMulInteger -> Cast(to float) -> Mul(Mul(x_scale, w_scale[N])) -> Add(bias[N]) [-> Gelu],
    // runs inside the contraction's epilogue with the same roundings (each product and sum on its own).
    if (!C.cfg().keep_intermediates && os.size() == 2) {
      auto only_user = [&](const std::string& name, const char* opn) -> int {
        if (graph_outputs_.count(name)) return -1;
        auto it = consumers_.find(name);
        if (it == consumers_.end() || it->second.size() != 1) return -1;
        const int ni2 = it->second[0].first;
        return (!skipped_[ni2] && nodes_[ni2].op == opn) ? ni2 : -1;
      };
      auto producer_of = [&](const std::string& name) -> int {
        for (size_t j = 0; j < nodes_.size(); ++j)
          for (const std::string& o : nodes_[j].outputs)
            if (o == name) return (int)j;
        return -1;
      };
      const int cast_i = only_user(n.outputs[0], "Cast");
      const int mul_i = cast_i >= 0 && nodes_[cast_i].attrs.i("to", 1) == 1 ? only_user(nodes_[cast_i].outputs[0], "Mul") : -1;
      const int add_i = mul_i >= 0 ? only_user(nodes_[mul_i].outputs[0], "Add") : -1;
      if (add_i >= 0 && nodes_[mul_i].inputs.size() == 2 && nodes_[add_i].inputs.size() == 2) {
        const NodeDef& mul = nodes_[mul_i];
        const NodeDef& add = nodes_[add_i];
        const std::string& sc_name = mul.inputs[0] == nodes_[cast_i].outputs[0] ? mul.inputs[1] : mul.inputs[0];
        const std::string& bias_name = add.inputs[0] == mul.outputs[0] ? add.inputs[1] : add.inputs[0];
        const HostTensor* bias = const_of(bias_name);
        const int sc_i = producer_of(sc_name);
        int sc_user = -1;
        if (sc_i >= 0 && !skipped_[sc_i] && nodes_[sc_i].op == "Mul" && nodes_[sc_i].inputs.size() == 2) sc_user = only_user(sc_name, "Mul");
        if (bias && (int64_t)bias->data.size() == N && S.index_.find(bias_name) == S.index_.end() && sc_user == mul_i) {
          const NodeDef& scn = nodes_[sc_i];
          for (int slot = 0; slot < 2; ++slot) {
            auto xs = S.index_.find(scn.inputs[slot]);
            const HostTensor* ws = const_of(scn.inputs[1 - slot]);
            if (xs == S.index_.end() || !ws || (int64_t)ws->data.size() != N || S.index_.count(scn.inputs[1 - slot])) continue;
            const Value& xv2 = V(xs->second);
            if (xv2.dt != DT::F32 || xv2.numel() != 1 || xv2.host != nullptr) continue;
            c.dq_xs_vi = xs->second;
            c.dq_w_scale = ws->data;
            c.dq_bias = bias->data;
            break;
          }
        }
        if (c.dq_xs_vi >= 0) {
          skipped_[cast_i] = skipped_[mul_i] = skipped_[add_i] = skipped_[sc_i] = 1;
          std::string out_name = add.outputs[0];
          c.epi.mode = k::EPI_DEQUANT;
          c.epi.out_dt = DT::F32;
          const int gelu_i = only_user(out_name, "Gelu");
          if (gelu_i >= 0 && nodes_[gelu_i].inputs.size() == 1) {
            skipped_[gelu_i] = 1;
            c.epi.dq_act = nodes_[gelu_i].attrs.s("approximate") == "tanh" ? 2 : 1;
            out_name = nodes_[gelu_i].outputs[0];
          }
          c.out_vi = add_value(out_name, os, DT::F32, Layout::PLAIN);
          c.epi.round_tf32 = feeds_contraction(out_name) ? 1 : 0;
          emit_contraction(n, c);
          return;
        }
      }
    }
    c.out_vi = add_value(n.outputs[0], os, DT::I32, Layout::PLAIN);
    emit_contraction(n, c);
    return;
  }
  auto scale_in = [&](size_t slot, const char* what) -> float {
    const HostTensor* t = const_in(n, slot);
    if (!t) OXB_DECLINE("QLinearMatMul '%s': %s is not an initializer", n.name.c_str(), what);
    if (t->data.empty()) OXB_DECLINE("QLinearMatMul: %s is empty", what);
    float v = t->data[0];
    if (!std::isfinite(v)) OXB_DECLINE("QLinearMatMul: %s must be finite", what);
    if (v == 0.0f) OXB_DECLINE("QLinearMatMul: %s scale is zero", what);
    return v;
  };
  float a_scale = scale_in(1, "a_scale"), b_scale = scale_in(4, "b_scale"), y_scale = scale_in(6, "y_scale");
  std::vector<int32_t> y_zp;
  bool y_const;
  zp_const(7, "y_zero_point", &y_zp, &y_const);
  if (!y_const) OXB_DECLINE("QLinearMatMul '%s': y_zero_point is not an initializer", n.name.c_str());
  volatile float ab = a_scale * b_scale;  // only lane 0 of b_scale is read (qlinear_matmul.rs:230,248)
  volatile float comb = ab / y_scale;
  if (!std::isfinite((float)comb)) OXB_DECLINE("QLinearMatMul: combined scale is not finite");
  c.combined.assign((size_t)N, (float)comb);
  Range r = sat_range(has_in(n, 7) ? const_in(n, 7) : nullptr, y_zp, a_zp);
  c.epi.mode = k::EPI_REQUANT;
  c.epi.y_zp = y_zp.empty() ? 0 : y_zp[0];
  c.epi.lo = r.lo;
  c.epi.hi = r.hi;
  std::string out_name = n.outputs[0];
  int relu = sole_consumer(out_name, "Relu");
  if (relu >= 0) {
    skipped_[relu] = 1;
    c.epi.relu_fused = 1;
    out_name = nodes_[relu].outputs[0];
    r.lo = std::max(r.lo, 0);
  }
  c.epi.out_dt = narrowest_int(r.lo, r.hi);
  c.out_vi = add_value(out_name, os, c.epi.out_dt, Layout::PLAIN);
  emit_contraction(n, c);
}

// ---- element-wise ----------------------------------------------------------------------------
void Planner::plan_unary(const NodeDef& n) {
  if (n.op == "Gelu") check_attrs(n, {"approximate"});
  else check_attrs(n, {});
  int xi = value_of(in_name(n, 0));
  const Value xv = V(xi);
  int op = n.op == "Relu" ? k::UN_RELU : (n.op == "Tanh" ? k::UN_TANH : ((n.op == "Silu" || n.op == "SiLU") ? k::UN_SILU : k::UN_SIGMOID));
  // Gelu: exact unless approximate == "tanh" (nn_ops/activations.rs:357-386); Erf: the same polynomial
  if (n.op == "Gelu") op = n.attrs.s("approximate") == "tanh" ? k::UN_GELU_TANH : k::UN_GELU_ERF;
  if (n.op == "Erf") op = k::UN_ERF;
  if (op != k::UN_RELU && xv.dt != DT::F32) OXB_DECLINE("%s '%s': input is not a float tensor", n.op.c_str(), n.name.c_str());
  DT odt = xv.dt;
  if (op == k::UN_RELU && xv.dt == DT::I16) odt = DT::I16;
  int yi = add_value(n.outputs[0], xv.shape, odt, xv.shape.size() == 4 ? xv.layout : Layout::PLAIN);
  Dims4 d{std::max<int64_t>(xv.numel(), 0), 1, 1, 1};
  TensorRef xr{nullptr, xv.dt, Layout::PLAIN, d}, yr{nullptr, odt, Layout::PLAIN, d};
  Step& st = add_step(n, "unary", 2, {xi}, {yi});
  st.work = (double)xv.bytes + (double)V(yi).bytes;
  st.launch = [this, xr, yr, xi, yi, op](cudaStream_t s) {
    k::unary(bound(xr, xi), bound(yr, yi), op, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

void Planner::plan_binary(const NodeDef& n, int ni) {
  (void)ni;
  check_attrs(n, {});
  if (try_plan_scaled_masked_softmax(n)) return;
  int ai = value_of(in_name(n, 0)), bi = value_of(in_name(n, 1));
  Value av = V(ai), bv = V(bi);
  if (av.dt != DT::F32 && av.dt != DT::I32) OXB_DECLINE("%s '%s': operand A is a quantised tensor", n.op.c_str(), n.name.c_str());
  if (bv.dt != DT::F32 && bv.dt != DT::I32) OXB_DECLINE("%s '%s': operand B is a quantised tensor", n.op.c_str(), n.name.c_str());
  size_t r = std::max(av.shape.size(), bv.shape.size());
  std::vector<int64_t> as(r, 1), bs(r, 1), os(r, 1);
  std::copy(av.shape.begin(), av.shape.end(), as.begin() + (r - av.shape.size()));
  std::copy(bv.shape.begin(), bv.shape.end(), bs.begin() + (r - bv.shape.size()));
  for (size_t i = 0; i < r; ++i) {
    if (as[i] != bs[i] && as[i] != 1 && bs[i] != 1) OXB_DECLINE("%s: shapes are not broadcastable", n.op.c_str());
    os[i] = (as[i] == 0 || bs[i] == 0) ? 0 : std::max(as[i], bs[i]);
  }
  Dims4 ad, bd, od;
  Layout al = Layout::PLAIN, bl = Layout::PLAIN, ol = Layout::PLAIN;
  if (as == bs) {
    // same shape: operands must share a memory order
    if (r == 4) {
      Layout want = (av.layout == Layout::NHWC || bv.layout == Layout::NHWC) ? Layout::NHWC : Layout::PLAIN;
      if (!order_free(av)) {
        ai = ensure_layout(n, ai, want);
        bi = ensure_layout(n, bi, want);
        av = V(ai);
        bv = V(bi);
      }
      ol = want;
      al = bl = want;
      ad = bd = od = Dims4{os[0], os[1], os[2], os[3]};
    } else {
      ad = bd = od = Dims4{std::max<int64_t>(prod(os), 0), 1, 1, 1};
    }
  } else if (r <= 4) {
    // broadcast: pad to rank 4 on the left; the full-size operand fixes the memory order
    std::vector<int64_t> a4(4, 1), b4(4, 1), o4(4, 1);
    std::copy(as.begin(), as.end(), a4.begin() + (4 - r));
    std::copy(bs.begin(), bs.end(), b4.begin() + (4 - r));
    std::copy(os.begin(), os.end(), o4.begin() + (4 - r));
    ad = Dims4{a4[0], a4[1], a4[2], a4[3]};
    bd = Dims4{b4[0], b4[1], b4[2], b4[3]};
    od = Dims4{o4[0], o4[1], o4[2], o4[3]};
    if (r == 4) {
      al = effective_layout(av);
      bl = effective_layout(bv);
      bool a_full = as == os, b_full = bs == os;
      ol = a_full ? al : (b_full ? bl : Layout::PLAIN);
      // a small operand whose own order is free ([N,C,1,1], [1,C,1,1], scalar) reads the same either way
      if (order_free(av)) al = ol;
      if (order_free(bv)) bl = ol;
    }
  } else {
    OXB_DECLINE("%s '%s': broadcasting above rank 4", n.op.c_str(), n.name.c_str());
  }
  int op = n.op == "Add" ? k::BIN_ADD : (n.op == "Sub" ? k::BIN_SUB : (n.op == "Mul" ? k::BIN_MUL : k::BIN_DIV));
  std::string out_name = n.outputs[0];
  int relu_after = 0;
  int relu = sole_consumer(out_name, "Relu");
  if (relu >= 0) {
    skipped_[relu] = 1;
    relu_after = 1;
    out_name = nodes_[relu].outputs[0];
  }
  int yi = add_value(out_name, os, DT::F32, r == 4 ? ol : Layout::PLAIN);
  int rt = feeds_contraction(out_name) ? 1 : 0;
  TensorRef ar{nullptr, av.dt, al, ad}, br{nullptr, bv.dt, bl, bd}, yr{nullptr, DT::F32, r == 4 ? ol : Layout::PLAIN, od};
  Step& st = add_step(n, relu_after ? "binary+relu" : "binary", 2, {ai, bi}, {yi});
  // a plain Add of two f32 tensors of one shape in the logical order may be absorbed by a LayerNormalization that
  // is its only reader (plan_layer_norm)
  last_add_ = LastAdd{};
  if (op == k::BIN_ADD && !relu_after && !rt && as == bs && (r != 4 || (order_free(av) && order_free(bv))) && av.dt == DT::F32 && bv.dt == DT::F32)
    last_add_ = LastAdd{(int)S.steps_.size() - 1, ai, bi, yi};
  st.work = (double)av.bytes + (double)bv.bytes + (double)V(yi).bytes;
  st.launch = [this, ar, br, yr, ai, bi, yi, op, relu_after, rt](cudaStream_t s) {
    k::binary(bound(ar, ai), bound(br, bi), bound(yr, yi), op, relu_after, rt, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

void Planner::plan_prelu(const NodeDef& n) {
  check_attrs(n, {});
  int xi = value_of(in_name(n, 0));
  const Value xv = V(xi);
  const HostTensor* slope = const_in(n, 1);
  if (!slope) OXB_DECLINE("PRelu '%s': slope is not an initializer", n.name.c_str());
  if (xv.dt != DT::F32) OXB_DECLINE("PRelu '%s': input is not a float tensor", n.name.c_str());
  int64_t ns = slope->numel();
  bool per_channel = xv.shape.size() >= 2 && ns == xv.shape[1] && ns > 1;
  if (per_channel) {
    // slope must be [C], [C,1,1] or [1,C,1,1]: one value per channel and nothing else
    int64_t nontrivial = 0;
    for (int64_t d : slope->shape) nontrivial += d != 1;
    if (nontrivial != 1) per_channel = false;
    if (slope->shape.size() == 1 && xv.shape.size() != 2 && xv.shape.size() != 1) per_channel = false;  // [C] broadcasts along the last axis
  }
  if (!(ns == 1 || per_channel)) OXB_DECLINE("PRelu '%s': slope shape is neither scalar nor per-channel", n.name.c_str());
  const float* dsl = (const float*)C.resident_form(in_name(n, 1), "raw_f32", slope->data.size() * 4,
                                                   [slope](void* p) { std::memcpy(p, slope->data.data(), slope->data.size() * 4); },
                                                   cacheable_const(in_name(n, 1)));
  int yi = add_value(n.outputs[0], xv.shape, DT::F32, xv.shape.size() == 4 ? xv.layout : Layout::PLAIN);
  TensorRef xr = ref_of(xi), yr = ref_of(yi);
  Step& st = add_step(n, "prelu", 2, {xi}, {yi});
  st.work = 2.0 * (double)xv.bytes;
  st.launch = [this, xr, yr, xi, yi, dsl, ns](cudaStream_t s) {
    k::prelu(bound(xr, xi), bound(yr, yi), dsl, ns, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

void Planner::plan_max_pool(const NodeDef& n) {
  check_attrs(n, {"kernel_shape", "strides", "pads", "dilations", "auto_pad", "ceil_mode", "storage_order"});
  if (n.outputs.size() > 1 && !n.outputs[1].empty()) OXB_DECLINE("MaxPool '%s': the Indices output", n.name.c_str());
  if (n.attrs.i("storage_order", 0) != 0) OXB_DECLINE("MaxPool '%s': column-major storage order", n.name.c_str());
  int xi = value_of(in_name(n, 0));
  if (V(xi).shape.size() != 4) OXB_DECLINE("MaxPool '%s': only rank-4 inputs are claimed", n.name.c_str());
  if (!(V(xi).dt == DT::F32 || V(xi).dt == DT::U8 || V(xi).dt == DT::I8)) OXB_DECLINE("MaxPool '%s': storage type", n.name.c_str());
  auto ks = n.attrs.int_list("kernel_shape");
  if (ks.size() < 2) OXB_DECLINE("MaxPool: kernel_shape requires 2 spatial dims, got %zu", ks.size());
  if (ks[0] < 1 || ks[1] < 1) OXB_DECLINE("MaxPool: kernel_shape must be >= 1");
  Geo g = resolve_geometry("MaxPool", n.attrs, V(xi).shape.data() + 2, ks.data(), 2, n.attrs.i("ceil_mode", 0) != 0);
  xi = ensure_layout(n, xi, Layout::NHWC);
  const Value xv = V(xi);
  std::vector<int64_t> os = {xv.shape[0], xv.shape[1], g.out_spatial[0], g.out_spatial[1]};
  int yi = add_value(n.outputs[0], os, xv.dt, Layout::NHWC);
  k::PoolShape ps{(int)ks[0], (int)ks[1], (int)g.strides[0], (int)g.strides[1], (int)g.pads[0], (int)g.pads[1], (int)g.dilations[0], (int)g.dilations[1],
                  (int)g.out_spatial[0], (int)g.out_spatial[1]};
  TensorRef xr = ref_of(xi), yr = ref_of(yi);
  xr.layout = yr.layout = Layout::NHWC;
  Step& st = add_step(n, "max_pool", 2, {xi}, {yi});
  st.work = (double)xv.bytes + (double)V(yi).bytes;
  st.launch = [this, xr, yr, xi, yi, ps](cudaStream_t s) {
    k::max_pool(bound(xr, xi), bound(yr, yi), ps, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

void Planner::plan_global_avg_pool(const NodeDef& n) {
  check_attrs(n, {});
  int xi = value_of(in_name(n, 0));
  if (V(xi).shape.size() != 4 || V(xi).dt != DT::F32) OXB_DECLINE("GlobalAveragePool '%s': needs a rank-4 float input", n.name.c_str());
  {
    // DequantizeLinear (per tensor) -> GlobalAveragePool with no other reader of the f32 tensor: the pool reads the
    // 8-bit lanes and dequantises on the fly, same operations in the same order, and the f32 tensor is never written
    const Value dv = V(xi);
    auto it = consumers_.find(dv.name);
    if (dv.dq_src >= 0 && dv.dq_step == (int)S.steps_.size() - 1 && !C.cfg().keep_intermediates && !graph_outputs_.count(dv.name) &&
        it != consumers_.end() && it->second.size() == 1 && effective_layout(V(dv.dq_src)) == Layout::NHWC && V(dv.dq_src).shape[1] % 4 == 0) {
      const int src = dv.dq_src;
      S.steps_.pop_back();
      V(xi).producer = -1;
      const Value sv = V(src);
      std::vector<int64_t> os = {sv.shape[0], sv.shape[1], 1, 1};
      int yi = add_value(n.outputs[0], os, DT::F32, Layout::NHWC);
      int rt = feeds_contraction(n.outputs[0]) ? 1 : 0;
      TensorRef xr = ref_of(src), yr = ref_of(yi);
      xr.layout = Layout::NHWC;
      const float sc = dv.dq_scale, zp = dv.dq_zp;
      Step& st = add_step(n, "dequantize+global_avg_pool", 2, {src}, {yi});
      st.work = (double)sv.bytes + (double)V(yi).bytes;
      st.launch = [this, xr, yr, src, yi, sc, zp, rt](cudaStream_t s) {
        k::global_avg_pool_dequant(bound(xr, src), bound(yr, yi), sc, zp, rt, s);
        C.counters.glue_launches++;
        C.counters.kernel_launches++;
      };
      return;
    }
  }
  xi = ensure_layout(n, xi, Layout::NHWC);
  const Value xv = V(xi);
  std::vector<int64_t> os = {xv.shape[0], xv.shape[1], 1, 1};
  int yi = add_value(n.outputs[0], os, DT::F32, Layout::NHWC);
  int rt = feeds_contraction(n.outputs[0]) ? 1 : 0;
  TensorRef xr = ref_of(xi), yr = ref_of(yi);
  xr.layout = Layout::NHWC;
  Step& st = add_step(n, "global_avg_pool", 2, {xi}, {yi});
  st.work = (double)xv.bytes + (double)V(yi).bytes;
  st.launch = [this, xr, yr, xi, yi, rt](cudaStream_t s) {
    k::global_avg_pool(bound(xr, xi), bound(yr, yi), rt, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

void Planner::plan_instance_norm(const NodeDef& n) {
  check_attrs(n, {"epsilon"});
  int xi = value_of(in_name(n, 0));
  if (V(xi).shape.size() != 4 || V(xi).dt != DT::F32) OXB_DECLINE("OxiInstanceNorm '%s': needs a rank-4 float input", n.name.c_str());
  xi = ensure_layout(n, xi, Layout::NHWC);
  const Value xv = V(xi);
  float eps = n.attrs.f("epsilon", 1e-5f);
  // AdaIN: OxiInstanceNorm -> Mul(scale[N,C,1,1]) -> Add(shift[N,C,1,1]) [-> Relu], the per-sample
  // modulation the optimizer leaves as separate nodes (src/optimizer/fusion/instance_norm.rs:23-26),
  // runs inside the normalisation's third pass with the same roundings.
  std::string out_name = n.outputs[0];
  int scale_vi = -1, shift_vi = -1, relu = 0;
  if (!C.cfg().keep_intermediates) {
    auto modulator = [&](const char* op) -> int {
      if (graph_outputs_.count(out_name)) return -1;
      auto it = consumers_.find(out_name);
      if (it == consumers_.end() || it->second.size() != 1) return -1;
      const int ni = it->second[0].first, slot = it->second[0].second;
      const NodeDef& m = nodes_[ni];
      if (skipped_[ni] || m.op != op || m.inputs.size() != 2 || slot > 1 || !m.attrs.names().empty()) return -1;
      auto other = S.index_.find(m.inputs[1 - slot]);
      if (other == S.index_.end()) return -1;
      const Value& ov = V(other->second);
      const std::vector<int64_t> want = {xv.shape[0], xv.shape[1], 1, 1};
      if (ov.dt != DT::F32 || ov.shape != want || ov.host != nullptr) return -1;
      skipped_[ni] = 1;
      out_name = m.outputs[0];
      return other->second;
    };
    scale_vi = modulator("Mul");
    if (scale_vi >= 0) shift_vi = modulator("Add");
    if (scale_vi >= 0) {
      const int relu_i = sole_consumer(out_name, "Relu");
      if (relu_i >= 0) {
        skipped_[relu_i] = 1;
        relu = 1;
        out_name = nodes_[relu_i].outputs[0];
      }
    }
  }
  const int rt = scale_vi >= 0 && feeds_contraction(out_name) ? 1 : 0;
  int yi = add_value(out_name, xv.shape, DT::F32, Layout::NHWC);
  TensorRef xr = ref_of(xi), yr = ref_of(yi);
  xr.layout = yr.layout = Layout::NHWC;
  std::vector<int> reads = {xi};
  if (scale_vi >= 0) reads.push_back(scale_vi);
  if (shift_vi >= 0) reads.push_back(shift_vi);
  Step& st = add_step(n, scale_vi >= 0 ? "instance_norm+adain" : "instance_norm", 2, reads, {yi});
  st.work = 3.0 * (double)xv.bytes;
  st.launch = [this, xr, yr, xi, yi, eps, scale_vi, shift_vi, relu, rt](cudaStream_t s) {
    k::instance_norm(bound(xr, xi), bound(yr, yi), eps, scale_vi >= 0 ? (const float*)V(scale_vi).ptr : nullptr,
                     shift_vi >= 0 ? (const float*)V(shift_vi).ptr : nullptr, relu, rt, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

void Planner::plan_resize(const NodeDef& n) {
  check_attrs(n, {"mode", "coordinate_transformation_mode", "nearest_mode", "antialias", "cubic_coeff_a", "exclude_outside", "extrapolation_value",
                  "keep_aspect_ratio_policy"});
  if (n.attrs.i("antialias", 0) != 0 || n.attrs.i("exclude_outside", 0) != 0) OXB_DECLINE("Resize '%s': antialias / exclude_outside", n.name.c_str());
  int xi = value_of(in_name(n, 0));
  if (V(xi).shape.size() != 4 || V(xi).dt != DT::F32) OXB_DECLINE("Resize '%s': needs a rank-4 float input", n.name.c_str());
  if (has_in(n, 1) && const_in(n, 1) && !const_in(n, 1)->data.empty()) OXB_DECLINE("Resize '%s': roi", n.name.c_str());
  const HostTensor* scales = has_in(n, 2) ? const_in(n, 2) : nullptr;
  const HostTensor* sizes = has_in(n, 3) ? const_in(n, 3) : nullptr;
  if ((has_in(n, 2) && !scales) || (has_in(n, 3) && !sizes)) OXB_DECLINE("Resize '%s': scales / sizes are not initializers", n.name.c_str());
  std::string mode = n.attrs.s("mode"), coord = n.attrs.s("coordinate_transformation_mode"), nearest = n.attrs.s("nearest_mode");
  int m = (mode.empty() || mode == "nearest") ? 0 : ((mode == "linear" || mode == "bilinear") ? 1 : -1);
  int cm = (coord.empty() || coord == "half_pixel") ? 0 : (coord == "pytorch_half_pixel" ? 1 : (coord == "asymmetric" ? 2 : (coord == "align_corners" ? 3 : -1)));
  int nr = (nearest.empty() || nearest == "round_prefer_floor") ? 0 : (nearest == "floor" ? 1 : (nearest == "ceil" ? 2 : (nearest == "round_prefer_ceil" ? 3 : -1)));
  if (m < 0 || cm < 0 || nr < 0) OXB_DECLINE("Resize '%s': mode combination not claimed", n.name.c_str());
  xi = ensure_layout(n, xi, Layout::NHWC);
  const Value xv = V(xi);
  std::vector<int64_t> os = xv.shape;
  float sc[4] = {1, 1, 1, 1};
  if (scales && scales->data.size() == 4) {
    for (int d = 0; d < 4; ++d) {
      sc[d] = scales->data[d];
      os[d] = (int64_t)std::floor((float)xv.shape[d] * sc[d]);
    }
  } else if (sizes && sizes->data.size() == 4) {
    for (int d = 0; d < 4; ++d) {
      os[d] = (int64_t)sizes->data[d];
      sc[d] = (float)os[d] / (float)xv.shape[d];
    }
  } else {
    OXB_DECLINE("Resize '%s': needs 4 scales or 4 sizes", n.name.c_str());
  }
  if (os[0] != xv.shape[0] || os[1] != xv.shape[1]) OXB_DECLINE("Resize '%s': only the spatial axes may change", n.name.c_str());
  int yi = add_value(n.outputs[0], os, DT::F32, Layout::NHWC);
  TensorRef xr = ref_of(xi), yr = ref_of(yi);
  xr.layout = yr.layout = Layout::NHWC;
  float shh = sc[2], sww = sc[3];
  // nearest-neighbour resizing only selects lanes: a TF32-rounded input stays rounded (tf32_ready looks for the name)
  Step& st = add_step(n, m == 0 ? "resize_nearest" : "resize", 2, {xi}, {yi});
  st.work = (double)xv.bytes + (double)V(yi).bytes;
  const int rt = (m == 1 && feeds_contraction(n.outputs[0])) ? 1 : 0;  // interpolated lanes are new values: round them here
  st.launch = [this, xr, yr, xi, yi, m, cm, nr, shh, sww, rt](cudaStream_t s) {
    k::resize(bound(xr, xi), bound(yr, yi), m, cm, nr, shh, sww, rt, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

void Planner::plan_pad(const NodeDef& n) {
  check_attrs(n, {"mode", "pads", "value"});
  int xi = value_of(in_name(n, 0));
  const Value xv = V(xi);
  if (xv.shape.size() != 4) OXB_DECLINE("Pad '%s': only rank-4 inputs are claimed", n.name.c_str());
  std::vector<int64_t> pads;
  if (has_in(n, 1)) {
    const HostTensor* p = const_in(n, 1);
    if (!p) OXB_DECLINE("Pad '%s': pads is not an initializer", n.name.c_str());
    for (float f : p->data) pads.push_back((int64_t)f);
  } else {
    pads = n.attrs.int_list("pads");
  }
  if (has_in(n, 3)) OXB_DECLINE("Pad '%s': axes input", n.name.c_str());
  if (pads.size() != 8) OXB_DECLINE("Pad: pads must have 2*rank entries");
  float value = n.attrs.f("value", 0.f);
  if (has_in(n, 2)) {
    const HostTensor* v = const_in(n, 2);
    if (!v) OXB_DECLINE("Pad '%s': constant value is not an initializer", n.name.c_str());
    if (!v->data.empty()) value = v->data[0];
  }
  std::string mode = n.attrs.s("mode");
  int m = (mode.empty() || mode == "constant") ? 0 : (mode == "reflect" ? 1 : (mode == "edge" ? 2 : -1));
  if (m < 0) OXB_DECLINE("Pad '%s': mode '%s'", n.name.c_str(), mode.c_str());
  std::vector<int64_t> os = xv.shape;
  for (int d = 0; d < 4; ++d) {
    if (pads[d] < 0 || pads[d + 4] < 0) OXB_DECLINE("Pad '%s': negative pads", n.name.c_str());
    if (m == 1 && (pads[d] >= xv.shape[d] || pads[d + 4] >= xv.shape[d]) && (pads[d] > 0 || pads[d + 4] > 0)) OXB_DECLINE("Pad: reflect pad must be smaller than the axis extent");
    os[d] += pads[d] + pads[d + 4];
  }
  int yi = add_value(n.outputs[0], os, xv.dt, xv.layout);
  TensorRef xr = ref_of(xi), yr = ref_of(yi);
  int pn = (int)pads[0], pc = (int)pads[1], ph = (int)pads[2], pw = (int)pads[3];
  Step& st = add_step(n, "pad", 2, {xi}, {yi});
  st.work = (double)xv.bytes + (double)V(yi).bytes;
  st.launch = [this, xr, yr, xi, yi, m, value, pn, pc, ph, pw](cudaStream_t s) {
    k::pad(bound(xr, xi), bound(yr, yi), m, value, pn, pc, ph, pw, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

void Planner::plan_concat(const NodeDef& n) {
  check_attrs(n, {"axis"});
  if (n.inputs.empty()) OXB_DECLINE("Concat: no inputs");
  std::vector<int> ins;
  for (size_t i = 0; i < n.inputs.size(); ++i) ins.push_back(value_of(n.inputs[i]));
  const Value first = V(ins[0]);
  int64_t rank = (int64_t)first.shape.size();
  int64_t axis = n.attrs.i("axis", 0);
  if (axis < 0) axis += rank;
  if (axis < 0 || axis >= rank) OXB_DECLINE("Concat: axis out of range");
  if (rank != 4) OXB_DECLINE("Concat '%s': only rank-4 inputs are claimed", n.name.c_str());
  std::vector<int64_t> os = first.shape;
  os[axis] = 0;
  for (size_t i = 0; i < ins.size(); ++i) {
    ins[i] = ensure_layout(n, ins[i], Layout::NHWC);
    const Value& v = V(ins[i]);
    if ((int64_t)v.shape.size() != rank || v.dt != first.dt) OXB_DECLINE("Concat '%s': operands differ in rank or storage type", n.name.c_str());
    for (int64_t d = 0; d < rank; ++d)
      if (d != axis && v.shape[d] != first.shape[d]) OXB_DECLINE("Concat: non-axis dims disagree");
    os[axis] += v.shape[axis];
  }
  int yi = add_value(n.outputs[0], os, first.dt, Layout::NHWC);
  int64_t off = 0;
  for (size_t i = 0; i < ins.size(); ++i) {
    int xi = ins[i];
    TensorRef xr = ref_of(xi), yr = ref_of(yi);
    xr.layout = yr.layout = Layout::NHWC;
    int ax = (int)axis;
    int64_t o = off;
    Step& st = add_step(n, "concat", 2, {xi}, {yi});
    st.work = 2.0 * (double)V(xi).bytes;
    st.launch = [this, xr, yr, xi, yi, ax, o](cudaStream_t s) {
      k::concat_into(bound(xr, xi), bound(yr, yi), ax, o, s);
      C.counters.glue_launches++;
      C.counters.kernel_launches++;
    };
    off += V(xi).shape[axis];
  }
}

// Slice (shape_ops/concat_slice_ops.rs:27, shape/sequence.rs:52): initializer starts/ends/axes,
// unit steps, rank <= 4; runs in the logical order, the output is a plain row-major tensor.
void Planner::plan_slice(const NodeDef& n) {
  check_attrs(n, {});
  const HostTensor* st = const_in(n, 1);
  const HostTensor* en = const_in(n, 2);
  const HostTensor* ax = has_in(n, 3) ? const_in(n, 3) : nullptr;
  const HostTensor* sp = has_in(n, 4) ? const_in(n, 4) : nullptr;
  if (!st || !en || (has_in(n, 3) && !ax) || (has_in(n, 4) && !sp)) OXB_DECLINE("Slice '%s': starts / ends / axes / steps are not initializers", n.name.c_str());
  int xi = value_of(in_name(n, 0));
  const int rank = (int)V(xi).shape.size();
  if (rank < 1 || rank > 4) OXB_DECLINE("Slice '%s': only ranks 1..4 are claimed", n.name.c_str());
  const size_t cnt = st->data.size();
  if (en->data.size() != cnt || (ax && ax->data.size() != cnt) || (sp && sp->data.size() != cnt)) OXB_DECLINE("slice: starts/ends/axes/steps length mismatch");
  auto lane = [](float v) -> int64_t {
    if (std::isnan(v)) return 0;
    if (v >= 9.2233720368547758e18f) return INT64_MAX;
    if (v <= -9.2233720368547758e18f) return INT64_MIN;
    return (int64_t)v;
  };
  std::vector<int64_t> ds(rank, 0), de = V(xi).shape;
  for (size_t i = 0; i < cnt; ++i) {
    int64_t a = ax ? lane(ax->data[i]) : (int64_t)i;
    if (a < 0) a += rank;
    if (a < 0 || a >= rank) OXB_DECLINE("Slice '%s': axis out of range", n.name.c_str());
    if (sp && lane(sp->data[i]) != 1) OXB_DECLINE("Slice '%s': only unit steps are claimed", n.name.c_str());
    const int64_t dim = V(xi).shape[a];
    int64_t s0 = lane(st->data[i]), e0 = lane(en->data[i]);
    if (s0 < 0) s0 += dim;
    if (e0 < 0) e0 += dim;
    ds[a] = std::min(std::max<int64_t>(s0, 0), dim);
    de[a] = std::min(std::max<int64_t>(e0, 0), dim);
  }
  std::vector<int64_t> os(rank);
  for (int d = 0; d < rank; ++d) os[d] = de[d] <= ds[d] ? 0 : de[d] - ds[d];
  if (rank == 4 && V(xi).layout == Layout::NHWC && !order_free(V(xi))) xi = ensure_layout(n, xi, Layout::PLAIN);
  const Value xv = V(xi);
  int yi = add_value(n.outputs[0], os, xv.dt, Layout::PLAIN);
  auto pad4 = [&](const std::vector<int64_t>& v, int64_t fill) {
    Dims4 d{fill, fill, fill, fill};
    int64_t* f[4] = {&d.N, &d.C, &d.H, &d.W};
    for (int i = 0; i < rank; ++i) *f[4 - rank + i] = v[i];
    return d;
  };
  const Dims4 xd = pad4(xv.shape, 1), yd = pad4(os, 1), sd = pad4(ds, 0);
  const DT dt = xv.dt;
  Step& stp = add_step(n, "slice", 2, {xi}, {yi});
  stp.work = 2.0 * (double)V(yi).bytes;
  stp.launch = [this, xi, yi, dt, xd, yd, sd](cudaStream_t s) {
    k::slice_rows(V(xi).ptr, V(yi).ptr, dt, xd, yd, sd, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

// Gather along axis 0 of a rank-2 initializer (an embedding table) with device-resident index lanes
// (indexing/gather.rs:12-44).  Other forms are declined.
void Planner::plan_gather(const NodeDef& n) {
  check_attrs(n, {"axis"});
  const HostTensor* table = const_in(n, 0);
  if (!table || table->shape.size() != 2) OXB_DECLINE("Gather '%s': only a rank-2 initializer table is claimed", n.name.c_str());
  int64_t axis = n.attrs.i("axis", 0);
  if (axis < 0) axis += 2;
  if (axis != 0) OXB_DECLINE("Gather '%s': only axis 0 is claimed", n.name.c_str());
  int ii = value_of(in_name(n, 1));
  if (V(ii).dt != DT::F32) OXB_DECLINE("Gather '%s': indices are not f32 lanes", n.name.c_str());
  if (V(ii).shape.size() == 4 && V(ii).layout == Layout::NHWC && !order_free(V(ii))) ii = ensure_layout(n, ii, Layout::PLAIN);
  const int64_t rows = table->shape[0], inner = table->shape[1];
  std::vector<int64_t> os = V(ii).shape;
  os.push_back(inner);
  if (os.size() > 4) OXB_DECLINE("Gather '%s': output rank above 4", n.name.c_str());
  const float* dtable = (const float*)C.resident_form(in_name(n, 0), "raw_f32", table->data.size() * 4,
                                                      [table](void* p) { std::memcpy(p, table->data.data(), table->data.size() * 4); },
                                                      cacheable_const(in_name(n, 0)));
  int yi = add_value(n.outputs[0], os, DT::F32, Layout::PLAIN);
  const int64_t n_idx = V(ii).numel();
  int* err = S.err_flag_;
  Step& st = add_step(n, "gather_rows", 2, {ii}, {yi});
  st.work = 2.0 * (double)V(yi).bytes;
  st.launch = [this, ii, yi, dtable, n_idx, rows, inner, err](cudaStream_t s) {
    k::gather_rows(dtable, (const float*)V(ii).ptr, (float*)V(yi).ptr, n_idx, rows, inner, err, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

// Transpose (shape/basic.rs:146): any permutation of up to four logical axes of a 32-bit tensor.
void Planner::plan_transpose(const NodeDef& n) {
  check_attrs(n, {"perm"});
  int xi = value_of(in_name(n, 0));
  const int rank = (int)V(xi).shape.size();
  if (rank < 1 || rank > 4) OXB_DECLINE("Transpose '%s': only ranks 1..4 are claimed", n.name.c_str());
  if (dt_size(V(xi).dt) != 4) OXB_DECLINE("Transpose '%s': only 32-bit storage is claimed", n.name.c_str());
  std::vector<int64_t> perm = n.attrs.int_list("perm");
  if (perm.empty())
    for (int d = rank - 1; d >= 0; --d) perm.push_back(d);
  if ((int)perm.size() != rank) OXB_DECLINE("transpose: perm len %zu != ndim %d", perm.size(), rank);
  std::vector<char> seen(rank, 0);
  for (int64_t pv : perm) {
    if (pv < 0 || pv >= rank || seen[pv]) OXB_DECLINE("transpose: perm is not a permutation");
    seen[pv] = 1;
  }
  if (rank == 4 && V(xi).layout == Layout::NHWC && !order_free(V(xi))) xi = ensure_layout(n, xi, Layout::PLAIN);
  const Value xv = V(xi);
  std::vector<int64_t> os(rank);
  for (int d = 0; d < rank; ++d) os[d] = xv.shape[perm[d]];
  int yi = add_value(n.outputs[0], os, xv.dt, Layout::PLAIN);
  // head split in front of an attention product: defer (see LazyHeads)
  if (rank == 4 && xv.dt == DT::F32 && !C.cfg().keep_intermediates && C.cfg().kernel_path == 0 && k::umma_available() && !graph_outputs_.count(n.outputs[0])) {
    const bool p0 = perm == std::vector<int64_t>{0, 2, 1, 3}, p1 = perm == std::vector<int64_t>{0, 2, 3, 1};
    int root = xi;
    while (V(root).alias_of >= 0) root = V(root).alias_of;
    auto it = consumers_.find(n.outputs[0]);
    const bool to_matmul = it != consumers_.end() && it->second.size() == 1 && nodes_[it->second[0].first].op == "MatMul";
    const int64_t B = xv.shape[0], Sq = xv.shape[1], H = xv.shape[2], D = xv.shape[3];
    if ((p0 || p1) && to_matmul && root != xi && V(root).shape == std::vector<int64_t>{B * Sq, H * D} && V(root).host == nullptr && Sq % 128 == 0 && D % 8 == 0) {
      lazy_heads_[yi] = LazyHeads{xi, root, B, Sq, H, D, p0 ? 0 : 1, cur_node_, perm, false};
      return;
    }
  }
  emit_transpose(n, xi, perm, yi);
}

void Planner::emit_transpose(const NodeDef& n, int xi, const std::vector<int64_t>& perm, int yi) {
  const Value xv = V(xi);
  const int rank = (int)xv.shape.size();
  std::vector<int64_t> xs(rank, 1);
  for (int d = rank - 2; d >= 0; --d) xs[d] = xs[d + 1] * xv.shape[d + 1];
  const std::vector<int64_t> os = V(yi).shape;
  Dims4 yd{1, 1, 1, 1}, st4{0, 0, 0, 0};
  int64_t* yf[4] = {&yd.N, &yd.C, &yd.H, &yd.W};
  int64_t* sf[4] = {&st4.N, &st4.C, &st4.H, &st4.W};
  for (int d = 0; d < rank; ++d) {
    *yf[4 - rank + d] = os[d];
    *sf[4 - rank + d] = xs[perm[d]];
  }
  Step& st = add_step(n, "transpose_perm", 2, {xi}, {yi});
  st.work = 2.0 * (double)xv.bytes;
  st.launch = [this, xi, yi, yd, st4](cudaStream_t s) {
    k::transpose_perm(V(xi).ptr, V(yi).ptr, yd, st4, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

void Planner::materialise_heads(int yi) {
  auto it = lazy_heads_.find(yi);
  if (it == lazy_heads_.end() || it->second.materialised) return;
  it->second.materialised = true;
  emit_transpose(nodes_[it->second.node], it->second.src_vi, it->second.perm, yi);
}

// The two products of an attention layer on the tensor cores (TF32), batched over (batch, head):
//   scores[b,h] = Q[b,h] (S x D) . K[b,h]^T         Q and K read as column windows of their [B*S, H*D] matrices
//   ctx[b,h]    = probs[b,h] (S x S) . V[b,h] (S x D)  V transposed once to [B,H,D,S]; the context is written
//                                                      straight into [B*S, H*D] when a head merge follows
bool Planner::try_plan_attention_product(const NodeDef& n, int ai, int bi) {
  auto la = lazy_heads_.find(ai), lb = lazy_heads_.find(bi);
  const bool a_lazy = la != lazy_heads_.end() && !la->second.materialised, b_lazy = lb != lazy_heads_.end() && !lb->second.materialised;
  if (!b_lazy) return false;
  const LazyHeads hb = lb->second;
  const int64_t B = hb.B, Sq = hb.S, H = hb.H, D = hb.D;
  if (B * H * Sq > 0x7fffffffLL || H * D > 0x7fffffffLL) return false;
  k::BatchedGemm g;
  g.outer = (int)B, g.inner = (int)H;
  std::vector<int> reads;
  int out_vi = -1;
  std::string label;
  if (a_lazy && la->second.kind == 0 && hb.kind == 1 && la->second.B == B && la->second.S == Sq && la->second.H == H && la->second.D == D) {
    if (try_plan_fused_attention(n, ai, bi)) return true;
    // scores
    g.M = (int)Sq, g.N = (int)Sq, g.K = (int)D;
    g.a_rows = B * Sq, g.a_cols = H * D, g.a_rb = (int)Sq, g.a_rh = 0, g.a_ch = (int)D;
    g.b_rows = B * Sq, g.b_cols = H * D, g.b_rb = (int)Sq, g.b_rh = 0, g.b_ch = (int)D;
    g.o_rows = B * H * Sq, g.o_cols = Sq, g.o_rb = (int)(H * Sq), g.o_rh = (int)Sq, g.o_ch = 0;
    out_vi = add_value(n.outputs[0], {B, H, Sq, Sq}, DT::F32, Layout::PLAIN);
    g.round_tf32 = feeds_contraction(n.outputs[0]) ? 1 : 0;
    reads = {la->second.root_vi, hb.root_vi};
    label = "scores";
  } else if (!a_lazy && hb.kind == 0 && V(ai).dt == DT::F32 && V(ai).shape == std::vector<int64_t>{B, H, Sq, Sq} && V(ai).layout == Layout::PLAIN &&
             V(ai).host == nullptr) {
    // context: V^T per head first
    const int vt = add_value(V(hb.src_vi).name + "@heads_t", {B, H, D, Sq}, DT::F32, Layout::PLAIN);
    emit_transpose(nodes_[hb.node], hb.src_vi, {0, 2, 3, 1}, vt);
    g.M = (int)Sq, g.N = (int)D, g.K = (int)Sq;
    g.a_rows = B * H * Sq, g.a_cols = Sq, g.a_rb = (int)(H * Sq), g.a_rh = (int)Sq, g.a_ch = 0;
    g.b_rows = B * H * D, g.b_cols = Sq, g.b_rb = (int)(H * D), g.b_rh = (int)D, g.b_ch = 0;
    // a head merge Transpose(0,2,1,3) -> Reshape([B*S, H*D]) behind the product is absorbed into the store
    std::string out_name = n.outputs[0];
    std::vector<int64_t> oshape = {B, H, Sq, D};
    g.o_rows = B * H * Sq, g.o_cols = D, g.o_rb = (int)(H * Sq), g.o_rh = (int)Sq, g.o_ch = 0;
    auto only_user = [&](const std::string& name, const char* opn) -> int {
      if (graph_outputs_.count(name)) return -1;
      auto it = consumers_.find(name);
      if (it == consumers_.end() || it->second.size() != 1) return -1;
      const int ni2 = it->second[0].first;
      return (!skipped_[ni2] && nodes_[ni2].op == opn && it->second[0].second == 0) ? ni2 : -1;
    };
    const int t_i = only_user(out_name, "Transpose");
    if (t_i >= 0 && nodes_[t_i].attrs.int_list("perm") == std::vector<int64_t>{0, 2, 1, 3}) {
      const int r_i = only_user(nodes_[t_i].outputs[0], "Reshape");
      const HostTensor* sh = r_i >= 0 ? const_in(nodes_[r_i], 1) : nullptr;
      if (sh && sh->data.size() == 2 && (int64_t)sh->data[0] == B * Sq && (int64_t)sh->data[1] == H * D) {
        skipped_[t_i] = skipped_[r_i] = 1;
        out_name = nodes_[r_i].outputs[0];
        oshape = {B * Sq, H * D};
        g.o_rows = B * Sq, g.o_cols = H * D, g.o_rb = (int)Sq, g.o_rh = 0, g.o_ch = (int)D;
      }
    }
    out_vi = add_value(out_name, oshape, DT::F32, Layout::PLAIN);
    g.round_tf32 = feeds_contraction(out_name) ? 1 : 0;
    reads = {ai, vt};
    lb->second.materialised = true;  // consumed through its transposed copy
    label = "context";
  } else {
    return false;
  }
  if (label == "scores") la->second.materialised = lb->second.materialised = true;
  g.zero_bias = upload_vec(std::vector<float>(align_up((size_t)g.N, 256), 0.f));
  Step& st = add_step(n, "umma", 0, reads, {out_vi});
  st.work = 2.0 * (double)B * H * g.M * g.N * g.K;
  st.work_is_bytes = false;
  const int step_index = (int)S.steps_.size() - 1;
  const int ra = reads[0], rb = reads[1];
  st.finalize = [this, step_index, g, ra, rb, out_vi, n]() mutable {
    k::BatchedGemm gg = g;
    gg.a = V(ra).ptr;
    gg.b = V(rb).ptr;
    gg.out = V(out_vi).ptr;
    gg.minmax_keys = (unsigned int*)V(out_vi).minmax_keys;
    std::string why2;
    k::UmmaPlan* plan = k::umma_plan_create_batched(gg, &why2);
    if (!plan) OXB_FAIL("MatMul '%s': batched tensor-core plan rejected: %s", n.name.c_str(), why2.c_str());
    S.umma_plans_.push_back(plan);
    Step& me = S.steps_[step_index];
    me.kernel = k::umma_plan_desc(plan);
    int* err = S.err_flag_;
    me.launch = [this, plan, err](cudaStream_t s) {
      k::umma_launch(plan, err, s);
      C.counters.umma_launches++;
      C.counters.kernel_launches++;
    };
  };
  return true;
}

// MatMul(Q heads, K heads^T) -> Mul(scalar) -> Add(mask[B,1,1,S]) -> Softmax -> MatMul(., V heads) [-> head merge] for
// sequences of 128 positions and heads of 64 lanes, none of the intermediates read by anything else: one kernel
// (umma_attention.cu).  The five or seven nodes are marked done; V is transposed per head first, as for the
// separate context product.
bool Planner::try_plan_fused_attention(const NodeDef& n, int qi, int ki) {
  if (C.cfg().keep_intermediates || C.cfg().kernel_path != 0 || !k::umma_available()) return false;
  const LazyHeads hq = lazy_heads_.find(qi)->second, hk = lazy_heads_.find(ki)->second;
  const int64_t B = hq.B, Sq = hq.S, H = hq.H, D = hq.D;
  if (Sq != 128 || D != 64 || B * H > 0x3fffffffLL) return false;
  auto only_user = [&](const std::string& name, const char* opn) -> int {
    if (graph_outputs_.count(name)) return -1;
    auto it = consumers_.find(name);
    if (it == consumers_.end() || it->second.size() != 1) return -1;
    const int ni2 = it->second[0].first;
    return (!skipped_[ni2] && nodes_[ni2].op == opn) ? ni2 : -1;
  };
  // Mul by a scalar initializer
  const int mul_i = only_user(n.outputs[0], "Mul");
  if (mul_i < 0 || nodes_[mul_i].inputs.size() != 2 || !nodes_[mul_i].attrs.names().empty()) return false;
  const NodeDef& mul = nodes_[mul_i];
  const int s_slot = mul.inputs[0] == n.outputs[0] ? 1 : 0;
  const HostTensor* sc = const_of(mul.inputs[s_slot]);
  if (!sc || sc->data.size() != 1 || S.index_.count(mul.inputs[s_slot])) return false;
  // Add of a mask [B,1,1,S]
  const int add_i = only_user(mul.outputs[0], "Add");
  if (add_i < 0 || nodes_[add_i].inputs.size() != 2) return false;
  const NodeDef& add = nodes_[add_i];
  const std::string& mask_name = add.inputs[0] == mul.outputs[0] ? add.inputs[1] : add.inputs[0];
  auto mit = S.index_.find(mask_name);
  if (mit == S.index_.end()) return false;
  const int mi = mit->second;
  if (V(mi).shape != std::vector<int64_t>{B, 1, 1, Sq} || V(mi).dt != DT::F32) return false;
  // Softmax over the last axis
  const int sm_i = only_user(add.outputs[0], "Softmax");
  if (sm_i < 0) return false;
  int64_t axis = nodes_[sm_i].attrs.i("axis", -1);
  if (axis < 0) axis += 4;
  if (axis != 3) return false;
  // MatMul(probabilities, V heads)
  const int av_i = only_user(nodes_[sm_i].outputs[0], "MatMul");
  if (av_i < 0 || nodes_[av_i].inputs.size() != 2 || nodes_[av_i].inputs[0] != nodes_[sm_i].outputs[0]) return false;
  auto vit = S.index_.find(nodes_[av_i].inputs[1]);
  if (vit == S.index_.end()) return false;
  auto lv = lazy_heads_.find(vit->second);
  if (lv == lazy_heads_.end() || lv->second.materialised || lv->second.kind != 0) return false;
  const LazyHeads hv = lv->second;
  if (hv.B != B || hv.S != Sq || hv.H != H || hv.D != D) return false;
  // a head merge Transpose(0,2,1,3) -> Reshape([B*S, H*D]) behind the product is absorbed into the store
  const NodeDef& av = nodes_[av_i];
  std::string out_name = av.outputs[0];
  std::vector<int64_t> oshape = {B, H, Sq, D};
  int o_rb = (int)(H * Sq), o_rh = (int)Sq, o_ch = 0;
  int64_t o_rows = B * H * Sq, o_cols = D;
  int t_i = only_user(out_name, "Transpose"), r_i = -1;
  if (t_i >= 0 && nodes_[t_i].attrs.int_list("perm") == std::vector<int64_t>{0, 2, 1, 3}) {
    r_i = only_user(nodes_[t_i].outputs[0], "Reshape");
    const HostTensor* sh = r_i >= 0 ? const_in(nodes_[r_i], 1) : nullptr;
    if (sh && sh->data.size() == 2 && (int64_t)sh->data[0] == B * Sq && (int64_t)sh->data[1] == H * D) {
      out_name = nodes_[r_i].outputs[0];
      oshape = {B * Sq, H * D};
      o_rows = B * Sq, o_cols = H * D, o_rb = (int)Sq, o_rh = 0, o_ch = (int)D;
    } else {
      t_i = r_i = -1;
    }
  } else {
    t_i = -1;
  }
  // from here on the plan is committed
  const float* dscale = (const float*)C.resident_form(mul.inputs[s_slot], "raw_f32", 4, [sc](void* p) { std::memcpy(p, sc->data.data(), 4); },
                                                      cacheable_const(mul.inputs[s_slot]));
  const int vt = add_value(V(hv.src_vi).name + "@heads_t", {B, H, D, Sq}, DT::F32, Layout::PLAIN);
  emit_transpose(nodes_[hv.node], hv.src_vi, {0, 2, 3, 1}, vt);
  skipped_[mul_i] = skipped_[add_i] = skipped_[sm_i] = skipped_[av_i] = 1;
  if (t_i >= 0) skipped_[t_i] = skipped_[r_i] = 1;
  lazy_heads_.find(qi)->second.materialised = lazy_heads_.find(ki)->second.materialised = lv->second.materialised = true;
  const int out_vi = add_value(out_name, oshape, DT::F32, Layout::PLAIN);
  const int q_root = hq.root_vi, k_root = hk.root_vi;
  Step& st = add_step(av, "umma", 0, {q_root, k_root, vt, mi}, {out_vi});
  st.work = 4.0 * (double)B * H * Sq * Sq * D;
  st.work_is_bytes = false;
  const int step_index = (int)S.steps_.size() - 1;
  const std::string av_name = av.name;
  st.finalize = [this, step_index, q_root, k_root, vt, mi, out_vi, dscale, B, H, Sq, D, o_rows, o_cols, o_rb, o_rh, o_ch, av_name]() {
    k::FusedAttention fa;
    fa.q = (const float*)V(q_root).ptr;
    fa.k = (const float*)V(k_root).ptr;
    fa.vt = (const float*)V(vt).ptr;
    fa.out = (float*)V(out_vi).ptr;
    fa.o_rows = o_rows, fa.o_cols = o_cols, fa.o_rb = o_rb, fa.o_rh = o_rh, fa.o_ch = o_ch;
    fa.B = (int)B, fa.H = (int)H, fa.S = (int)Sq, fa.D = (int)D;
    fa.scale = dscale;
    fa.mask = (const float*)V(mi).ptr;
    fa.round_probs = 1;
    fa.minmax_keys = (unsigned int*)V(out_vi).minmax_keys;
    std::string why2;
    k::UmmaAttentionPlan* plan = k::umma_attention_create(fa, &why2);
    if (!plan) OXB_FAIL("MatMul '%s': fused attention plan rejected: %s", av_name.c_str(), why2.c_str());
    S.umma_attentions_.push_back(plan);
    Step& me = S.steps_[step_index];
    me.kernel = k::umma_attention_desc(plan);
    int* err = S.err_flag_;
    me.launch = [this, plan, err](cudaStream_t s) {
      k::umma_attention_launch(plan, err, s);
      C.counters.umma_launches++;
      C.counters.kernel_launches++;
    };
  };
  return true;
}

// Softmax over the last axis (nn/normalization.rs softmax_into); other axes are declined.
// Mul(x, scalar) -> Add(., mask[B,1,1,S]) -> Softmax(last axis) over x[B,H,Q,S]: the attention-score chain.  The
// softmax kernel applies the product and the sum (rounded as the nodes would) while it reads its input.
bool Planner::try_plan_scaled_masked_softmax(const NodeDef& n) {
  if (C.cfg().keep_intermediates || n.op != "Mul" || n.inputs.size() != 2 || !n.attrs.names().empty()) return false;
  int slot = -1;
  for (int sl = 0; sl < 2; ++sl) {
    auto it = S.index_.find(n.inputs[sl]);
    const HostTensor* sc = const_of(n.inputs[1 - sl]);
    if (it != S.index_.end() && sc && sc->data.size() == 1 && !S.index_.count(n.inputs[1 - sl]) && V(it->second).shape.size() == 4 && V(it->second).dt == DT::F32 &&
        V(it->second).host == nullptr)
      slot = sl;
  }
  if (slot < 0) return false;
  const int xi0 = S.index_.find(n.inputs[slot])->second;
  if (V(xi0).layout == Layout::NHWC && !order_free(V(xi0))) return false;
  auto only_user = [&](const std::string& name, const char* opn) -> int {
    if (graph_outputs_.count(name)) return -1;
    auto it = consumers_.find(name);
    if (it == consumers_.end() || it->second.size() != 1) return -1;
    const int ni2 = it->second[0].first;
    return (!skipped_[ni2] && nodes_[ni2].op == opn) ? ni2 : -1;
  };
  const int add_i = only_user(n.outputs[0], "Add");
  if (add_i < 0 || nodes_[add_i].inputs.size() != 2) return false;
  const NodeDef& add = nodes_[add_i];
  const std::string& mask_name = add.inputs[0] == n.outputs[0] ? add.inputs[1] : add.inputs[0];
  auto mit = S.index_.find(mask_name);
  if (mit == S.index_.end()) return false;
  const std::vector<int64_t>& xs = V(xi0).shape;
  const std::vector<int64_t> want = {xs[0], 1, 1, xs[3]};
  if (V(mit->second).shape != want || V(mit->second).dt != DT::F32) return false;
  const int sm_i = only_user(add.outputs[0], "Softmax");
  if (sm_i < 0) return false;
  int64_t axis = nodes_[sm_i].attrs.i("axis", -1);
  if (axis < 0) axis += 4;
  if (axis != 3) return false;
  const float* dscale = (const float*)C.resident_form(n.inputs[1 - slot], "raw_f32", 4, [sc = const_of(n.inputs[1 - slot])](void* p) { std::memcpy(p, sc->data.data(), 4); },
                                                      cacheable_const(n.inputs[1 - slot]));
  skipped_[add_i] = skipped_[sm_i] = 1;
  const int mi = mit->second;
  const int64_t len = xs[3], rows = V(xi0).numel() / len, rows_per_mask = xs[1] * xs[2];
  int yi = add_value(nodes_[sm_i].outputs[0], xs, DT::F32, Layout::PLAIN);
  const int rt = feeds_contraction(nodes_[sm_i].outputs[0]) ? 1 : 0;
  Step& st = add_step(nodes_[sm_i], "softmax_rows+scale+mask", 2, {xi0, mi}, {yi});
  st.work = 2.0 * (double)V(xi0).bytes;
  st.launch = [this, xi0, mi, yi, rows, len, dscale, rows_per_mask, rt](cudaStream_t s) {
    k::softmax_rows((const float*)V(xi0).ptr, (float*)V(yi).ptr, rows, len, dscale, (const float*)V(mi).ptr, rows_per_mask, rt, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
  return true;
}

void Planner::plan_softmax(const NodeDef& n) {
  check_attrs(n, {"axis"});
  int xi = value_of(in_name(n, 0));
  if (V(xi).dt != DT::F32) OXB_DECLINE("Softmax '%s': input is not a float tensor", n.name.c_str());
  const int rank = (int)V(xi).shape.size();
  int64_t axis = n.attrs.i("axis", -1);
  if (axis < 0) axis += rank;
  if (rank < 1 || axis != rank - 1) OXB_DECLINE("Softmax '%s': only the last axis is claimed", n.name.c_str());
  if (rank == 4 && V(xi).layout == Layout::NHWC && !order_free(V(xi))) xi = ensure_layout(n, xi, Layout::PLAIN);
  const Value xv = V(xi);
  const int64_t len = xv.shape[rank - 1], rows = len ? xv.numel() / len : 0;
  int yi = add_value(n.outputs[0], xv.shape, DT::F32, Layout::PLAIN);
  const int rt = feeds_contraction(n.outputs[0]) ? 1 : 0;
  Step& st = add_step(n, "softmax_rows", 2, {xi}, {yi});
  st.work = 2.0 * (double)xv.bytes;
  st.launch = [this, xi, yi, rows, len, rt](cudaStream_t s) {
    k::softmax_rows((const float*)V(xi).ptr, (float*)V(yi).ptr, rows, len, nullptr, nullptr, 1, rt, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

// LayerNormalization over the last axis with initializer scale (and bias) of that length
// (nn/normalization.rs layer_norm_into, the ONNX-conformant case); other forms are declined.
void Planner::plan_layer_norm(const NodeDef& n) {
  check_attrs(n, {"axis", "epsilon", "stash_type"});
  int xi = value_of(in_name(n, 0));
  if (V(xi).dt != DT::F32) OXB_DECLINE("LayerNormalization '%s': input is not a float tensor", n.name.c_str());
  const int rank = (int)V(xi).shape.size();
  int64_t axis = n.attrs.i("axis", -1);
  if (axis < 0) axis += rank;
  if (rank < 1 || axis != rank - 1) OXB_DECLINE("LayerNormalization '%s': only the last axis is claimed", n.name.c_str());
  if (n.outputs.size() > 1 && !n.outputs[1].empty()) OXB_DECLINE("LayerNormalization '%s': mean / inv-std outputs are not produced", n.name.c_str());
  const HostTensor* scale = const_in(n, 1);
  const HostTensor* bias = has_in(n, 2) ? const_in(n, 2) : nullptr;
  if (!scale || (has_in(n, 2) && !bias)) OXB_DECLINE("LayerNormalization '%s': scale / bias are not initializers", n.name.c_str());
  if (rank == 4 && V(xi).layout == Layout::NHWC && !order_free(V(xi))) xi = ensure_layout(n, xi, Layout::PLAIN);
  const Value xv = V(xi);
  const int64_t len = xv.shape[rank - 1], rows = len ? xv.numel() / len : 0;
  if ((int64_t)scale->data.size() != len || (bias && (int64_t)bias->data.size() != len)) OXB_DECLINE("LayerNormalization '%s': scale / bias length differs from the axis", n.name.c_str());
  const float eps = n.attrs.f("epsilon", 1e-5f);
  const float* dscale = (const float*)C.resident_form(in_name(n, 1), "raw_f32", scale->data.size() * 4,
                                                      [scale](void* p) { std::memcpy(p, scale->data.data(), scale->data.size() * 4); },
                                                      cacheable_const(in_name(n, 1)));
  const float* dbias = nullptr;
  if (bias)
    dbias = (const float*)C.resident_form(in_name(n, 2), "raw_f32", bias->data.size() * 4, [bias](void* p) { std::memcpy(p, bias->data.data(), bias->data.size() * 4); },
                                          cacheable_const(in_name(n, 2)));
  // The residual Add right in front, read by nothing else: the normalisation adds the two operands while it loads
  // them (one rounded sum per lane, as the node gives) and the sum is never written.
  int x2 = -1;
  if (!C.cfg().keep_intermediates && last_add_.y == xi && last_add_.step == (int)S.steps_.size() - 1 && !graph_outputs_.count(xv.name)) {
    auto it = consumers_.find(xv.name);
    if (it != consumers_.end() && it->second.size() == 1) {
      S.steps_.pop_back();
      V(xi).producer = -1;
      x2 = last_add_.b;
      xi = last_add_.a;
    }
  }
  last_add_ = LastAdd{};
  int yi = add_value(n.outputs[0], xv.shape, DT::F32, Layout::PLAIN);
  std::vector<int> reads = {xi};
  if (x2 >= 0) reads.push_back(x2);
  Step& st = add_step(n, x2 >= 0 ? "add+layer_norm_rows" : "layer_norm_rows", 2, reads, {yi});
  st.work = (x2 >= 0 ? 3.0 : 2.0) * (double)xv.bytes;
  st.launch = [this, xi, x2, yi, rows, len, dscale, dbias, eps](cudaStream_t s) {
    k::layer_norm_rows((const float*)V(xi).ptr, (float*)V(yi).ptr, rows, len, dscale, dbias, eps, s, (unsigned int*)V(yi).minmax_keys,
                       x2 >= 0 ? (const float*)V(x2).ptr : nullptr);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
}

// Flatten / Reshape / Identity / Cast: the logical row-major order is untouched, so the output
// shares the input's storage.  A channels-last activation whose order matters is first brought
// back to the logical order; int32 lanes cast to float become f32 lanes (round to nearest even).
void Planner::plan_alias(const NodeDef& n) {
  int xi = value_of(in_name(n, 0));
  std::vector<int64_t> os;
  const Value xv0 = V(xi);
  if (n.op == "Flatten") {
    check_attrs(n, {"axis"});
    int64_t axis = n.attrs.i("axis", 1), rank = (int64_t)xv0.shape.size();
    if (axis < 0) axis += rank;
    if (axis < 0 || axis > rank) OXB_DECLINE("Flatten: axis out of range");
    int64_t outer = 1, inner = 1;
    for (int64_t d = 0; d < rank; ++d) (d < axis ? outer : inner) *= xv0.shape[d];
    os = {outer, inner};
  } else if (n.op == "Reshape") {
    check_attrs(n, {"allowzero"});
    const HostTensor* sh = const_in(n, 1);
    if (!sh) OXB_DECLINE("Reshape '%s': the shape is not an initializer", n.name.c_str());
    bool allowzero = n.attrs.i("allowzero", 0) != 0;
    int64_t known = 1;
    int infer = -1;
    for (size_t i = 0; i < sh->data.size(); ++i) {
      int64_t d = (int64_t)sh->data[i];
      if (d == -1) {
        if (infer >= 0) OXB_DECLINE("Reshape: more than one -1");
        infer = (int)i;
        os.push_back(1);
        continue;
      }
      if (d == 0 && !allowzero) {
        if (i >= xv0.shape.size()) OXB_DECLINE("Reshape: 0 dim out of range");
        d = xv0.shape[i];
      }
      os.push_back(d);
      known *= d;
    }
    if (infer >= 0) {
      if (known == 0 || xv0.numel() % known != 0) OXB_DECLINE("Reshape: cannot infer dimension");
      os[infer] = xv0.numel() / known;
      known *= os[infer];
    }
    if (known != xv0.numel()) OXB_DECLINE("Reshape: element count changes");
  } else {
    if (n.op == "Cast") check_attrs(n, {"to", "saturate"});
    else check_attrs(n, {});
    os = xv0.shape;
  }
  if (n.op == "Cast") {
    int64_t to = n.attrs.i("to", 1);
    if (to != 1) OXB_DECLINE("Cast '%s': only casts to float are claimed", n.name.c_str());
    if (xv0.dt != DT::F32) {
      // integer storage -> f32 lanes
      int yi = add_value(n.outputs[0], os, DT::F32, xv0.shape.size() == 4 ? xv0.layout : Layout::PLAIN);
      Dims4 d{std::max<int64_t>(xv0.numel(), 0), 1, 1, 1};
      TensorRef a{nullptr, xv0.dt, Layout::PLAIN, d}, b{nullptr, DT::F32, Layout::PLAIN, d};
      Step& st = add_step(n, "cast_to_f32", 2, {xi}, {yi});
      st.work = (double)xv0.bytes + (double)V(yi).bytes;
      st.launch = [this, a, b, xi, yi](cudaStream_t s) {
        k::convert(bound(a, xi), bound(b, yi), s);
        C.counters.glue_launches++;
        C.counters.kernel_launches++;
      };
      return;
    }
  }
  bool shape_changes = os != xv0.shape;
  if (shape_changes && xv0.shape.size() == 4 && xv0.layout == Layout::NHWC && !order_free(xv0)) xi = ensure_layout(n, xi, Layout::PLAIN);
  const Value xv = V(xi);
  Layout ol = Layout::PLAIN;
  if (os.size() == 4) ol = shape_changes ? Layout::PLAIN : xv.layout;
  int yi = add_value(n.outputs[0], os, xv.dt, ol);
  V(yi).alias_of = xi;
  V(yi).host = xv.host;
  if (xv.external && xv.ptr) V(yi).ptr = xv.ptr;
}

// DequantizeLinear(a) , DequantizeLinear(b) -> Add -> Relu -> QuantizeLinear with per-tensor
// parameters: the residual join of a quantised ResNet.  One kernel performs the same f32
// operations in the same order, so the lanes equal the unfused chain's bit for bit; the
// float intermediates never reach memory.
bool Planner::try_plan_residual_chain(const NodeDef& n, int ni) {
  // per-tensor parameters held by initializers: scale at slot 1, optional zero point at slot 2
  auto per_tensor = [&](const NodeDef& d, float* scale, float* zp, bool* has_zp) -> bool {
    for (const std::string& a : d.attrs.names())
      if (a != "axis") return false;
    const HostTensor* sc = const_in(d, 1);
    if (!sc || sc->data.size() != 1 || !std::isfinite(sc->data[0]) || sc->data[0] == 0.f) return false;
    *scale = sc->data[0];
    *zp = 0.f;
    *has_zp = false;
    if (has_in(d, 2)) {
      const HostTensor* z = const_in(d, 2);
      if (!z || z->data.size() != 1 || !std::isfinite(z->data[0]) || z->data[0] != std::nearbyint(z->data[0])) return false;
      *zp = z->data[0];
      *has_zp = true;
    }
    return true;
  };
  auto only_consumer = [&](const std::string& name, int* node, int* slot) -> bool {
    if (graph_outputs_.count(name)) return false;
    auto it = consumers_.find(name);
    if (it == consumers_.end() || it->second.size() != 1) return false;
    *node = it->second[0].first;
    *slot = it->second[0].second;
    return !skipped_[*node];
  };
  k::ResidualParams rp{};
  bool hz;
  if (!per_tensor(n, &rp.a_scale, &rp.a_zp, &hz)) return false;
  auto x1 = S.index_.find(in_name(n, 0));
  if (x1 == S.index_.end()) return false;
  int add_i, add_slot;
  if (!only_consumer(n.outputs[0], &add_i, &add_slot) || nodes_[add_i].op != "Add" || add_slot > 1 || !nodes_[add_i].attrs.names().empty()) return false;
  const NodeDef& add = nodes_[add_i];
  if (add.inputs.size() != 2) return false;
  const std::string& other = add.inputs[1 - add_slot];
  if (S.index_.count(other)) return false;  // already materialised by an earlier node
  int d2_i = -1;
  for (int j = ni + 1; j < add_i; ++j)
    if (!skipped_[j] && nodes_[j].op == "DequantizeLinear" && !nodes_[j].outputs.empty() && nodes_[j].outputs[0] == other) d2_i = j;
  if (d2_i < 0) return false;
  const NodeDef& d2 = nodes_[d2_i];
  int c2, s2;
  if (!only_consumer(other, &c2, &s2) || c2 != add_i) return false;
  if (!per_tensor(d2, &rp.b_scale, &rp.b_zp, &hz)) return false;
  auto x2 = S.index_.find(in_name(d2, 0));
  if (x2 == S.index_.end()) return false;
  const Value va = V(x1->second), vb = V(x2->second);
  auto eight_bit = [](const Value& v) { return v.dt == DT::U8 || v.dt == DT::I8; };
  if (!eight_bit(va) || !eight_bit(vb) || va.shape != vb.shape) return false;
  if (va.shape.size() == 4 && !order_free(va) && va.layout != vb.layout) return false;
  std::string cur = add.outputs[0];
  int relu_i = sole_consumer(cur, "Relu");
  rp.relu = relu_i >= 0 ? 1 : 0;
  if (relu_i >= 0) cur = nodes_[relu_i].outputs[0];
  int q_i, q_slot;
  if (!only_consumer(cur, &q_i, &q_slot) || nodes_[q_i].op != "QuantizeLinear" || q_slot != 0) return false;
  const NodeDef& q = nodes_[q_i];
  bool q_has_zp;
  if (!per_tensor(q, &rp.y_scale, &rp.y_zp, &q_has_zp)) return false;
  // saturation_range (oxionnx-ops src/indexing/quantize.rs:58-64)
  const bool u8 = !q_has_zp || rp.y_zp > 127.0f;
  rp.lo = u8 ? 0.f : -128.f;
  rp.hi = u8 ? 255.f : 127.f;
  const DT odt = u8 ? DT::U8 : DT::I8;
  skipped_[d2_i] = skipped_[add_i] = skipped_[q_i] = 1;
  if (relu_i >= 0) skipped_[relu_i] = 1;
  const int ai = x1->second, bi = x2->second;
  const int yi = add_value(q.outputs[0], va.shape, odt, va.shape.size() == 4 ? va.layout : Layout::PLAIN);
  const int64_t count = va.numel();
  const DT adt = va.dt, bdt = vb.dt;
  k::residual_requant_prepare(rp, adt, bdt);
  Step& st = add_step(n, "residual_requant", 2, {ai, bi}, {yi});
  st.node_name = add.name;
  st.op_type = "DequantizeLinear+Add+Relu+QuantizeLinear";
  st.kernel = rp.proven_fast == 2 ? "residual_requant (division-free, packed pairs, proven per parameter set)"
                                  : (rp.proven_fast ? "residual_requant (division-free, proven per parameter set)" : "residual_requant");
  st.work = 3.0 * (double)count;
  st.launch = [this, ai, bi, yi, adt, bdt, odt, count, rp](cudaStream_t s) {
    k::residual_requant(V(ai).ptr, adt, V(bi).ptr, bdt, V(yi).ptr, odt, count, rp, s);
    C.counters.glue_launches++;
    C.counters.kernel_launches++;
  };
  return true;
}

// =========================================================================================
void Session::plan(const std::vector<NodeDef>& nodes, const std::vector<std::pair<std::string, std::vector<int64_t>>>& inputs,
                   const std::map<std::string, const HostTensor*>& volatile_consts, const std::vector<std::string>& outputs) {
  auto p = std::make_shared<Planner>(*this, *ctx_, nodes, volatile_consts);
  planner_ = p;
  p->run(inputs, outputs);
}

}  // namespace oxb
