// ONNX model loading and the host-side fusion passes that produce the fused-node contract of the kernels.
//
// Loading restates, for the parts of the format the hot path needs, what the reference's oxionnx-proto crate does:
// a protobuf wire-format reader (src/reader.rs), the ModelProto / GraphProto / NodeProto / TensorProto /
// ValueInfoProto field tables (src/parser.rs, src/types.rs), every numeric tensor decoded to f32 lanes with its
// declared element type kept beside them (TensorProto::try_to_tensor, src/types.rs:98-118), Constant nodes
// folded into initializers, initializers removed from the graph inputs (src/model.rs:286-355).
//
// The passes restate the reference's optimizer for this path, in its order (src/optimizer/mod.rs):
// fuse_conv_batchnorm (src/optimizer/fusion/conv/batchnorm.rs:17-188), fuse_conv_relu (relu.rs:69-179),
// fuse_conv_clip_to_conv_relu6 (relu6.rs:30), fuse_instance_norm (src/optimizer/fusion/instance_norm.rs:199-268),
// fuse_matmul_add (src/optimizer/fusion/matmul/matmul_add.rs:34-132) and fuse_conv_add_relu
// (src/optimizer/fusion/conv/add_relu.rs:27-156).
#include "model.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <set>
#include <unordered_map>
#include <unordered_set>

namespace oxb {

namespace {

// ---- protobuf wire format ------------------------------------------------------------------
struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  bool done() const { return p >= end; }
  uint64_t varint() {
    uint64_t v = 0;
    int shift = 0;
    while (true) {
      if (p >= end) raise(OXB200_FAILED, "onnx: truncated varint");
      const uint8_t b = *p++;
      if (shift < 64) v |= (uint64_t)(b & 0x7f) << shift;
      if (!(b & 0x80)) break;
      shift += 7;
      if (shift > 70) raise(OXB200_FAILED, "onnx: varint longer than ten bytes");
    }
    return v;
  }
  uint32_t fixed32() {
    if (end - p < 4) raise(OXB200_FAILED, "onnx: truncated 32-bit field");
    uint32_t v;
    std::memcpy(&v, p, 4);
    p += 4;
    return v;
  }
  uint64_t fixed64() {
    if (end - p < 8) raise(OXB200_FAILED, "onnx: truncated 64-bit field");
    uint64_t v;
    std::memcpy(&v, p, 8);
    p += 8;
    return v;
  }
  Reader sub() {
    const uint64_t n = varint();
    if ((uint64_t)(end - p) < n) raise(OXB200_FAILED, "onnx: length-delimited field runs past the end of its message");
    Reader r{p, p + n};
    p += n;
    return r;
  }
  std::string str() {
    Reader r = sub();
    return std::string((const char*)r.p, (size_t)(r.end - r.p));
  }
  void skip(uint32_t wire) {
    switch (wire) {
      case 0: (void)varint(); break;
      case 1: (void)fixed64(); break;
      case 2: (void)sub(); break;
      case 5: (void)fixed32(); break;
      default: raise(OXB200_FAILED, "onnx: unsupported wire type %u", wire);
    }
  }
};

float f32_of(uint32_t bits) {
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}
float half_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h >> 15) << 31, exp = (h >> 10) & 0x1f, man = h & 0x3ff;
  if (exp == 0) {
    if (man == 0) return f32_of(sign);
    float v = std::ldexp((float)man, -24);
    return (h >> 15) ? -v : v;
  }
  if (exp == 31) return f32_of(sign | 0x7f800000u | (man << 13));
  return f32_of(sign | ((exp + 112) << 23) | (man << 13));
}
float bf16_to_f32(uint16_t h) { return f32_of((uint32_t)h << 16); }

// TensorProto.DataType
enum { ONNX_FLOAT = 1, ONNX_UINT8 = 2, ONNX_INT8 = 3, ONNX_UINT16 = 4, ONNX_INT16 = 5, ONNX_INT32 = 6, ONNX_INT64 = 7, ONNX_BOOL = 9, ONNX_FLOAT16 = 10,
       ONNX_DOUBLE = 11, ONNX_UINT32 = 12, ONNX_UINT64 = 13, ONNX_BFLOAT16 = 16 };

size_t onnx_elem_size(int32_t dt) {
  switch (dt) {
    case ONNX_FLOAT: case ONNX_INT32: case ONNX_UINT32: return 4;
    case ONNX_UINT8: case ONNX_INT8: case ONNX_BOOL: return 1;
    case ONNX_UINT16: case ONNX_INT16: case ONNX_FLOAT16: case ONNX_BFLOAT16: return 2;
    case ONNX_INT64: case ONNX_UINT64: case ONNX_DOUBLE: return 8;
    default: return 0;
  }
}

struct RawTensor {
  std::string name;
  std::vector<int64_t> dims;
  int32_t data_type = ONNX_FLOAT;
  std::vector<float> float_data;
  std::vector<int32_t> int32_data;
  std::vector<int64_t> int64_data;
  std::vector<double> double_data;
  std::vector<uint64_t> uint64_data;
  const uint8_t* raw = nullptr;
  size_t raw_len = 0;
  bool external = false;
};

template <typename T, typename F>
void read_packed_or_single(Reader& r, uint32_t wire, std::vector<T>& out, F one) {
  if (wire == 2) {
    Reader s = r.sub();
    while (!s.done()) out.push_back(one(s));
  } else {
    out.push_back(one(r));
  }
}

RawTensor parse_tensor(Reader r) {
  RawTensor t;
  while (!r.done()) {
    const uint64_t key = r.varint();
    const uint32_t field = (uint32_t)(key >> 3), wire = (uint32_t)(key & 7);
    switch (field) {
      case 1: read_packed_or_single(r, wire, t.dims, [](Reader& s) { return (int64_t)s.varint(); }); break;
      case 2: t.data_type = (int32_t)r.varint(); break;
      case 4: read_packed_or_single(r, wire, t.float_data, [](Reader& s) { return f32_of(s.fixed32()); }); break;
      case 5: read_packed_or_single(r, wire, t.int32_data, [](Reader& s) { return (int32_t)s.varint(); }); break;
      case 7: read_packed_or_single(r, wire, t.int64_data, [](Reader& s) { return (int64_t)s.varint(); }); break;
      case 8: t.name = r.str(); break;
      case 9: {
        Reader s = r.sub();
        t.raw = s.p;
        t.raw_len = (size_t)(s.end - s.p);
        break;
      }
      case 10: read_packed_or_single(r, wire, t.double_data, [](Reader& s) {
                 const uint64_t b = s.fixed64();
                 double d;
                 std::memcpy(&d, &b, 8);
                 return d;
               });
        break;
      case 11: read_packed_or_single(r, wire, t.uint64_data, [](Reader& s) { return s.varint(); }); break;
      case 13: t.external = true; r.skip(wire); break;
      case 14: if (r.varint() == 1) t.external = true; break;
      default: r.skip(wire);
    }
  }
  return t;
}

// try_to_tensor (oxionnx-proto src/types.rs:98-118): every numeric element type becomes f32 lanes.
HostTensor tensor_to_host(const RawTensor& t) {
  if (t.external) raise(OXB200_DECLINED, "onnx: tensor '%s' keeps its data in an external file", t.name.c_str());
  HostTensor h;
  int64_t count = 1;
  for (int64_t d : t.dims) {
    if (d < 0) raise(OXB200_FAILED, "onnx: tensor '%s' has a negative dimension", t.name.c_str());
    if (d != 0 && count > std::numeric_limits<int64_t>::max() / d) raise(OXB200_FAILED, "onnx: tensor '%s': shape overflows", t.name.c_str());
    count *= d;
    h.shape.push_back(d);
  }
  const int32_t dt = t.data_type;
  const size_t es = onnx_elem_size(dt);
  if (es == 0) raise(OXB200_DECLINED, "onnx: tensor '%s' has element type %d, which has no f32-lane form", t.name.c_str(), (int)dt);
  h.data.resize((size_t)count);
  auto lane_from_i32 = [&](int32_t v) -> float {  // int32_field_to_f32 (types.rs:38-56)
    switch (dt) {
      case ONNX_FLOAT16: return half_to_f32((uint16_t)v);
      case ONNX_BFLOAT16: return bf16_to_f32((uint16_t)v);
      case ONNX_INT8: return (float)(int8_t)v;
      case ONNX_UINT8: return (float)(uint8_t)v;
      case ONNX_INT16: return (float)(int16_t)v;
      case ONNX_UINT16: return (float)(uint16_t)v;
      case ONNX_BOOL: return v != 0 ? 1.f : 0.f;
      default: return (float)v;
    }
  };
  if (t.raw_len > 0 || (count > 0 && t.raw != nullptr && t.float_data.empty() && t.int32_data.empty() && t.int64_data.empty() && t.double_data.empty() &&
                        t.uint64_data.empty())) {
    if (t.raw_len != (size_t)count * es)
      raise(OXB200_FAILED, "onnx: tensor '%s': %zu raw bytes for %lld elements of %zu bytes", t.name.c_str(), t.raw_len, (long long)count, es);
    const uint8_t* b = t.raw;
    for (int64_t i = 0; i < count; ++i) {
      switch (dt) {
        case ONNX_FLOAT: { uint32_t u; std::memcpy(&u, b + 4 * i, 4); h.data[i] = f32_of(u); break; }
        case ONNX_UINT8: h.data[i] = (float)b[i]; break;
        case ONNX_INT8: h.data[i] = (float)(int8_t)b[i]; break;
        case ONNX_BOOL: h.data[i] = b[i] ? 1.f : 0.f; break;
        case ONNX_UINT16: { uint16_t u; std::memcpy(&u, b + 2 * i, 2); h.data[i] = (float)u; break; }
        case ONNX_INT16: { int16_t u; std::memcpy(&u, b + 2 * i, 2); h.data[i] = (float)u; break; }
        case ONNX_FLOAT16: { uint16_t u; std::memcpy(&u, b + 2 * i, 2); h.data[i] = half_to_f32(u); break; }
        case ONNX_BFLOAT16: { uint16_t u; std::memcpy(&u, b + 2 * i, 2); h.data[i] = bf16_to_f32(u); break; }
        case ONNX_INT32: { int32_t u; std::memcpy(&u, b + 4 * i, 4); h.data[i] = (float)u; break; }
        case ONNX_UINT32: { uint32_t u; std::memcpy(&u, b + 4 * i, 4); h.data[i] = (float)u; break; }
        case ONNX_INT64: { int64_t u; std::memcpy(&u, b + 8 * i, 8); h.data[i] = (float)u; break; }
        case ONNX_UINT64: { uint64_t u; std::memcpy(&u, b + 8 * i, 8); h.data[i] = (float)u; break; }
        case ONNX_DOUBLE: { double u; std::memcpy(&u, b + 8 * i, 8); h.data[i] = (float)u; break; }
        default: break;
      }
    }
  } else if (!t.float_data.empty()) {
    if ((int64_t)t.float_data.size() != count) raise(OXB200_FAILED, "onnx: tensor '%s': float_data length disagrees with its shape", t.name.c_str());
    h.data = t.float_data;
  } else if (!t.int32_data.empty()) {
    if ((int64_t)t.int32_data.size() != count) raise(OXB200_FAILED, "onnx: tensor '%s': int32_data length disagrees with its shape", t.name.c_str());
    for (int64_t i = 0; i < count; ++i) h.data[i] = lane_from_i32(t.int32_data[i]);
  } else if (!t.int64_data.empty()) {
    if ((int64_t)t.int64_data.size() != count) raise(OXB200_FAILED, "onnx: tensor '%s': int64_data length disagrees with its shape", t.name.c_str());
    for (int64_t i = 0; i < count; ++i) h.data[i] = (float)t.int64_data[i];
  } else if (!t.double_data.empty()) {
    if ((int64_t)t.double_data.size() != count) raise(OXB200_FAILED, "onnx: tensor '%s': double_data length disagrees with its shape", t.name.c_str());
    for (int64_t i = 0; i < count; ++i) h.data[i] = (float)t.double_data[i];
  } else if (!t.uint64_data.empty()) {
    if ((int64_t)t.uint64_data.size() != count) raise(OXB200_FAILED, "onnx: tensor '%s': uint64_data length disagrees with its shape", t.name.c_str());
    for (int64_t i = 0; i < count; ++i) h.data[i] = (float)t.uint64_data[i];
  } else if (count != 0) {
    raise(OXB200_FAILED, "onnx: tensor '%s' carries no data for %lld elements", t.name.c_str(), (long long)count);
  }
  DT declared;
  h.declared = onnx_dtype_to_dt(dt, &declared) ? declared : DT::F32;
  return h;
}

struct ParsedAttr {
  std::string name;
  bool has_f = false, has_i = false, has_s = false, has_t = false, has_graph = false;
  float f = 0.f;
  int64_t i = 0;
  std::string s;
  std::vector<float> floats;
  std::vector<int64_t> ints;
  RawTensor t;
  int32_t type = 0;
};

ParsedAttr parse_attr(Reader r) {
  ParsedAttr a;
  while (!r.done()) {
    const uint64_t key = r.varint();
    const uint32_t field = (uint32_t)(key >> 3), wire = (uint32_t)(key & 7);
    switch (field) {
      case 1: a.name = r.str(); break;
      case 2: a.f = f32_of(r.fixed32()); a.has_f = true; break;
      case 3: a.i = (int64_t)r.varint(); a.has_i = true; break;
      case 4: a.s = r.str(); a.has_s = true; break;
      case 5: a.t = parse_tensor(r.sub()); a.has_t = true; break;
      case 6: a.has_graph = true; r.skip(wire); break;
      case 7: read_packed_or_single(r, wire, a.floats, [](Reader& s) { return f32_of(s.fixed32()); }); break;
      case 8: read_packed_or_single(r, wire, a.ints, [](Reader& s) { return (int64_t)s.varint(); }); break;
      case 11: a.has_graph = true; r.skip(wire); break;
      case 20: a.type = (int32_t)r.varint(); break;
      default: r.skip(wire);
    }
  }
  return a;
}

struct ParsedNode {
  NodeDef def;
  std::vector<ParsedAttr> attrs;
  std::string domain;
};

ParsedNode parse_node(Reader r) {
  ParsedNode n;
  while (!r.done()) {
    const uint64_t key = r.varint();
    const uint32_t field = (uint32_t)(key >> 3), wire = (uint32_t)(key & 7);
    switch (field) {
      case 1: n.def.inputs.push_back(r.str()); break;
      case 2: n.def.outputs.push_back(r.str()); break;
      case 3: n.def.name = r.str(); break;
      case 4: n.def.op = r.str(); break;
      case 5: n.attrs.push_back(parse_attr(r.sub())); break;
      case 7: n.domain = r.str(); break;
      default: r.skip(wire);
    }
  }
  return n;
}

ModelValueInfo parse_value_info(Reader r) {
  ModelValueInfo v;
  bool have_shape = false;
  while (!r.done()) {
    const uint64_t key = r.varint();
    const uint32_t field = (uint32_t)(key >> 3), wire = (uint32_t)(key & 7);
    if (field == 1) {
      v.name = r.str();
    } else if (field == 2 && wire == 2) {  // TypeProto
      Reader tp = r.sub();
      while (!tp.done()) {
        const uint64_t k2 = tp.varint();
        if ((k2 >> 3) == 1 && (k2 & 7) == 2) {  // tensor_type
          Reader tt = tp.sub();
          while (!tt.done()) {
            const uint64_t k3 = tt.varint();
            if ((k3 >> 3) == 1) {
              v.onnx_dtype = (int32_t)tt.varint();
            } else if ((k3 >> 3) == 2 && (k3 & 7) == 2) {  // TensorShapeProto
              Reader sh = tt.sub();
              have_shape = true;
              while (!sh.done()) {
                const uint64_t k4 = sh.varint();
                if ((k4 >> 3) == 1 && (k4 & 7) == 2) {  // Dimension
                  Reader dm = sh.sub();
                  int64_t value = -1;
                  while (!dm.done()) {
                    const uint64_t k5 = dm.varint();
                    if ((k5 >> 3) == 1) value = (int64_t)dm.varint();
                    else dm.skip((uint32_t)(k5 & 7));
                  }
                  v.shape.push_back(value);
                } else {
                  sh.skip((uint32_t)(k4 & 7));
                }
              }
            } else {
              tt.skip((uint32_t)(k3 & 7));
            }
          }
        } else {
          tp.skip((uint32_t)(k2 & 7));
        }
      }
    } else {
      r.skip(wire);
    }
  }
  (void)have_shape;
  return v;
}

void attr_into(const ParsedAttr& a, AttrMap& out, const std::string& op) {
  if (a.has_graph) raise(OXB200_DECLINED, "onnx: node attribute '%s' of a %s holds a subgraph", a.name.c_str(), op.c_str());
  // AttributeProto.type: 1 FLOAT, 2 INT, 3 STRING, 4 TENSOR, 6 FLOATS, 7 INTS; files written before the field
  // existed carry the value only
  if (a.type == 1 || (a.type == 0 && a.has_f)) out.floats[a.name] = a.f;
  else if (a.type == 2 || (a.type == 0 && a.has_i)) out.ints[a.name] = a.i;
  else if (a.type == 3 || (a.type == 0 && a.has_s)) out.strings[a.name] = a.s;
  else if (a.type == 6 || (a.type == 0 && !a.floats.empty())) out.float_lists[a.name] = a.floats;
  else if (a.type == 7 || (a.type == 0 && !a.ints.empty())) out.int_lists[a.name] = a.ints;
  else if (a.type == 7) out.int_lists[a.name] = {};
  else if (a.type == 4 || a.has_t) raise(OXB200_DECLINED, "onnx: tensor-valued attribute '%s' on a %s", a.name.c_str(), op.c_str());
  else raise(OXB200_DECLINED, "onnx: attribute '%s' of a %s has a type this provider does not take (%d)", a.name.c_str(), op.c_str(), (int)a.type);
}

}  // namespace

bool onnx_dtype_to_dt(int32_t onnx_dtype, DT* out) {
  switch (onnx_dtype) {
    case ONNX_FLOAT: *out = DT::F32; return true;
    case ONNX_UINT8: *out = DT::U8; return true;
    case ONNX_INT8: *out = DT::I8; return true;
    case ONNX_INT32: *out = DT::I32; return true;
    case ONNX_INT16: *out = DT::I16; return true;
    case ONNX_FLOAT16: *out = DT::F16; return true;
    case ONNX_BFLOAT16: *out = DT::BF16; return true;
    default: return false;
  }
}

Model load_onnx(const uint8_t* bytes, size_t len) {
  if (!bytes || len == 0) raise(OXB200_FAILED, "onnx: empty model");
  Model m;
  Reader top{bytes, bytes + len};
  bool have_graph = false;
  Reader graph{nullptr, nullptr};
  while (!top.done()) {
    const uint64_t key = top.varint();
    const uint32_t field = (uint32_t)(key >> 3), wire = (uint32_t)(key & 7);
    if (field == 1 && wire == 0) m.ir_version = (int64_t)top.varint();
    else if (field == 2 && wire == 2) m.producer = top.str();
    else if (field == 7 && wire == 2) {
      graph = top.sub();
      have_graph = true;
    } else if (field == 8 && wire == 2) {  // OperatorSetIdProto: the default domain's version
      Reader os = top.sub();
      std::string domain;
      int64_t version = 0;
      while (!os.done()) {
        const uint64_t k2 = os.varint();
        if ((k2 >> 3) == 1) domain = os.str();
        else if ((k2 >> 3) == 2) version = (int64_t)os.varint();
        else os.skip((uint32_t)(k2 & 7));
      }
      if (domain.empty() || domain == "ai.onnx") m.opset = std::max(m.opset, version);
    } else {
      top.skip(wire);
    }
  }
  if (!have_graph) raise(OXB200_FAILED, "onnx: the model holds no graph");

  std::vector<ParsedNode> nodes;
  std::vector<ModelValueInfo> declared_inputs;
  while (!graph.done()) {
    const uint64_t key = graph.varint();
    const uint32_t field = (uint32_t)(key >> 3), wire = (uint32_t)(key & 7);
    switch (field) {
      case 1: nodes.push_back(parse_node(graph.sub())); break;
      case 5: {
        RawTensor t = parse_tensor(graph.sub());
        if (t.name.empty()) raise(OXB200_FAILED, "onnx: an initializer has no name");
        m.initializers[t.name] = tensor_to_host(t);
        m.initializer_order.push_back(t.name);
        break;
      }
      case 11: declared_inputs.push_back(parse_value_info(graph.sub())); break;
      case 12: m.outputs.push_back(parse_value_info(graph.sub())); break;
      case 13: {
        ModelValueInfo v = parse_value_info(graph.sub());
        if (!v.name.empty()) m.known_shapes[v.name] = v.shape;
        break;
      }
      case 15: raise(OXB200_DECLINED, "onnx: sparse initializers are not taken");
      default: graph.skip(wire);
    }
  }
  // initializers are not graph inputs (older exporters list them among the inputs)
  for (auto& in : declared_inputs) {
    if (m.initializers.count(in.name)) continue;
    m.known_shapes[in.name] = in.shape;
    m.inputs.push_back(in);
  }
  for (auto& kv : m.initializers) m.known_shapes[kv.first] = kv.second.shape;

  for (ParsedNode& pn : nodes) {
    if (!pn.domain.empty() && pn.domain != "ai.onnx" && pn.domain != "com.microsoft")
      raise(OXB200_DECLINED, "onnx: node '%s' (%s) belongs to domain '%s'", pn.def.name.c_str(), pn.def.op.c_str(), pn.domain.c_str());
    if (pn.def.op == "Constant") {
      // fold into an initializer: value (tensor), value_float / value_int, value_floats / value_ints
      if (pn.def.outputs.size() != 1 || pn.def.outputs[0].empty()) raise(OXB200_FAILED, "onnx: Constant node without an output name");
      HostTensor h;
      bool ok = false;
      for (const ParsedAttr& a : pn.attrs) {
        if (a.name == "value" && a.has_t) {
          h = tensor_to_host(a.t);
          ok = true;
        } else if (a.name == "value_float") {
          h.data = {a.f};
          ok = true;
        } else if (a.name == "value_int") {
          h.data = {(float)a.i};
          h.declared = DT::F32;
          ok = true;
        } else if (a.name == "value_floats") {
          h.data = a.floats;
          h.shape = {(int64_t)a.floats.size()};
          ok = true;
        } else if (a.name == "value_ints") {
          for (int64_t v : a.ints) h.data.push_back((float)v);
          h.shape = {(int64_t)a.ints.size()};
          ok = true;
        }
      }
      if (!ok) raise(OXB200_DECLINED, "onnx: Constant node '%s' has a value form this provider does not take", pn.def.name.c_str());
      m.known_shapes[pn.def.outputs[0]] = h.shape;
      m.initializers[pn.def.outputs[0]] = std::move(h);
      m.initializer_order.push_back(pn.def.outputs[0]);
      continue;
    }
    for (const ParsedAttr& a : pn.attrs) attr_into(a, pn.def.attrs, pn.def.op);
    m.nodes.push_back(std::move(pn.def));
  }
  topo_sort(m);
  return m;
}

// ---- graph helpers of the passes (src/optimizer/graph_utils.rs) ------------------------------
namespace {

struct Usage {  // TensorUsage: consumer slots per tensor, graph outputs
  std::unordered_map<std::string, int> consumers;
  std::unordered_set<std::string> outputs;
  explicit Usage(const Model& m) {
    for (const NodeDef& n : m.nodes)
      for (const std::string& in : n.inputs)
        if (!in.empty()) consumers[in] += 1;
    for (const ModelValueInfo& o : m.outputs) outputs.insert(o.name);
  }
  int count(const std::string& name) const {
    auto it = consumers.find(name);
    return it == consumers.end() ? 0 : it->second;
  }
  bool is_output(const std::string& name) const { return outputs.count(name) != 0; }
  // a pass may fuse a tensor away only when it has exactly one consumer and is not a graph output
  bool fusable(const std::string& name) const { return !name.empty() && !is_output(name) && count(name) == 1; }
};

std::unordered_map<std::string, int> producers(const Model& m) {
  std::unordered_map<std::string, int> p;
  for (size_t i = 0; i < m.nodes.size(); ++i)
    for (const std::string& o : m.nodes[i].outputs)
      if (!o.empty()) p[o] = (int)i;
  return p;
}

// NameAllocator: a generated name never shadows an existing tensor or another generated one
struct Names {
  std::unordered_set<std::string> taken;
  explicit Names(const Model& m) {
    for (auto& kv : m.initializers) taken.insert(kv.first);
    for (const NodeDef& n : m.nodes) {
      for (auto& s : n.inputs) taken.insert(s);
      for (auto& s : n.outputs) taken.insert(s);
    }
  }
  std::string allocate(const std::string& base, const std::string& suffix) {
    std::string cand = base + suffix;
    int k = 0;
    while (taken.count(cand)) cand = base + suffix + "_" + std::to_string(++k);
    taken.insert(cand);
    return cand;
  }
};

bool const_scalar(const Model& m, const std::string& name, float* out) {
  if (name.empty()) return false;
  auto it = m.initializers.find(name);
  if (it == m.initializers.end() || it->second.data.size() != 1) return false;
  *out = it->second.data[0];
  return true;
}

int apply(Model& m, const std::set<int>& skip, std::map<int, NodeDef>& replace) {
  std::vector<NodeDef> out;
  for (size_t i = 0; i < m.nodes.size(); ++i) {
    if (skip.count((int)i)) continue;
    auto it = replace.find((int)i);
    out.push_back(it == replace.end() ? std::move(m.nodes[i]) : std::move(it->second));
  }
  const int removed = (int)(m.nodes.size() - out.size());
  m.nodes = std::move(out);
  return removed;
}

// Shape propagation for the matchers that need a rank (shape_inference.rs feeds the reference's passes the same
// way): shapes the file states win; otherwise elementwise ops broadcast, reductions keep or drop their axes,
// spatial operators keep their rank.  A dimension that cannot be derived is -1; a tensor whose rank cannot be
// derived stays out of the table, and a matcher that needs it declines.
void infer_shapes(Model& m) {
  static const std::set<std::string> unary = {"Relu", "Sigmoid", "Tanh", "Sqrt", "Reciprocal", "Neg", "Abs", "Exp", "Log", "Erf", "Gelu", "Silu", "SiLU",
                                              "Clip", "LeakyRelu", "PRelu", "Softmax", "LogSoftmax", "Identity", "Cast", "Dropout", "Floor", "Ceil",
                                              "HardSigmoid", "HardSwish", "Elu", "Selu", "Softplus", "Mish", "LayerNormalization", "BatchNormalization",
                                              "InstanceNormalization", "OxiInstanceNorm", "QuantizeLinear", "DequantizeLinear", "LRN"};
  static const std::set<std::string> binary = {"Add", "Sub", "Mul", "Div", "Pow", "Min", "Max", "Equal", "Less", "Greater", "And", "Or", "Where"};
  static const std::set<std::string> reductions = {"ReduceMean", "ReduceSum", "ReduceMax", "ReduceMin", "ReduceProd", "ReduceL2", "ReduceL1", "ReduceSumSquare"};
  static const std::set<std::string> spatial = {"Conv", "ConvAddRelu", "MaxPool", "AveragePool", "GlobalAveragePool", "GlobalMaxPool", "ConvTranspose",
                                                "QLinearConv", "ConvInteger", "Resize", "Upsample", "Pad"};
  auto known = [&](const std::string& name) -> const std::vector<int64_t>* {
    auto it = m.known_shapes.find(name);
    return it == m.known_shapes.end() ? nullptr : &it->second;
  };
  for (const NodeDef& n : m.nodes) {
    if (n.outputs.empty() || n.outputs[0].empty() || known(n.outputs[0]) || n.inputs.empty()) continue;
    std::vector<int64_t> out;
    bool ok = false;
    const std::vector<int64_t>* a = known(n.inputs[0]);
    if (unary.count(n.op)) {
      if (a) out = *a, ok = true;
    } else if (binary.count(n.op)) {
      std::vector<const std::vector<int64_t>*> ins;
      bool all = true;
      for (const std::string& in : n.inputs) {
        const std::vector<int64_t>* s = known(in);
        if (!s) all = false;
        else ins.push_back(s);
      }
      if (all && !ins.empty()) {
        size_t rank = 0;
        for (auto* s : ins) rank = std::max(rank, s->size());
        out.assign(rank, 1);
        for (auto* s : ins)
          for (size_t d = 0; d < s->size(); ++d) {
            int64_t& o = out[rank - s->size() + d];
            const int64_t v = (*s)[d];
            if (v == 1) continue;
            o = (o == 1 || o == v) ? v : (v < 0 ? o : (o < 0 ? v : -1));
          }
        ok = true;
      }
    } else if (reductions.count(n.op)) {
      if (a) {
        std::vector<int64_t> axes = n.attrs.int_list("axes");
        bool axes_known = true;
        if (axes.empty() && n.inputs.size() > 1 && !n.inputs[1].empty()) {
          auto it = m.initializers.find(n.inputs[1]);
          if (it == m.initializers.end()) axes_known = false;
          else
            for (float v : it->second.data) axes.push_back((int64_t)v);
        }
        const int64_t rank = (int64_t)a->size();
        const bool keep = n.attrs.i("keepdims", 1) != 0;
        if (axes_known) {
          std::set<int64_t> red;
          if (axes.empty())
            for (int64_t d = 0; d < rank; ++d) red.insert(d);
          for (int64_t ax : axes) red.insert(ax < 0 ? ax + rank : ax);
          for (int64_t d = 0; d < rank; ++d) {
            if (!red.count(d)) out.push_back((*a)[d]);
            else if (keep) out.push_back(1);
          }
          ok = true;
        }
      }
    } else if (spatial.count(n.op)) {
      if (a) {
        out.assign(a->size(), -1);
        if (!out.empty()) out[0] = (*a)[0];
        if (out.size() > 1 && (n.op == "MaxPool" || n.op == "AveragePool" || n.op == "GlobalAveragePool" || n.op == "GlobalMaxPool" || n.op == "Pad" ||
                               n.op == "Resize" || n.op == "Upsample"))
          out[1] = (*a)[1];
        if (out.size() > 1 && (n.op == "Conv" || n.op == "ConvAddRelu") && n.inputs.size() > 1)
          if (const std::vector<int64_t>* w = known(n.inputs[1]))
            if (!w->empty()) out[1] = (*w)[0];
        if (n.op == "GlobalAveragePool" || n.op == "GlobalMaxPool")
          for (size_t d = 2; d < out.size(); ++d) out[d] = 1;
        ok = true;
      }
    } else if (n.op == "MatMul") {
      const std::vector<int64_t>* b = n.inputs.size() > 1 ? known(n.inputs[1]) : nullptr;
      if (a && b && a->size() >= 2 && b->size() >= 2) {
        const size_t rank = std::max(a->size(), b->size());
        out.assign(rank, -1);
        const std::vector<int64_t>& lead = a->size() >= b->size() ? *a : *b;
        for (size_t d = 0; d + 2 < rank; ++d) out[d] = lead[d];
        out[rank - 2] = (*a)[a->size() - 2];
        out[rank - 1] = (*b)[b->size() - 1];
        ok = true;
      }
    } else if (n.op == "Gemm") {
      const std::vector<int64_t>* b = n.inputs.size() > 1 ? known(n.inputs[1]) : nullptr;
      if (a && b && a->size() == 2 && b->size() == 2) {
        out = {(*a)[n.attrs.i("transA", 0) ? 1 : 0], (*b)[n.attrs.i("transB", 0) ? 0 : 1]};
        ok = true;
      }
    } else if (n.op == "Flatten") {
      if (a) {
        int64_t axis = n.attrs.i("axis", 1);
        if (axis < 0) axis += (int64_t)a->size();
        int64_t lo = 1, hi = 1;
        for (int64_t d = 0; d < (int64_t)a->size(); ++d) {
          int64_t& acc = d < axis ? lo : hi;
          acc = (acc < 0 || (*a)[d] < 0) ? -1 : acc * (*a)[d];
        }
        out = {lo, hi};
        ok = true;
      }
    } else if (n.op == "Transpose") {
      if (a) {
        std::vector<int64_t> perm = n.attrs.int_list("perm");
        out.resize(a->size());
        for (size_t d = 0; d < a->size(); ++d) {
          const size_t src = perm.size() == a->size() ? (size_t)perm[d] : a->size() - 1 - d;
          out[d] = src < a->size() ? (*a)[src] : -1;
        }
        ok = true;
      }
    } else if (n.op == "Concat") {
      if (a) {
        out = *a;
        int64_t axis = n.attrs.i("axis", 0);
        if (axis < 0) axis += (int64_t)out.size();
        if (axis >= 0 && axis < (int64_t)out.size()) out[axis] = -1;
        ok = true;
      }
    }
    if (ok) m.known_shapes[n.outputs[0]] = std::move(out);
  }
}

struct ClipBounds {
  float lo, hi;
};
// resolve_clip_bounds (relu.rs): a bound is an input when the slot is wired (it must then be a constant scalar),
// else the attribute, else unbounded; NaN or inverted bounds are not fused
bool clip_bounds(const Model& m, const NodeDef& n, ClipBounds* out) {
  auto bound = [&](size_t slot, const char* attr, float unbounded, float* v) -> bool {
    if (slot < n.inputs.size() && !n.inputs[slot].empty()) return const_scalar(m, n.inputs[slot], v);
    *v = n.attrs.f(attr, unbounded);
    return true;
  };
  float lo, hi;
  if (!bound(1, "min", -std::numeric_limits<float>::infinity(), &lo)) return false;
  if (!bound(2, "max", std::numeric_limits<float>::infinity(), &hi)) return false;
  if (std::isnan(lo) || std::isnan(hi) || lo > hi) return false;
  *out = {lo, hi};
  return true;
}

}  // namespace

void topo_sort(Model& m) {
  const size_t n = m.nodes.size();
  std::unordered_map<std::string, int> prod = producers(m);
  std::vector<std::vector<int>> users(n);
  std::vector<int> pending(n, 0);
  for (size_t i = 0; i < n; ++i) {
    std::set<int> deps;
    for (const std::string& in : m.nodes[i].inputs) {
      auto it = prod.find(in);
      if (it != prod.end() && it->second != (int)i) deps.insert(it->second);
    }
    pending[i] = (int)deps.size();
    for (int d : deps) users[d].push_back((int)i);
  }
  // Kahn's algorithm, lowest original index first: an already sorted graph keeps its order
  std::set<int> ready;
  for (size_t i = 0; i < n; ++i)
    if (pending[i] == 0) ready.insert((int)i);
  std::vector<NodeDef> out;
  out.reserve(n);
  while (!ready.empty()) {
    const int i = *ready.begin();
    ready.erase(ready.begin());
    out.push_back(std::move(m.nodes[i]));
    for (int u : users[i])
      if (--pending[u] == 0) ready.insert(u);
  }
  if (out.size() != n) raise(OXB200_FAILED, "onnx: the graph has a cycle");
  m.nodes = std::move(out);
}

// fuse_conv_batchnorm (batchnorm.rs:17-188): W' = W * factor[oc], b' = (b - mean) * factor + beta with
// factor = gamma / sqrt(var + eps); new initializers <conv_out>_fused_weight / _fused_bias, node <name>_fused_convbn.
int fuse_conv_batchnorm(Model& m) {
  if (m.nodes.size() < 2) return 0;
  auto prod = producers(m);
  Usage usage(m);
  Names names(m);
  std::set<int> skip;
  std::map<int, NodeDef> replace;
  for (size_t i = 0; i < m.nodes.size(); ++i) {
    const NodeDef& bn = m.nodes[i];
    if (bn.op != "BatchNormalization" || bn.inputs.size() < 5) continue;
    const std::string& conv_tensor = bn.inputs[0];
    if (!usage.fusable(conv_tensor)) continue;
    auto pit = prod.find(conv_tensor);
    if (pit == prod.end()) continue;
    const int ci = pit->second;
    if (skip.count(ci) || replace.count(ci)) continue;
    const NodeDef& conv = m.nodes[ci];
    if (conv.op != "Conv" || !conv.attrs.s("activation").empty() || conv.inputs.size() < 2) continue;
    auto get = [&](const std::string& name) -> const HostTensor* {
      auto it = m.initializers.find(name);
      return it == m.initializers.end() ? nullptr : &it->second;
    };
    const HostTensor *scale = get(bn.inputs[1]), *beta = get(bn.inputs[2]), *mean = get(bn.inputs[3]), *var = get(bn.inputs[4]), *w = get(conv.inputs[1]);
    if (!scale || !beta || !mean || !var || !w) continue;
    const float eps = bn.attrs.f("epsilon", 1e-5f);
    const size_t c_out = scale->data.size();
    if (c_out == 0 || beta->data.size() != c_out || mean->data.size() != c_out || var->data.size() != c_out || w->shape.empty() ||
        (size_t)w->shape[0] != c_out || w->data.size() % c_out != 0)
      continue;
    std::vector<float> bias(c_out, 0.f);
    if (conv.inputs.size() > 2 && !conv.inputs[2].empty()) {
      const HostTensor* b = get(conv.inputs[2]);
      if (b) {
        if (b->data.size() != c_out) continue;  // malformed: fold nothing rather than guess
        bias = b->data;
      }
    }
    if (conv.outputs.empty() || conv.outputs[0].empty()) continue;
    const size_t per = w->data.size() / c_out;
    HostTensor fw = *w, fb;
    fb.shape = {(int64_t)c_out};
    fb.data.resize(c_out);
    for (size_t c = 0; c < c_out; ++c) {
      const float inv_std = 1.0f / std::sqrt(var->data[c] + eps);
      const float factor = scale->data[c] * inv_std;
      for (size_t k = 0; k < per; ++k) fw.data[c * per + k] *= factor;
      fb.data[c] = (bias[c] - mean->data[c]) * factor + beta->data[c];
    }
    const std::string wn = names.allocate(conv.outputs[0], "_fused_weight"), bnm = names.allocate(conv.outputs[0], "_fused_bias");
    m.known_shapes[wn] = fw.shape;
    m.known_shapes[bnm] = fb.shape;
    m.initializers[wn] = std::move(fw);
    m.initializers[bnm] = std::move(fb);
    m.initializer_order.push_back(wn);
    m.initializer_order.push_back(bnm);
    NodeDef fused = conv;
    fused.name = conv.name + "_fused_convbn";
    fused.inputs = {conv.inputs[0], wn, bnm};
    fused.outputs = bn.outputs;
    replace[ci] = std::move(fused);
    skip.insert((int)i);
  }
  return apply(m, skip, replace);
}

// fuse_conv_relu (relu.rs:69-179): Relu, or Clip(0, +inf), becomes activation = "relu"; any other Clip becomes
// activation = "clip" with activation_min / activation_max; node <name>_fused_activation.
int fuse_conv_relu(Model& m) {
  if (m.nodes.size() < 2) return 0;
  auto prod = producers(m);
  Usage usage(m);
  std::set<int> skip;
  std::map<int, NodeDef> replace;
  for (size_t i = 0; i < m.nodes.size(); ++i) {
    const NodeDef& act = m.nodes[i];
    const bool is_relu = act.op == "Relu", is_clip = act.op == "Clip";
    if ((!is_relu && !is_clip) || act.inputs.empty() || act.outputs.empty()) continue;
    ClipBounds cb{0.f, 0.f};
    if (is_clip && !clip_bounds(m, act, &cb)) continue;
    const std::string& conv_tensor = act.inputs[0];
    if (!usage.fusable(conv_tensor)) continue;
    auto pit = prod.find(conv_tensor);
    if (pit == prod.end()) continue;
    const int ci = pit->second;
    if (skip.count(ci) || replace.count(ci)) continue;
    const NodeDef& conv = m.nodes[ci];
    if (conv.op != "Conv" || !conv.attrs.s("activation").empty()) continue;
    NodeDef fused = conv;
    if (is_relu || (cb.lo == 0.0f && cb.hi == std::numeric_limits<float>::infinity())) {
      fused.attrs.strings["activation"] = "relu";
    } else {
      fused.attrs.strings["activation"] = "clip";
      fused.attrs.floats["activation_min"] = cb.lo;
      fused.attrs.floats["activation_max"] = cb.hi;
    }
    fused.name = conv.name + "_fused_activation";
    fused.outputs = act.outputs;
    replace[ci] = std::move(fused);
    skip.insert((int)i);
  }
  return apply(m, skip, replace);
}

// fuse_conv_clip_to_conv_relu6 (relu6.rs:30): Clip(0, 6) behind a Conv; node <name>_fused_relu6.
int fuse_conv_clip_to_relu6(Model& m) {
  if (m.nodes.size() < 2) return 0;
  auto prod = producers(m);
  Usage usage(m);
  std::set<int> skip;
  std::map<int, NodeDef> replace;
  for (size_t i = 0; i < m.nodes.size(); ++i) {
    const NodeDef& clip = m.nodes[i];
    if (clip.op != "Clip" || clip.inputs.empty() || clip.outputs.empty()) continue;
    ClipBounds cb;
    if (!clip_bounds(m, clip, &cb)) continue;
    if (std::fabs(cb.lo - 0.0f) > 1e-7f || std::fabs(cb.hi - 6.0f) > 1e-7f) continue;
    if (!usage.fusable(clip.inputs[0])) continue;
    auto pit = prod.find(clip.inputs[0]);
    if (pit == prod.end()) continue;
    const int ci = pit->second;
    if (skip.count(ci) || replace.count(ci)) continue;
    const NodeDef& conv = m.nodes[ci];
    if (conv.op != "Conv" || !conv.attrs.s("activation").empty()) continue;
    NodeDef fused = conv;
    fused.attrs.strings["activation"] = "clip";
    fused.attrs.floats["activation_min"] = 0.0f;
    fused.attrs.floats["activation_max"] = 6.0f;
    fused.name = conv.name + "_fused_relu6";
    fused.outputs = clip.outputs;
    replace[ci] = std::move(fused);
    skip.insert((int)i);
  }
  return apply(m, skip, replace);
}

// fuse_instance_norm (instance_norm.rs:199-470): ReduceMean, Sub, Mul(diff, diff) | Pow(diff, 2), ReduceMean,
// Add(eps), Sqrt, [Reciprocal | Div(1, .)], Mul | Div  ->  OxiInstanceNorm{epsilon}; the runtime scale and shift
// that follow stay separate nodes.
int fuse_instance_norm(Model& m) {
  if (m.nodes.size() < 6) return 0;
  infer_shapes(m);
  auto prod = producers(m);
  Usage usage(m);
  auto rank_of = [&](const std::string& name) -> int {
    auto it = m.known_shapes.find(name);
    return it == m.known_shapes.end() ? -1 : (int)it->second.size();
  };
  auto spatial_reduce = [&](const NodeDef& n) -> bool {  // keepdims, axes == every axis from 2 on
    if (n.op != "ReduceMean" || n.attrs.i("keepdims", 1) != 1 || n.inputs.empty()) return false;
    std::vector<int64_t> axes = n.attrs.int_list("axes");
    if (axes.empty()) {
      if (n.inputs.size() < 2 || n.inputs[1].empty()) return false;
      auto it = m.initializers.find(n.inputs[1]);
      if (it == m.initializers.end() || it->second.data.empty()) return false;
      for (float v : it->second.data) axes.push_back((int64_t)v);
    }
    const int rank = rank_of(n.inputs[0]);
    if (rank < 3) return false;
    std::set<int64_t> resolved;
    for (int64_t a : axes) {
      const int64_t r = a < 0 ? a + rank : a;
      if (r < 0 || r >= rank) return false;
      resolved.insert(r);
    }
    if ((int)resolved.size() != rank - 2) return false;
    int64_t want = 2;
    for (int64_t r : resolved)
      if (r != want++) return false;
    return true;
  };
  auto is_recip_producer = [&](const std::string& name) {
    auto it = prod.find(name);
    return it != prod.end() && (m.nodes[it->second].op == "Reciprocal" || m.nodes[it->second].op == "Div");
  };
  std::set<int> claimed, skip;
  std::map<int, NodeDef> replace;
  for (size_t i = 0; i < m.nodes.size(); ++i) {
    if (claimed.count((int)i)) continue;
    const NodeDef& norm = m.nodes[i];
    if (norm.inputs.size() < 2 || norm.outputs.empty() || norm.outputs[0].empty()) continue;
    std::vector<int> consumed = {(int)i};
    std::string diff, std_name;
    if (norm.op == "Mul") {
      const bool l = is_recip_producer(norm.inputs[0]), r = is_recip_producer(norm.inputs[1]);
      if (l == r) continue;
      diff = l ? norm.inputs[1] : norm.inputs[0];
      const std::string recip_out = l ? norm.inputs[0] : norm.inputs[1];
      if (!usage.fusable(recip_out)) continue;
      const int ri = prod[recip_out];
      const NodeDef& recip = m.nodes[ri];
      if (recip.op == "Reciprocal") {
        if (recip.inputs.empty()) continue;
        std_name = recip.inputs[0];
      } else {
        float one;
        if (recip.inputs.size() < 2 || !const_scalar(m, recip.inputs[0], &one) || std::fabs(one - 1.0f) > 1e-6f) continue;
        std_name = recip.inputs[1];
      }
      consumed.push_back(ri);
    } else if (norm.op == "Div") {
      diff = norm.inputs[0];
      std_name = norm.inputs[1];
    } else {
      continue;
    }
    auto step = [&](const std::string& name, const char* op) -> int {  // the sole producer of a fusable tensor, of kind `op`
      if (!usage.fusable(name)) return -1;
      auto it = prod.find(name);
      if (it == prod.end() || m.nodes[it->second].op != op) return -1;
      return it->second;
    };
    const int sqrt_i = step(std_name, "Sqrt");
    if (sqrt_i < 0 || m.nodes[sqrt_i].inputs.empty()) continue;
    consumed.push_back(sqrt_i);
    const int add_i = step(m.nodes[sqrt_i].inputs[0], "Add");
    if (add_i < 0 || m.nodes[add_i].inputs.size() < 2) continue;
    // resolve_epsilon: one operand a finite non-negative constant scalar, the other not a constant
    std::string var_name;
    float eps = 0.f, tmp;
    {
      const std::string &lhs = m.nodes[add_i].inputs[0], &rhs = m.nodes[add_i].inputs[1];
      float e;
      if (const_scalar(m, rhs, &e) && std::isfinite(e) && e >= 0.f && !const_scalar(m, lhs, &tmp)) {
        var_name = lhs;
        eps = e;
      } else if (const_scalar(m, lhs, &e) && std::isfinite(e) && e >= 0.f && !const_scalar(m, rhs, &tmp)) {
        var_name = rhs;
        eps = e;
      } else {
        continue;
      }
    }
    consumed.push_back(add_i);
    const int var_i = step(var_name, "ReduceMean");
    if (var_i < 0 || !spatial_reduce(m.nodes[var_i])) continue;
    consumed.push_back(var_i);
    const std::string& sq_name = m.nodes[var_i].inputs[0];
    if (!usage.fusable(sq_name)) continue;
    auto sq_it = prod.find(sq_name);
    if (sq_it == prod.end()) continue;
    const NodeDef& sq = m.nodes[sq_it->second];
    if (sq.inputs.size() < 2) continue;
    int diff_slots;
    if (sq.op == "Mul" && sq.inputs[0] == diff && sq.inputs[1] == diff) {
      diff_slots = 2;
    } else if (sq.op == "Pow" && sq.inputs[0] == diff) {
      float ex;
      if (!const_scalar(m, sq.inputs[1], &ex) || std::fabs(ex - 2.0f) > 1e-6f) continue;
      diff_slots = 1;
    } else {
      continue;
    }
    consumed.push_back(sq_it->second);
    if (usage.count(diff) != diff_slots + 1 || usage.is_output(diff)) continue;
    auto sub_it = prod.find(diff);
    if (sub_it == prod.end() || m.nodes[sub_it->second].op != "Sub" || m.nodes[sub_it->second].inputs.size() < 2) continue;
    const std::string x_name = m.nodes[sub_it->second].inputs[0], mean_name = m.nodes[sub_it->second].inputs[1];
    consumed.push_back(sub_it->second);
    const int mean_i = step(mean_name, "ReduceMean");
    if (mean_i < 0 || m.nodes[mean_i].inputs.empty() || m.nodes[mean_i].inputs[0] != x_name || !spatial_reduce(m.nodes[mean_i])) continue;
    consumed.push_back(mean_i);
    std::set<int> unique(consumed.begin(), consumed.end());
    if (unique.size() != consumed.size()) continue;
    bool free_nodes = true;
    for (int c : consumed) free_nodes = free_nodes && !claimed.count(c);
    if (!free_nodes) continue;
    const int anchor = *unique.begin();
    NodeDef fused;
    fused.op = "OxiInstanceNorm";
    fused.name = m.nodes[anchor].name + "_fused_instancenorm";
    fused.inputs = {x_name};
    fused.outputs = {norm.outputs[0]};
    fused.attrs.floats["epsilon"] = eps;
    for (int c : consumed) {
      claimed.insert(c);
      if (c != anchor) skip.insert(c);
    }
    auto ks = m.known_shapes.find(x_name);
    if (ks != m.known_shapes.end()) m.known_shapes[norm.outputs[0]] = ks->second;
    replace[anchor] = std::move(fused);
  }
  return apply(m, skip, replace);
}

// fuse_matmul_add (matmul_add.rs:34-132): MatMul of two rank-2 operands + Add of a rank-1 constant -> Gemm.
int fuse_matmul_add(Model& m) {
  if (m.nodes.size() < 2) return 0;
  infer_shapes(m);
  auto prod = producers(m);
  Usage usage(m);
  std::set<int> skip;
  std::map<int, NodeDef> replace;
  auto rank_of = [&](const std::string& name) -> int {
    auto it = m.known_shapes.find(name);
    return it == m.known_shapes.end() ? -1 : (int)it->second.size();
  };
  for (size_t i = 0; i < m.nodes.size(); ++i) {
    const NodeDef& add = m.nodes[i];
    if (add.op != "Add" || add.inputs.size() < 2) continue;
    if (!usage.fusable(add.inputs[0])) continue;
    auto pit = prod.find(add.inputs[0]);
    if (pit == prod.end()) continue;
    const int mi = pit->second;
    if (skip.count(mi) || replace.count(mi)) continue;
    const NodeDef& mm = m.nodes[mi];
    if (mm.op != "MatMul" || mm.inputs.size() < 2) continue;
    if (rank_of(mm.inputs[0]) != 2 || rank_of(mm.inputs[1]) != 2) continue;
    auto bias = m.initializers.find(add.inputs[1]);
    if (bias == m.initializers.end() || bias->second.shape.size() != 1) continue;
    NodeDef fused;
    fused.op = "Gemm";
    fused.name = mm.name + "_fused_gemm";
    fused.inputs = {mm.inputs[0], mm.inputs[1], add.inputs[1]};
    fused.outputs = add.outputs;
    fused.attrs.floats["alpha"] = 1.0f;
    fused.attrs.floats["beta"] = 1.0f;
    fused.attrs.ints["transA"] = 0;
    fused.attrs.ints["transB"] = 0;
    replace[mi] = std::move(fused);
    skip.insert((int)i);
  }
  return apply(m, skip, replace);
}

// fuse_conv_add_relu (add_relu.rs:27-156): Conv -> Add(residual) -> Relu becomes ConvAddRelu with inputs
// (x, w, bias or "", residual), the Conv's attributes and fused_ops = "Add,Relu"; node <name>_fused_conv_add_relu.
int fuse_conv_add_relu(Model& m) {
  if (m.nodes.size() < 3) return 0;
  auto prod = producers(m);
  Usage usage(m);
  std::set<int> skip;
  std::map<int, NodeDef> replace;
  for (size_t i = 0; i < m.nodes.size(); ++i) {
    const NodeDef& relu = m.nodes[i];
    if (relu.op != "Relu" || relu.inputs.empty()) continue;
    if (!usage.fusable(relu.inputs[0])) continue;
    auto ait = prod.find(relu.inputs[0]);
    if (ait == prod.end()) continue;
    const int ai = ait->second;
    if (skip.count(ai)) continue;
    const NodeDef& add = m.nodes[ai];
    if (add.op != "Add" || add.inputs.size() < 2) continue;
    int ci = -1;
    std::string residual;
    auto try_conv = [&](const std::string& conv_c, const std::string& res_c) -> bool {
      if (!usage.fusable(conv_c)) return false;
      auto it = prod.find(conv_c);
      if (it == prod.end() || skip.count(it->second) || replace.count(it->second)) return false;
      const NodeDef& c = m.nodes[it->second];
      if (c.op != "Conv" || !c.attrs.s("activation").empty()) return false;
      ci = it->second;
      residual = res_c;
      return true;
    };
    if (!try_conv(add.inputs[0], add.inputs[1]) && !try_conv(add.inputs[1], add.inputs[0])) continue;
    const NodeDef& conv = m.nodes[ci];
    if (conv.inputs.size() < 2) continue;
    NodeDef fused = conv;
    fused.op = "ConvAddRelu";
    fused.name = conv.name + "_fused_conv_add_relu";
    fused.inputs = {conv.inputs[0], conv.inputs[1], conv.inputs.size() > 2 ? conv.inputs[2] : std::string(), residual};
    fused.outputs = relu.outputs;
    fused.attrs.strings["fused_ops"] = "Add,Relu";
    replace[ci] = std::move(fused);
    skip.insert(ai);
    skip.insert((int)i);
  }
  const int removed = apply(m, skip, replace);
  if (removed) topo_sort(m);  // the residual may be produced after the convolution it now feeds
  return removed;
}

// fuse_mul_sigmoid_to_silu (src/optimizer/fusion/simplify/functions.rs:346-415): Mul(x, Sigmoid(x)) in either
// operand order -> SiLU(x); node <mul name>_fused_silu.
int fuse_mul_sigmoid_to_silu(Model& m) {
  if (m.nodes.size() < 2) return 0;
  auto prod = producers(m);
  Usage usage(m);
  std::set<int> skip;
  std::map<int, NodeDef> replace;
  for (size_t i = 0; i < m.nodes.size(); ++i) {
    const NodeDef& mul = m.nodes[i];
    if (mul.op != "Mul" || mul.inputs.size() < 2) continue;
    int si = -1;
    std::string x_name;
    auto try_order = [&](const std::string& sig_c, const std::string& x_c) -> bool {
      auto it = prod.find(sig_c);
      if (it == prod.end() || skip.count(it->second)) return false;
      const NodeDef& sg = m.nodes[it->second];
      if (sg.op != "Sigmoid" || !usage.fusable(sig_c) || sg.inputs.empty() || sg.inputs[0] != x_c) return false;
      si = it->second;
      x_name = x_c;
      return true;
    };
    if (!try_order(mul.inputs[1], mul.inputs[0]) && !try_order(mul.inputs[0], mul.inputs[1])) continue;
    NodeDef fused;
    fused.op = "SiLU";
    fused.name = mul.name + "_fused_silu";
    fused.inputs = {x_name};
    fused.outputs = mul.outputs;
    replace[(int)i] = std::move(fused);
    skip.insert(si);
  }
  return apply(m, skip, replace);
}

// The reference's order (src/optimizer/mod.rs:134-167).
int optimize_model(Model& m, int level) {
  if (level <= 0) return 0;
  int removed = 0;
  removed += fuse_matmul_add(m);
  removed += fuse_conv_batchnorm(m);
  removed += fuse_conv_relu(m);
  removed += fuse_conv_clip_to_relu6(m);
  removed += fuse_mul_sigmoid_to_silu(m);
  removed += fuse_instance_norm(m);
  removed += fuse_conv_add_relu(m);
  return removed;
}

}  // namespace oxb
