// extern "C" entry points for ONNX models (include/oxb200.h): load, optimise, inspect, plan.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <memory>

#include "abi_internal.hpp"
#include "model.hpp"

using namespace oxb;

struct oxb200_model {
  Model m;
  // C views of the nodes, rebuilt whenever the model changes
  struct NodeView {
    std::vector<const char*> inputs, outputs;
    std::vector<oxb200_attr> attrs;
    std::vector<std::string> attr_names;
  };
  std::vector<NodeView> views;
  std::vector<std::vector<uint64_t>> input_shapes, init_shapes;
  bool views_valid = false;
  void rebuild() {
    views.clear();
    views.resize(m.nodes.size());
    for (size_t i = 0; i < m.nodes.size(); ++i) {
      const NodeDef& n = m.nodes[i];
      NodeView& v = views[i];
      for (auto& s : n.inputs) v.inputs.push_back(s.c_str());
      for (auto& s : n.outputs) v.outputs.push_back(s.c_str());
      auto add = [&](const std::string& name, int kind) -> oxb200_attr& {
        oxb200_attr a;
        std::memset(&a, 0, sizeof a);
        a.kind = kind;
        v.attrs.push_back(a);
        v.attr_names.push_back(name);
        return v.attrs.back();
      };
      for (auto& kv : n.attrs.ints) add(kv.first, OXB200_ATTR_INT).i = kv.second;
      for (auto& kv : n.attrs.floats) add(kv.first, OXB200_ATTR_FLOAT).f = kv.second;
      for (auto& kv : n.attrs.strings) add(kv.first, OXB200_ATTR_STRING).s = kv.second.c_str();
      for (auto& kv : n.attrs.int_lists) {
        oxb200_attr& a = add(kv.first, OXB200_ATTR_INTS);
        a.ints = kv.second.data();
        a.len = kv.second.size();
      }
      for (auto& kv : n.attrs.float_lists) {
        oxb200_attr& a = add(kv.first, OXB200_ATTR_FLOATS);
        a.floats = kv.second.data();
        a.len = kv.second.size();
      }
      for (size_t k = 0; k < v.attrs.size(); ++k) v.attrs[k].name = v.attr_names[k].c_str();
    }
    input_shapes.clear();
    for (auto& in : m.inputs) {
      std::vector<uint64_t> sh;
      for (int64_t d : in.shape) sh.push_back(d < 0 ? UINT64_MAX : (uint64_t)d);
      input_shapes.push_back(sh);
    }
    init_shapes.clear();
    for (auto& name : m.initializer_order) {
      std::vector<uint64_t> sh;
      for (int64_t d : m.initializers[name].shape) sh.push_back((uint64_t)d);
      init_shapes.push_back(sh);
    }
    views_valid = true;
  }
};

namespace {

int model_fail(int code, const std::string& msg) {
  set_thread_error(msg);
  return code;
}

template <typename F>
int model_guarded(F&& f) {
  try {
    return f();
  } catch (const Error& e) {
    return model_fail(e.code, e.what());
  } catch (const std::exception& e) {
    return model_fail(OXB200_FAILED, e.what());
  } catch (...) {
    return model_fail(OXB200_FAILED, "unknown internal error");
  }
}

int dt_to_abi(DT d) {
  switch (d) {
    case DT::U8: return OXB200_DT_U8;
    case DT::I8: return OXB200_DT_I8;
    case DT::I32: return OXB200_DT_I32;
    case DT::F16: return OXB200_DT_F16;
    case DT::BF16: return OXB200_DT_BF16;
    default: return OXB200_DT_F32;
  }
}

}  // namespace

extern "C" {

int oxb200_model_load(const void* bytes, uint64_t len, oxb200_model** out) {
  if (!out) return model_fail(OXB200_FAILED, "model_load: out is NULL");
  *out = nullptr;
  return model_guarded([&]() {
    auto m = std::make_unique<oxb200_model>();
    m->m = load_onnx((const uint8_t*)bytes, (size_t)len);
    *out = m.release();
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_model_load_file(const char* path, oxb200_model** out) {
  if (!out || !path) return model_fail(OXB200_FAILED, "model_load_file: NULL argument");
  *out = nullptr;
  return model_guarded([&]() {
    std::ifstream fh(path, std::ios::binary | std::ios::ate);
    if (!fh) raise(OXB200_FAILED, "model_load_file: cannot open '%s'", path);
    const std::streamsize n = fh.tellg();
    fh.seekg(0);
    std::vector<uint8_t> buf((size_t)std::max<std::streamsize>(n, 0));
    if (n > 0 && !fh.read((char*)buf.data(), n)) raise(OXB200_FAILED, "model_load_file: cannot read '%s'", path);
    auto m = std::make_unique<oxb200_model>();
    m->m = load_onnx(buf.data(), buf.size());
    *out = m.release();
    return (int)OXB200_OK_HOST;
  });
}

void oxb200_model_free(oxb200_model* m) { delete m; }

int oxb200_model_optimize(oxb200_model* m, int32_t level, uint32_t* removed) {
  if (!m) return model_fail(OXB200_FAILED, "model_optimize: model is NULL");
  return model_guarded([&]() {
    const int r = optimize_model(m->m, level);
    m->views_valid = false;
    if (removed) *removed = (uint32_t)r;
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_model_run_pass(oxb200_model* m, const char* pass, uint32_t* removed) {
  if (!m || !pass) return model_fail(OXB200_FAILED, "model_run_pass: NULL argument");
  return model_guarded([&]() {
    const std::string p = pass;
    int r;
    if (p == "fuse_conv_batchnorm") r = fuse_conv_batchnorm(m->m);
    else if (p == "fuse_conv_relu") r = fuse_conv_relu(m->m);
    else if (p == "fuse_conv_clip_to_conv_relu6") r = fuse_conv_clip_to_relu6(m->m);
    else if (p == "fuse_instance_norm") r = fuse_instance_norm(m->m);
    else if (p == "fuse_matmul_add") r = fuse_matmul_add(m->m);
    else if (p == "fuse_mul_sigmoid_to_silu") r = fuse_mul_sigmoid_to_silu(m->m);
    else if (p == "fuse_conv_add_relu") r = fuse_conv_add_relu(m->m);
    else raise(OXB200_FAILED, "model_run_pass: no pass named '%s'", pass);
    m->views_valid = false;
    if (removed) *removed = (uint32_t)r;
    return (int)OXB200_OK_HOST;
  });
}

uint32_t oxb200_model_node_count(const oxb200_model* m) { return m ? (uint32_t)m->m.nodes.size() : 0; }

int oxb200_model_node(oxb200_model* m, uint32_t index, oxb200_node* out) {
  if (!m || !out || index >= m->m.nodes.size()) return model_fail(OXB200_FAILED, "model_node: bad argument");
  if (!m->views_valid) m->rebuild();
  const NodeDef& n = m->m.nodes[index];
  const oxb200_model::NodeView& v = m->views[index];
  out->op_type = n.op.c_str();
  out->name = n.name.c_str();
  out->inputs = v.inputs.data();
  out->n_inputs = (uint32_t)v.inputs.size();
  out->outputs = v.outputs.data();
  out->n_outputs = (uint32_t)v.outputs.size();
  out->attrs = v.attrs.data();
  out->n_attrs = (uint32_t)v.attrs.size();
  return OXB200_OK_HOST;
}

uint32_t oxb200_model_input_count(const oxb200_model* m) { return m ? (uint32_t)m->m.inputs.size() : 0; }

int oxb200_model_input(oxb200_model* m, uint32_t index, oxb200_value_info* out) {
  if (!m || !out || index >= m->m.inputs.size()) return model_fail(OXB200_FAILED, "model_input: bad argument");
  if (!m->views_valid) m->rebuild();
  out->name = m->m.inputs[index].name.c_str();
  out->shape = m->input_shapes[index].data();
  out->rank = (uint32_t)m->input_shapes[index].size();
  DT dt;
  out->dtype = onnx_dtype_to_dt(m->m.inputs[index].onnx_dtype, &dt) ? dt_to_abi(dt) : -1;
  return OXB200_OK_HOST;
}

uint32_t oxb200_model_output_count(const oxb200_model* m) { return m ? (uint32_t)m->m.outputs.size() : 0; }

const char* oxb200_model_output_name(const oxb200_model* m, uint32_t index) {
  return (m && index < m->m.outputs.size()) ? m->m.outputs[index].name.c_str() : nullptr;
}

uint32_t oxb200_model_initializer_count(const oxb200_model* m) { return m ? (uint32_t)m->m.initializer_order.size() : 0; }

int oxb200_model_initializer(oxb200_model* m, uint32_t index, oxb200_operand* out) {
  if (!m || !out || index >= m->m.initializer_order.size()) return model_fail(OXB200_FAILED, "model_initializer: bad argument");
  if (!m->views_valid) m->rebuild();
  const std::string& name = m->m.initializer_order[index];
  const HostTensor& t = m->m.initializers[name];
  std::memset(out, 0, sizeof *out);
  out->name = name.c_str();
  out->lanes = t.data.data();
  out->len = t.data.size();
  out->shape = m->init_shapes[index].data();
  out->rank = (uint32_t)m->init_shapes[index].size();
  out->dtype = dt_to_abi(t.declared);
  return OXB200_OK_HOST;
}

int oxb200_session_plan_model(oxb200_ctx* ctx, oxb200_model* m, const oxb200_value_info* shapes, uint32_t n_shapes) {
  if (!ctx || !m) return model_fail(OXB200_FAILED, "session_plan_model: NULL argument");
  auto fail_ctx = [&](int code, const std::string& msg) {
    ctx->impl.last_error = msg;
    if (code == OXB200_DECLINED) ctx->impl.counters.declines++;
    else ctx->impl.counters.failures++;
    return model_fail(code, msg);
  };
  try {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    Context& C = ctx->impl;
    C.make_current();
    C.session.reset();
    // the model's initializers are the context's weights, with their declared element types
    for (const std::string& name : m->m.initializer_order) {
      const HostTensor& t = m->m.initializers[name];
      bool used = false;
      for (const NodeDef& n : m->m.nodes)
        for (const std::string& in : n.inputs) used = used || in == name;
      if (!used) continue;  // folded away by a pass
      std::vector<uint64_t> sh(t.shape.begin(), t.shape.end());
      C.register_weight(name, t.data.data(), t.data.size(), sh.data(), (uint32_t)sh.size(), t.declared);
    }
    std::vector<std::pair<std::string, std::vector<int64_t>>> in;
    auto sess = std::make_unique<Session>(&C);
    for (const ModelValueInfo& vi : m->m.inputs) {
      std::vector<int64_t> sh = vi.shape;
      for (uint32_t k = 0; k < n_shapes; ++k)
        if (shapes && shapes[k].name && vi.name == shapes[k].name) sh.assign(shapes[k].shape, shapes[k].shape + shapes[k].rank);
      for (int64_t d : sh)
        if (d < 0) raise(OXB200_FAILED, "session_plan_model: input '%s' has a symbolic dimension; pass its concrete shape", vi.name.c_str());
      DT dt;
      if (!onnx_dtype_to_dt(vi.onnx_dtype, &dt) || !(dt == DT::F32 || dt == DT::U8 || dt == DT::I8))
        raise(OXB200_DECLINED, "session_plan_model: input '%s' has ONNX element type %d, which the boundary does not take", vi.name.c_str(), (int)vi.onnx_dtype);
      sess->declare_input_type(vi.name, dt);
      in.push_back({vi.name, sh});
    }
    std::vector<std::string> outs;
    for (const ModelValueInfo& o : m->m.outputs) outs.push_back(o.name);
    std::map<std::string, const HostTensor*> none;
    sess->plan(m->m.nodes, in, none, outs);
    sess->allow_graph(true);
    C.session = std::move(sess);
    return (int)OXB200_OK_DEVICE;
  } catch (const Error& e) {
    return fail_ctx(e.code, e.what());
  } catch (const std::exception& e) {
    return fail_ctx(OXB200_FAILED, e.what());
  }
}

}  // extern "C"
