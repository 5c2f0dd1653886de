// extern "C" boundary of the oxb200 provider (include/oxb200.h).  Every entry point converts
// internal errors into a status plus a message; nothing throws across the boundary.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "runtime.hpp"

using namespace oxb;

#include "abi_internal.hpp"

namespace {

thread_local std::string g_thread_error;

}  // namespace

namespace oxb {
void set_thread_error(const std::string& message) { g_thread_error = message; }
}  // namespace oxb

namespace {


// The proved-wrong marker of the reference (oxionnx-cuda src/error.rs:75).
const char kVerifyPrefix[] = "CUDA VERIFY MISMATCH: ";

int fail_with(oxb200_ctx* ctx, int code, const std::string& msg) {
  g_thread_error = msg;
  if (ctx) {
    ctx->impl.last_error = msg;
    if (code == OXB200_DECLINED) ctx->impl.counters.declines++;
    else ctx->impl.counters.failures++;
  }
  return code;
}

template <typename F>
int guarded(oxb200_ctx* ctx, F&& f) {
  try {
    return f();
  } catch (const Error& e) {
    return fail_with(ctx, e.code, e.what());
  } catch (const std::exception& e) {
    return fail_with(ctx, OXB200_FAILED, e.what());
  } catch (...) {
    return fail_with(ctx, OXB200_FAILED, "unknown internal error");
  }
}

NodeDef to_node(const oxb200_node* n) {
  NodeDef d;
  if (!n || !n->op_type) raise(OXB200_FAILED, "node or op_type is NULL");
  d.op = n->op_type;
  d.name = n->name ? n->name : "";
  for (uint32_t i = 0; i < n->n_inputs; ++i) d.inputs.push_back(n->inputs[i] ? n->inputs[i] : "");
  for (uint32_t i = 0; i < n->n_outputs; ++i) d.outputs.push_back(n->outputs[i] ? n->outputs[i] : "");
  for (uint32_t i = 0; i < n->n_attrs; ++i) {
    const oxb200_attr& a = n->attrs[i];
    if (!a.name) raise(OXB200_FAILED, "attribute %u has no name", i);
    switch (a.kind) {
      case OXB200_ATTR_INT: d.attrs.ints[a.name] = a.i; break;
      case OXB200_ATTR_FLOAT: d.attrs.floats[a.name] = a.f; break;
      case OXB200_ATTR_STRING: d.attrs.strings[a.name] = a.s ? a.s : ""; break;
      case OXB200_ATTR_INTS: d.attrs.int_lists[a.name] = std::vector<int64_t>(a.ints, a.ints + a.len); break;
      case OXB200_ATTR_FLOATS: d.attrs.float_lists[a.name] = std::vector<float>(a.floats, a.floats + a.len); break;
      default: raise(OXB200_DECLINED, "attribute '%s' has a kind this provider does not handle", a.name);
    }
  }
  return d;
}

}  // namespace

extern "C" {

int oxb200_is_supported_op(const char* op_type) { return op_type && is_supported_op(op_type) ? 1 : 0; }

int oxb200_accepts_resident_slot(const char* op_type, uint32_t slot) { return op_type && accepts_resident_slot(op_type, slot) ? 1 : 0; }

// decide_placement (root crate src/execution_providers.rs:352-387) seen from this provider.
int oxb200_decide_placement(int policy, uint64_t gpu_threshold_bytes, int manual_pin, const char* op_type, uint64_t output_bytes) {
  const uint64_t kMinGpuDispatchBytes = 4096;  // MIN_GPU_DISPATCH_BYTES (src/execution_providers.rs:207)
  if (!op_type) return 0;
  switch (policy) {
    case 0: return 0;  // CpuOnly
    case 1:            // Auto { gpu_threshold_bytes }
      if (output_bytes < gpu_threshold_bytes) return 0;
      return is_supported_op(op_type) ? 1 : 0;
    case 2:  // Manual(map)
      if (manual_pin != 2) return 0;
      if (output_bytes < kMinGpuDispatchBytes) return 0;
      return 1;
    default: return 0;
  }
}

int oxb200_is_verify_mismatch(const char* message) { return message && std::strncmp(message, kVerifyPrefix, sizeof(kVerifyPrefix) - 1) == 0 ? 1 : 0; }

// env_flag (oxionnx-cuda src/context.rs:179-192): unset, empty, 0, false, off, no are off;
// anything else, including unrecognised text, is on.
int oxb200_env_truthy(const char* value) {
  if (!value) return 0;
  std::string v(value);
  size_t b = v.find_first_not_of(" \t\r\n"), e = v.find_last_not_of(" \t\r\n");
  if (b == std::string::npos) return 0;
  v = v.substr(b, e - b + 1);
  std::transform(v.begin(), v.end(), v.begin(), [](unsigned char c) { return (char)std::tolower(c); });
  if (v.empty() || v == "0" || v == "false" || v == "off" || v == "no") return 0;
  return 1;
}

void oxb200_config_from_env(oxb200_config* cfg) {
  if (!cfg) return;
  std::memset(cfg, 0, sizeof(*cfg));
  cfg->struct_size = sizeof(*cfg);
  cfg->verify = oxb200_env_truthy(std::getenv("OXIONNX_CUDA_VERIFY"));
  cfg->strict = oxb200_env_truthy(std::getenv("OXIONNX_CUDA_STRICT"));
  const char* res = std::getenv("OXIONNX_CUDA_RESIDENCY");
  cfg->residency = res ? oxb200_env_truthy(res) : 1;
  cfg->cuda_graph = oxb200_env_truthy(std::getenv("OXIONNX_CUDA_GRAPH"));
  const char* kp = std::getenv("OXB200_KERNEL_PATH");
  cfg->kernel_path = (kp && std::string(kp) == "direct") ? 1 : 0;
}

int oxb200_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return n;
}

int oxb200_ctx_create(int device_ordinal, const oxb200_config* cfg, oxb200_ctx** out) {
  if (!out) return fail_with(nullptr, OXB200_FAILED, "ctx_create: out is NULL");
  *out = nullptr;
  return guarded(nullptr, [&]() {
    oxb200_config c;
    std::memset(&c, 0, sizeof c);
    c.residency = 1;
    if (cfg) std::memcpy(&c, cfg, std::min<size_t>(sizeof c, cfg->struct_size ? cfg->struct_size : sizeof c));
    *out = new oxb200_ctx(device_ordinal, c);
    return (int)OXB200_OK_HOST;
  });
}

void oxb200_ctx_destroy(oxb200_ctx* ctx) { delete ctx; }

const char* oxb200_last_error(const oxb200_ctx* ctx) { return ctx ? ctx->impl.last_error.c_str() : g_thread_error.c_str(); }

void oxb200_get_counters(const oxb200_ctx* ctx, oxb200_counters* out) {
  if (ctx && out) *out = ctx->impl.counters;
}

int oxb200_release_device_caches(oxb200_ctx* ctx) {
  if (!ctx) return OXB200_FAILED;
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    ctx->impl.make_current();
    ctx->impl.session.reset();
    ctx->impl.release_caches();
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_set_profile(oxb200_ctx* ctx, int on) {
  if (!ctx) return OXB200_FAILED;
  std::lock_guard<std::mutex> lock(ctx->impl.mu);
  ctx->impl.set_profile(on);
  return OXB200_OK_HOST;
}

int oxb200_probe_tensor_peak(oxb200_ctx* ctx, int32_t kind, double* ops_per_second) {
  if (!ctx || !ops_per_second) return fail_with(ctx, OXB200_FAILED, "probe_tensor_peak: NULL argument");
  if (kind < 0 || kind > 3) return fail_with(ctx, OXB200_FAILED, "probe_tensor_peak: kind must be 0 (i8), 1 (tf32), 2 (f16) or 3 (bf16)");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    Context& C = ctx->impl;
    C.make_current();
    int* err = (int*)C.alloc_device(256);
    OXB_CUDA(cudaMemsetAsync(err, 0, 256, C.stream()));
    double rate = 0.0;
    int flag = 0;
    try {
      rate = k::umma_probe_peak(kind, err, C.stream());
      OXB_CUDA(cudaMemcpy(&flag, err, sizeof(int), cudaMemcpyDeviceToHost));
    } catch (...) {
      C.free_device(err);
      throw;
    }
    C.free_device(err);
    if (flag != 0) raise(OXB200_FAILED, "probe_tensor_peak: a bounded wait ran out (code %d)", flag);
    *ops_per_second = rate;
    return (int)OXB200_OK_HOST;
  });
}

void* oxb200_host_alloc(size_t bytes) {
  void* p = nullptr;
  if (cudaMallocHost(&p, bytes ? bytes : 1) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return p;
}

void oxb200_host_free(void* p) {
  if (p) cudaFreeHost(p);
}

int oxb200_weight_register(oxb200_ctx* ctx, const char* name, const float* lanes, uint64_t len, const uint64_t* shape, uint32_t rank) {
  if (!ctx || !name || (!lanes && len)) return fail_with(ctx, OXB200_FAILED, "weight_register: NULL argument");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    ctx->impl.register_weight(name, lanes, len, shape, rank);
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_weight_register_typed(oxb200_ctx* ctx, const char* name, const float* lanes, uint64_t len, const uint64_t* shape, uint32_t rank, int32_t dtype) {
  if (!ctx || !name || (!lanes && len)) return fail_with(ctx, OXB200_FAILED, "weight_register_typed: NULL argument");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    DT declared = DT::F32;
    switch (dtype) {
      case OXB200_DT_U8: declared = DT::U8; break;
      case OXB200_DT_I8: declared = DT::I8; break;
      case OXB200_DT_I32: declared = DT::I32; break;
      case OXB200_DT_F16: declared = DT::F16; break;
      case OXB200_DT_BF16: declared = DT::BF16; break;
      default: declared = DT::F32; break;
    }
    ctx->impl.register_weight(name, lanes, len, shape, rank, declared);
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_is_weight_resident(const oxb200_ctx* ctx, const char* name) { return ctx && name && ctx->impl.weight_resident(name) ? 1 : 0; }

int oxb200_tensor_shape(const oxb200_tensor* t, uint64_t* shape, uint32_t* rank, uint64_t* len) {
  if (!t) return OXB200_FAILED;
  if (rank) *rank = (uint32_t)t->h.shape.size();
  if (shape)
    for (size_t d = 0; d < t->h.shape.size() && d < OXB200_MAX_RANK; ++d) shape[d] = (uint64_t)t->h.shape[d];
  if (len) *len = (uint64_t)prod(t->h.shape);
  return OXB200_OK_HOST;
}

int oxb200_tensor_read_back(oxb200_ctx* ctx, const oxb200_tensor* t, float* dst_lanes, uint64_t cap) {
  if (!ctx || !t || !dst_lanes) return fail_with(ctx, OXB200_FAILED, "tensor_read_back: NULL argument");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    Context& C = ctx->impl;
    C.make_current();
    int64_t n = prod(t->h.shape);
    if ((uint64_t)n > cap) raise(OXB200_FAILED, "tensor_read_back: destination holds %llu lanes, %lld needed", (unsigned long long)cap, (long long)n);
    if (n == 0) return (int)OXB200_OK_HOST;
    void* tmp = C.alloc_device((size_t)n * 4);
    k::Dims4 d = t->h.shape.size() == 4 ? k::Dims4{t->h.shape[0], t->h.shape[1], t->h.shape[2], t->h.shape[3]} : k::Dims4{n, 1, 1, 1};
    k::TensorRef src{t->h.ptr, t->h.dt, t->h.shape.size() == 4 ? t->h.layout : Layout::PLAIN, d};
    k::TensorRef dst{tmp, DT::F32, Layout::PLAIN, d};
    k::convert(src, dst, C.stream());
    OXB_CUDA(cudaMemcpyAsync(dst_lanes, tmp, (size_t)n * 4, cudaMemcpyDeviceToHost, C.stream()));
    OXB_CUDA(cudaStreamSynchronize(C.stream()));
    C.free_device(tmp);
    C.counters.downloads++;
    C.counters.download_bytes += (uint64_t)n * 4;
    C.counters.fences++;
    return (int)OXB200_OK_HOST;
  });
}

void oxb200_tensor_release(oxb200_ctx* ctx, oxb200_tensor* t) {
  if (!t) return;
  if (ctx) {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    cudaSetDevice(ctx->impl.device());
    cudaStreamSynchronize(ctx->impl.stream());
  }
  // an allocation shared with aliases (oxb200_tensor_alias) lives until its last handle is released
  if (t->h.ptr && t->h.owners.use_count() == 1) cudaFree(t->h.ptr);
  delete t;
}

int oxb200_tensor_alias(oxb200_ctx* ctx, const oxb200_tensor* t, const uint64_t* shape, uint32_t rank, oxb200_tensor** out) {
  if (!t || !out || (!shape && rank) || rank > OXB200_MAX_RANK) return fail_with(ctx, OXB200_FAILED, "tensor_alias: bad argument");
  *out = nullptr;
  // CudaDeviceTensor::alias returns None when the element counts differ; so does this (DECLINED)
  uint64_t len = 1;
  for (uint32_t d = 0; d < rank; ++d) {
    if (shape[d] != 0 && len > UINT64_MAX / shape[d]) return fail_with(ctx, OXB200_DECLINED, "tensor_alias: the shape's element count overflows");
    len *= shape[d];
  }
  if (len != (uint64_t)prod(t->h.shape)) return fail_with(ctx, OXB200_DECLINED, "tensor_alias: the shape has another element count");
  // the lanes of a rank-4 value are stored channels-last: another shape over the same bytes is the same tensor
  // only when the two orders coincide (one channel, or a 1x1 plane) -- otherwise the caller reads back and reshapes
  const std::vector<int64_t>& s0 = t->h.shape;
  const bool order_free = s0.size() != 4 || t->h.layout == Layout::PLAIN || s0[1] == 1 || (s0[2] == 1 && s0[3] == 1);
  if (!order_free) return fail_with(ctx, OXB200_DECLINED, "tensor_alias: the tensor is stored channels-last; its bytes are not in the order of the new shape");
  bool new_order_free = rank != 4 || shape[1] == 1 || (shape[2] == 1 && shape[3] == 1);
  if (!new_order_free && t->h.layout != Layout::PLAIN) return fail_with(ctx, OXB200_DECLINED, "tensor_alias: a rank-4 view of these bytes would be read channels-last");
  oxb200_tensor* a = new oxb200_tensor();
  a->h = t->h;  // shares `owners`
  a->h.shape.assign(shape, shape + rank);
  if (rank == 4 && !new_order_free) a->h.layout = Layout::PLAIN;
  *out = a;
  return OXB200_OK_DEVICE;
}

uint64_t oxb200_tensor_reserved_bytes(const oxb200_tensor* t) { return t ? (uint64_t)t->h.bytes : 0; }

int oxb200_streams_unified(const oxb200_ctx* ctx) { return ctx ? 1 : 0; }

uint64_t oxb200_cached_device_bytes(oxb200_ctx* ctx) {
  if (!ctx) return 0;
  std::lock_guard<std::mutex> lock(ctx->impl.mu);
  return ctx->impl.cached_bytes();
}

int oxb200_set_graph_capture(oxb200_ctx* ctx, int on) {
  if (!ctx) return OXB200_FAILED;
  std::lock_guard<std::mutex> lock(ctx->impl.mu);
  ctx->impl.set_graph_capture(on);
  return OXB200_OK_HOST;
}

int oxb200_graph_capture_enabled(const oxb200_ctx* ctx) { return ctx && ctx->impl.cfg().cuda_graph && !ctx->impl.cfg().verify ? 1 : 0; }

int oxb200_dispatch(oxb200_ctx* ctx, const oxb200_node* node, const oxb200_operand* operands, uint32_t n_operands, int want_placement,
                    oxb200_result* results, uint32_t n_results) {
  if (!ctx || !node || (!operands && n_operands) || !results) return fail_with(ctx, OXB200_FAILED, "dispatch: NULL argument");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    Context& C = ctx->impl;
    C.make_current();
    C.counters.dispatches++;
    NodeDef nd = to_node(node);
    if (!is_supported_op(nd.op)) raise(OXB200_DECLINED, "operator '%s' is not claimed by this provider", nd.op.c_str());
    if (n_operands != nd.inputs.size()) raise(OXB200_FAILED, "dispatch: %u operands for %zu node inputs", n_operands, nd.inputs.size());
    if (n_results != nd.outputs.size()) raise(OXB200_FAILED, "dispatch: %u result slots for %zu node outputs", n_results, nd.outputs.size());
    // operands: registered weights by name, host lanes as plan-time constants, resident tensors as bound inputs
    std::vector<HostTensor> temps;
    temps.reserve(n_operands);
    std::map<std::string, const HostTensor*> vconsts;
    std::vector<std::pair<std::string, std::vector<int64_t>>> inputs;
    Session sess(&C);
    for (uint32_t i = 0; i < n_operands; ++i) {
      const std::string& nm = nd.inputs[i];
      if (nm.empty()) continue;
      const oxb200_operand& o = operands[i];
      if (o.resident) {
        if (!accepts_resident_slot(nd.op, i)) raise(OXB200_DECLINED, "%s: operand %u cannot be bound from the device", nd.op.c_str(), i);
        inputs.push_back({nm, o.resident->h.shape});
        sess.bind_external(nm, o.resident->h.ptr, o.resident->h.dt, o.resident->h.layout);
        continue;
      }
      if (!o.lanes && o.typed && (o.dtype == OXB200_DT_U8 || o.dtype == OXB200_DT_I8)) {
        // a typed 8-bit operand (TypedTensor): exact integers as f32 lanes, the declared type kept beside them
        HostTensor t;
        t.shape.assign(o.shape, o.shape + o.rank);
        if ((uint64_t)prod(t.shape) != o.len) raise(OXB200_DECLINED, "%s: operand %u data length %llu does not match its shape", nd.op.c_str(), i, (unsigned long long)o.len);
        t.data.resize(o.len);
        for (uint64_t e = 0; e < o.len; ++e) t.data[e] = o.dtype == OXB200_DT_U8 ? (float)((const uint8_t*)o.typed)[e] : (float)((const int8_t*)o.typed)[e];
        t.declared = o.dtype == OXB200_DT_U8 ? DT::U8 : DT::I8;
        temps.push_back(std::move(t));
        vconsts[nm] = &temps.back();
        continue;
      }
      if (!o.lanes) {
        if (!C.weight(nm)) raise(OXB200_FAILED, "dispatch: operand '%s' has no lanes and is not a registered weight", nm.c_str());
        continue;
      }
      if (C.weight(nm) && vconsts.find(nm) == vconsts.end()) {
        const HostTensor* wt = C.weight(nm);
        // the weight map is invariant for the context's life; a mismatch means it was swapped
        if (wt->data.size() != o.len) raise(OXB200_FAILED, "dispatch: operand '%s' disagrees with the registered weight of that name", nm.c_str());
        continue;
      }
      HostTensor t;
      t.shape.assign(o.shape, o.shape + o.rank);
      t.data.assign(o.lanes, o.lanes + o.len);  // a length that disagrees with the shape is the operator's own error: decline below
      if ((uint64_t)prod(t.shape) != o.len) raise(OXB200_DECLINED, "%s: operand %u data length %llu does not match its shape", nd.op.c_str(), i, (unsigned long long)o.len);
      temps.push_back(std::move(t));
      vconsts[nm] = &temps.back();
    }
    std::vector<std::string> outs;
    const bool to_device = want_placement == OXB200_PLACE_DEVICE && nd.outputs.size() == 1 && C.cfg().residency != 0;
    if (!to_device)
      for (auto& o : nd.outputs)
        if (!o.empty()) outs.push_back(o);
    std::vector<NodeDef> nodes = {nd};
    struct Cleanup {
      Context& c;
      ~Cleanup() { c.free_temp_forms(); }
    } cleanup{C};
    sess.plan(nodes, inputs, vconsts, outs);
    sess.run_steps(false);
    if (to_device) {
      Value* v = sess.find_value(nd.outputs[0]);
      if (!v || !v->ptr) raise(OXB200_FAILED, "dispatch: output '%s' was not produced", nd.outputs[0].c_str());
      auto* t = new oxb200_tensor();
      t->h.bytes = std::max<size_t>(v->bytes, 256);
      t->h.dt = v->dt;
      t->h.layout = v->shape.size() == 4 ? v->layout : Layout::PLAIN;
      t->h.shape = v->shape;
      t->h.ptr = C.alloc_device(t->h.bytes);
      if (v->bytes) OXB_CUDA(cudaMemcpyAsync(t->h.ptr, v->ptr, v->bytes, cudaMemcpyDeviceToDevice, C.stream()));
      sess.sync();
      int flag = sess.check_error_flag();
      if (flag) {
        cudaFree(t->h.ptr);
        delete t;
        raise(OXB200_FAILED, flag == 20 ? "Gather: an index is out of range (device code %d)" : "a tensor-core kernel gave up on a bounded wait (code %d)", flag);
      }
      results[0].resident = t;
      results[0].rank = (uint32_t)v->shape.size();
      for (size_t d = 0; d < v->shape.size() && d < OXB200_MAX_RANK; ++d) results[0].shape[d] = (uint64_t)v->shape[d];
      results[0].len = (uint64_t)v->numel();
      return (int)OXB200_OK_DEVICE;
    }
    // host results, positionally aligned with node outputs (elided outputs keep len 0)
    std::vector<oxb200_result> fetch(outs.size());
    std::vector<uint32_t> slot_of;
    for (uint32_t i = 0; i < nd.outputs.size(); ++i)
      if (!nd.outputs[i].empty()) slot_of.push_back(i);
    for (size_t j = 0; j < outs.size(); ++j) fetch[j] = results[slot_of[j]];
    sess.download(fetch.data(), (uint32_t)fetch.size());
    for (size_t j = 0; j < outs.size(); ++j) {
      results[slot_of[j]] = fetch[j];
      results[slot_of[j]].resident = nullptr;
    }
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_session_plan(oxb200_ctx* ctx, const oxb200_node* nodes, uint32_t n_nodes, const oxb200_value_info* inputs, uint32_t n_inputs,
                        const char* const* outputs, uint32_t n_outputs) {
  if (!ctx || (!nodes && n_nodes) || (!inputs && n_inputs) || (!outputs && n_outputs)) return fail_with(ctx, OXB200_FAILED, "session_plan: NULL argument");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    Context& C = ctx->impl;
    C.make_current();
    C.session.reset();
    std::vector<NodeDef> nd;
    for (uint32_t i = 0; i < n_nodes; ++i) nd.push_back(to_node(&nodes[i]));
    std::vector<std::pair<std::string, std::vector<int64_t>>> in;
    for (uint32_t i = 0; i < n_inputs; ++i) {
      std::vector<int64_t> sh(inputs[i].shape, inputs[i].shape + inputs[i].rank);
      in.push_back({inputs[i].name, sh});
    }
    auto declared_dt = [](int32_t d, const char* name) -> DT {
      switch (d) {
        case OXB200_DT_F32: return DT::F32;
        case OXB200_DT_U8: return DT::U8;
        case OXB200_DT_I8: return DT::I8;
        default: raise(OXB200_DECLINED, "graph input '%s': element type %d is not taken at the boundary", name, (int)d);
      }
    };
    std::vector<std::string> outs;
    for (uint32_t i = 0; i < n_outputs; ++i) outs.push_back(outputs[i]);
    auto sess = std::make_unique<Session>(&C);
    for (uint32_t i = 0; i < n_inputs; ++i) sess->declare_input_type(inputs[i].name, declared_dt(inputs[i].dtype, inputs[i].name));
    std::map<std::string, const HostTensor*> none;
    sess->plan(nd, in, none, outs);
    sess->allow_graph(true);
    C.session = std::move(sess);
    return (int)OXB200_OK_DEVICE;
  });
}

static Session& planned(oxb200_ctx* ctx) {
  if (!ctx->impl.session) raise(OXB200_FAILED, "no session has been planned on this context");
  return *ctx->impl.session;
}

int oxb200_run(oxb200_ctx* ctx, const oxb200_operand* feeds, uint32_t n_feeds, oxb200_result* fetches, uint32_t n_fetches) {
  if (!ctx) return fail_with(ctx, OXB200_FAILED, "run: ctx is NULL");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    ctx->impl.make_current();
    Session& s = planned(ctx);
    Context& C = ctx->impl;
    if (!C.run_ev0) {
      OXB_CUDA(cudaEventCreate(&C.run_ev0));
      OXB_CUDA(cudaEventCreate(&C.run_ev1));
    }
    OXB_CUDA(cudaEventRecord(C.run_ev0, C.stream()));
    s.upload(feeds, n_feeds);
    s.run_steps(C.cfg().profile != 0);
    s.download_async(fetches, n_fetches);
    OXB_CUDA(cudaEventRecord(C.run_ev1, C.stream()));
    s.finish_download();
    float ms = -1.f;
    if (cudaEventElapsedTime(&ms, C.run_ev0, C.run_ev1) == cudaSuccess) C.last_run_ms = ms;
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_run_submit(oxb200_ctx* ctx, const oxb200_operand* feeds, uint32_t n_feeds) {
  if (!ctx) return fail_with(ctx, OXB200_FAILED, "run_submit: ctx is NULL");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    ctx->impl.make_current();
    Session& s = planned(ctx);
    s.submit(feeds, n_feeds, ctx->impl.cfg().profile != 0);
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_run_collect(oxb200_ctx* ctx, oxb200_result* fetches, uint32_t n_fetches) {
  if (!ctx) return fail_with(ctx, OXB200_FAILED, "run_collect: ctx is NULL");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    ctx->impl.make_current();
    Session& s = planned(ctx);
    s.collect(fetches, n_fetches);
    return (int)OXB200_OK_HOST;
  });
}

float oxb200_last_run_ms(const oxb200_ctx* ctx) { return ctx ? ctx->impl.last_run_ms : -1.f; }

// ---- device I/O binding (IoBinding / run_with_binding over device memory) ----
int oxb200_bind_input_device(oxb200_ctx* ctx, const char* name, const void* device_ptr, int32_t dtype, uint64_t len) {
  if (!ctx || !name) return fail_with(ctx, OXB200_FAILED, "bind_input_device: NULL argument");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    ctx->impl.make_current();
    DT dt;
    switch (dtype) {
      case OXB200_DT_F32: dt = DT::F32; break;
      case OXB200_DT_U8: dt = DT::U8; break;
      case OXB200_DT_I8: dt = DT::I8; break;
      default: raise(OXB200_FAILED, "bind_input_device: element type %d is not taken at the boundary", (int)dtype);
    }
    planned(ctx).bind_input_device(name, device_ptr, dt, len);
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_bind_output_device(oxb200_ctx* ctx, const char* name, void* device_ptr, uint64_t cap) {
  if (!ctx || !name) return fail_with(ctx, OXB200_FAILED, "bind_output_device: NULL argument");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    ctx->impl.make_current();
    planned(ctx).bind_output_device(name, device_ptr, cap);
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_output_device_ptr(oxb200_ctx* ctx, const char* name, void** device_ptr, uint64_t* len) {
  if (!ctx || !name) return fail_with(ctx, OXB200_FAILED, "output_device_ptr: NULL argument");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    planned(ctx).output_device_ptr(name, device_ptr, len);
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_run_bound(oxb200_ctx* ctx, const oxb200_operand* feeds, uint32_t n_feeds, oxb200_result* fetches, uint32_t n_fetches) {
  if (!ctx) return fail_with(ctx, OXB200_FAILED, "run_bound: ctx is NULL");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    ctx->impl.make_current();
    planned(ctx).run_bound(feeds, n_feeds, fetches, n_fetches, ctx->impl.cfg().profile != 0);
    return (int)OXB200_OK_DEVICE;
  });
}

int oxb200_clear_bindings(oxb200_ctx* ctx) {
  if (!ctx) return fail_with(ctx, OXB200_FAILED, "clear_bindings: ctx is NULL");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    ctx->impl.make_current();
    planned(ctx).clear_bindings();
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_upload_feeds(oxb200_ctx* ctx, const oxb200_operand* feeds, uint32_t n_feeds) {
  if (!ctx) return fail_with(ctx, OXB200_FAILED, "upload_feeds: ctx is NULL");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    ctx->impl.make_current();
    Session& s = planned(ctx);
    s.upload(feeds, n_feeds);
    s.sync();
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_run_resident(oxb200_ctx* ctx, uint32_t iters, float* elapsed_ms) {
  if (!ctx) return fail_with(ctx, OXB200_FAILED, "run_resident: ctx is NULL");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    Context& C = ctx->impl;
    C.make_current();
    Session& s = planned(ctx);
    cudaEvent_t e0, e1;
    OXB_CUDA(cudaEventCreate(&e0));
    OXB_CUDA(cudaEventCreate(&e1));
    OXB_CUDA(cudaEventRecord(e0, C.stream()));
    for (uint32_t i = 0; i < iters; ++i) s.run_steps(C.cfg().profile != 0 && i + 1 == iters);
    OXB_CUDA(cudaEventRecord(e1, C.stream()));
    s.sync();
    float ms = 0.f;
    OXB_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (elapsed_ms) *elapsed_ms = ms;
    if (C.cfg().profile)
      for (auto& st : s.steps())
        if (st.ev0 && st.ev1) {
          float t = -1.f;
          if (cudaEventElapsedTime(&t, st.ev0, st.ev1) == cudaSuccess) st.last_ms = t;
        }
    int flag = s.check_error_flag();
    if (flag) raise(OXB200_FAILED, flag == 20 ? "Gather: an index is out of range (device code %d); results are not valid" : "a tensor-core kernel gave up on a bounded wait (code %d); results are not valid", flag);
    return (int)OXB200_OK_DEVICE;
  });
}

int oxb200_download_fetches(oxb200_ctx* ctx, oxb200_result* fetches, uint32_t n_fetches) {
  if (!ctx) return fail_with(ctx, OXB200_FAILED, "download_fetches: ctx is NULL");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    ctx->impl.make_current();
    planned(ctx).download(fetches, n_fetches);
    return (int)OXB200_OK_HOST;
  });
}

int oxb200_fetch_value(oxb200_ctx* ctx, const char* name, oxb200_result* out) {
  if (!ctx || !name || !out) return fail_with(ctx, OXB200_FAILED, "fetch_value: NULL argument");
  return guarded(ctx, [&]() {
    std::lock_guard<std::mutex> lock(ctx->impl.mu);
    ctx->impl.make_current();
    planned(ctx).fetch_value(name, out);
    return (int)OXB200_OK_HOST;
  });
}

uint32_t oxb200_plan_step_count(const oxb200_ctx* ctx) {
  if (!ctx || !ctx->impl.session) return 0;
  return (uint32_t)const_cast<oxb200_ctx*>(ctx)->impl.session->steps().size();
}

int oxb200_plan_step_info(const oxb200_ctx* ctx, uint32_t index, oxb200_step_info* out) {
  if (!ctx || !out || !ctx->impl.session) return OXB200_FAILED;
  auto& steps = const_cast<oxb200_ctx*>(ctx)->impl.session->steps();
  if (index >= steps.size()) return OXB200_FAILED;
  const Step& s = steps[index];
  out->node_name = s.node_name.c_str();
  out->op_type = s.op_type.c_str();
  out->kernel = s.kernel.c_str();
  out->work = s.work;
  out->work_is_bytes = s.work_is_bytes ? 1 : 0;
  out->last_ms = s.last_ms;
  out->launches = s.launches;
  out->bytes = s.bytes;
  return OXB200_OK_HOST;
}

// Shadow verification (oxionnx-cuda src/reference.rs:115-119,198-240): the caller, who owns the
// CPU operators, hands the CPU result of the same node; a mismatch beyond ATOL 1e-4 / RTOL 1e-3
// is "proved wrong".  Under strict mode the status is VERIFY_MISMATCH (the run must fail),
// otherwise FAILED (log and fall back); the message carries the reference's marker either way.
int oxb200_shadow_verify(oxb200_ctx* ctx, const char* op_type, const float* device_lanes, const float* cpu_lanes, uint64_t len) {
  if (!ctx || !device_lanes || !cpu_lanes) return fail_with(ctx, OXB200_FAILED, "shadow_verify: NULL argument");
  const float atol = 1e-4f, rtol = 1e-3f;
  for (uint64_t i = 0; i < len; ++i) {
    float a = device_lanes[i], b = cpu_lanes[i];
    bool ok = (std::isnan(a) && std::isnan(b)) || std::fabs(a - b) <= atol + rtol * std::fabs(b);
    if (!ok) {
      char buf[256];
      snprintf(buf, sizeof buf, "%s%s: element %llu: device %g vs cpu %g", kVerifyPrefix, op_type ? op_type : "?", (unsigned long long)i, (double)a, (double)b);
      return fail_with(ctx, ctx->impl.cfg().strict ? OXB200_VERIFY_MISMATCH : OXB200_FAILED, buf);
    }
  }
  return OXB200_OK_HOST;
}

}  // extern "C"
