// Context, weight residency, arena planning and the run loop of the oxb200 provider.
// The per-operator planning rules live in planner.cpp.
#include "runtime.hpp"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace oxb {

std::vector<std::string> AttrMap::names() const {
  std::vector<std::string> out;
  for (auto& kv : ints) out.push_back(kv.first);
  for (auto& kv : floats) out.push_back(kv.first);
  for (auto& kv : strings) out.push_back(kv.first);
  for (auto& kv : int_lists) out.push_back(kv.first);
  for (auto& kv : float_lists) out.push_back(kv.first);
  return out;
}

// ---------------------------------------------------------------------------------------
// Context
// ---------------------------------------------------------------------------------------
Context::Context(int device, const oxb200_config& cfg) : device_(device), cfg_(cfg) {
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess || count <= 0) {
    (void)cudaGetLastError();
    raise(OXB200_FAILED, "no CUDA device is available (%s); this provider has no CPU path", e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
  }
  if (device < 0 || device >= count) raise(OXB200_FAILED, "device ordinal %d out of range (%d devices)", device, count);
  OXB_CUDA(cudaSetDevice(device));
  cudaDeviceProp prop;
  OXB_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) raise(OXB200_FAILED, "device %d is sm_%d%d; this library carries sm_100a code only", device, prop.major, prop.minor);
  OXB_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
}

Context::~Context() {
  cudaSetDevice(device_);
  session.reset();
  release_caches();
  if (run_ev0) cudaEventDestroy(run_ev0);
  if (run_ev1) cudaEventDestroy(run_ev1);
  if (stream_) cudaStreamDestroy(stream_);
}

void Context::make_current() { OXB_CUDA(cudaSetDevice(device_)); }

void Context::register_weight(const std::string& name, const float* lanes, uint64_t len, const uint64_t* shape, uint32_t rank, DT declared) {
  HostTensor t;
  t.declared = declared;
  t.shape.assign(shape, shape + rank);
  if ((uint64_t)prod(t.shape) != len) raise(OXB200_FAILED, "weight '%s': %llu lanes do not match its shape", name.c_str(), (unsigned long long)len);
  t.data.assign(lanes, lanes + len);
  weights_[name] = std::move(t);
  // a re-registered weight invalidates its packed forms
  for (auto it = forms_.begin(); it != forms_.end();) {
    if (it->first.first == name) {
      cudaFree(it->second.ptr);
      counters.weight_bytes_resident -= it->second.bytes;
      it = forms_.erase(it);
    } else {
      ++it;
    }
  }
  resident_names_.erase(name);
}

const HostTensor* Context::weight(const std::string& name) const {
  auto it = weights_.find(name);
  return it == weights_.end() ? nullptr : &it->second;
}

bool Context::weight_resident(const std::string& name) const { return resident_names_.count(name) != 0; }

void* Context::alloc_device(size_t bytes) {
  void* p = nullptr;
  if (bytes == 0) bytes = 256;
  OXB_CUDA(cudaMalloc(&p, align_up(bytes, 256)));
  return p;
}

void Context::free_device(void* p) {
  if (p) cudaFree(p);
}

void* Context::resident_form(const std::string& name, const std::string& form, size_t bytes, const std::function<void(void*)>& fill_host,
                             bool cacheable) {
  auto key = std::make_pair(name, form);
  if (cacheable) {
    auto it = forms_.find(key);
    if (it != forms_.end() && it->second.bytes == bytes) return it->second.ptr;
  }
  std::vector<uint8_t> host(std::max<size_t>(bytes, 16), 0);
  fill_host(host.data());
  void* dev = alloc_device(bytes);
  OXB_CUDA(cudaMemcpyAsync(dev, host.data(), bytes, cudaMemcpyHostToDevice, stream_));
  OXB_CUDA(cudaStreamSynchronize(stream_));
  if (cacheable) {
    counters.weight_uploads += 1;
    forms_[key] = DeviceBuffer{dev, bytes};
    counters.weight_bytes_resident += bytes;
    resident_names_.insert(name);
  } else {
    // an operand of a one-node dispatch: activation traffic, not a resident weight
    counters.uploads += 1;
    counters.upload_bytes += bytes;
    temp_forms_.push_back(dev);
  }
  return dev;
}

void Context::free_temp_forms() {
  for (void* p : temp_forms_) cudaFree(p);
  temp_forms_.clear();
}

uint64_t Context::cached_bytes() const {
  uint64_t total = 0;
  for (const auto& kv : forms_) total += kv.second.bytes;
  return total;
}

void Context::release_caches() {
  for (auto& kv : forms_) cudaFree(kv.second.ptr);
  forms_.clear();
  for (void* p : temp_forms_) cudaFree(p);
  temp_forms_.clear();
  resident_names_.clear();
  counters.weight_bytes_resident = 0;
}

// ---------------------------------------------------------------------------------------
// Session: arena layout, upload, run, download
// ---------------------------------------------------------------------------------------
Session::~Session() {
  cudaSetDevice(ctx_->device());
  cudaStreamSynchronize(ctx_->stream());
  for (auto* p : umma_plans_) k::umma_plan_destroy(p);
  for (auto* c : umma_chains_) k::umma_chain_destroy(c);
  for (auto* a : umma_attentions_) k::umma_attention_destroy(a);
  for (auto& s : steps_) {
    if (s.ev0) cudaEventDestroy(s.ev0);
    if (s.ev1) cudaEventDestroy(s.ev1);
  }
  if (arena_.ptr) cudaFree(arena_.ptr);
  for (auto& b : owned_) cudaFree(b.ptr);
  if (err_flag_) cudaFree(err_flag_);
  for (int f = 0; f < 2; ++f) {
    Flight& fl = flight_[f];
    if (fl.up) cudaEventDestroy(fl.up);
    if (fl.done) cudaEventDestroy(fl.done);
    if (fl.down) cudaEventDestroy(fl.down);
    if (f == 1 && pipe_double_)
      for (void* p : fl.in_dev) cudaFree(p);
    for (float* p : fl.out_host) cudaFreeHost(p);
    for (void* p : fl.out_dev) cudaFree(p);
    if (fl.err_host) cudaFreeHost(fl.err_host);
  }
  if (copy_stream_) cudaStreamDestroy(copy_stream_);
  if (down_stream_) cudaStreamDestroy(down_stream_);
  for (auto& g : graphs_)
    if (g.exec) cudaGraphExecDestroy(g.exec);
}

Value* Session::find_value(const std::string& name) {
  auto it = index_.find(name);
  return it == index_.end() ? nullptr : &values_[it->second];
}

void Session::sync() {
  OXB_CUDA(cudaStreamSynchronize(ctx_->stream()));
  ctx_->counters.fences += 1;
}

int Session::check_error_flag() {
  int flag = 0;
  OXB_CUDA(cudaMemcpy(&flag, err_flag_, sizeof(int), cudaMemcpyDeviceToHost));
  if (flag != 0) {
    int zero = 0;
    OXB_CUDA(cudaMemcpy(err_flag_, &zero, sizeof(int), cudaMemcpyHostToDevice));
    for (auto* p : umma_plans_) k::umma_plan_reset_after_error(p);
    for (auto* c : umma_chains_) k::umma_chain_reset_after_error(c);
  }
  return flag;
}

// The host lanes of a feed for graph input `v`, checked against the plan: f32 lanes for an input declared f32, typed
// lanes of the declared type otherwise.
static const void* feed_lanes(const oxb200_operand& f, const Value& v, const char* name) {
  if ((int64_t)f.len != v.numel()) raise(OXB200_FAILED, "run: feed '%s' has %llu lanes, the plan expects %lld", name, (unsigned long long)f.len, (long long)v.numel());
  if (f.rank != v.shape.size()) raise(OXB200_FAILED, "run: feed '%s' rank differs from the planned shape", name);
  for (uint32_t d = 0; d < f.rank; ++d)
    if ((int64_t)f.shape[d] != v.shape[d]) raise(OXB200_FAILED, "run: feed '%s' shape differs from the planned shape", name);
  if (v.dt == DT::F32) {
    if (f.lanes) return f.lanes;
    if (f.typed && f.dtype == OXB200_DT_F32) return f.typed;
    raise(OXB200_FAILED, "run: feed '%s' has no f32 host lanes", name);
  }
  if (!f.typed || f.dtype != (int32_t)v.dt)
    raise(OXB200_FAILED, "run: graph input '%s' was declared %s; its feed must carry typed lanes of that type", name, dt_name(v.dt));
  return f.typed;
}

void Session::upload(const oxb200_operand* feeds, uint32_t n) {
  for (auto& in : input_staging_) {
    const oxb200_operand* f = nullptr;
    for (uint32_t i = 0; i < n; ++i)
      if (feeds[i].name && in.first == feeds[i].name) f = &feeds[i];
    if (!f) raise(OXB200_FAILED, "run: no feed for graph input '%s'", in.first.c_str());
    Value& v = values_[in.second];
    if (external_bind_.count(in.first)) continue;  // bound to a value that already lives on the device
    const void* src = feed_lanes(*f, v, in.first.c_str());
    OXB_CUDA(cudaMemcpyAsync(v.ptr, src, (size_t)v.numel() * dt_size(v.dt), cudaMemcpyHostToDevice, ctx_->stream()));
    ctx_->counters.uploads += 1;
    ctx_->counters.upload_bytes += (uint64_t)v.numel() * dt_size(v.dt);
  }
}

bool Session::capture_graph(GraphSlot& g) {
  cudaStream_t s = ctx_->stream();
  const oxb200_counters before = ctx_->counters;
  if (cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  bool ok = true;
  try {
    for (auto& st : steps_) st.launch(s);
  } catch (...) {
    ok = false;
  }
  cudaGraph_t graph = nullptr;
  if (cudaStreamEndCapture(s, &graph) != cudaSuccess || !graph) ok = false;
  if (ok && cudaGraphInstantiate(&g.exec, graph, 0) != cudaSuccess) ok = false;
  if (graph) cudaGraphDestroy(graph);
  (void)cudaGetLastError();
  // a recording executes nothing: the counters go back, and each replay adds what it stands for
  g.d_kernel = ctx_->counters.kernel_launches - before.kernel_launches;
  g.d_umma = ctx_->counters.umma_launches - before.umma_launches;
  g.d_simt = ctx_->counters.simt_launches - before.simt_launches;
  g.d_glue = ctx_->counters.glue_launches - before.glue_launches;
  ctx_->counters = before;
  if (!ok) {
    if (g.exec) cudaGraphExecDestroy(g.exec);
    g.exec = nullptr;
  }
  return ok;
}

bool Session::replay_graph() {
  std::vector<void*> key;
  for (auto& in : input_staging_) key.push_back(values_[in.second].ptr);
  GraphSlot* g = nullptr;
  for (auto& c : graphs_)
    if (c.key == key) g = &c;
  if (!g) {
    if (graphs_.size() >= 4) return false;  // more input buffers than the pipeline ever rotates through
    graphs_.push_back(GraphSlot{});
    g = &graphs_.back();
    g->key = key;
  }
  if (g->poisoned) return false;
  if (!g->exec) {
    // the first run on these addresses goes the ordinary way: it sets the kernels' one-time attributes
    if (!g->warmed) {
      g->warmed = true;
      return false;
    }
    if (!capture_graph(*g)) {
      g->poisoned = true;
      ctx_->counters.graph_poisoned += 1;
      return false;
    }
    ctx_->counters.graph_captures += 1;
  }
  OXB_CUDA(cudaGraphLaunch(g->exec, ctx_->stream()));
  ctx_->counters.graph_replays += 1;
  ctx_->counters.kernel_launches += g->d_kernel;
  ctx_->counters.umma_launches += g->d_umma;
  ctx_->counters.simt_launches += g->d_simt;
  ctx_->counters.glue_launches += g->d_glue;
  for (auto& st : steps_) st.launches += 1;
  return true;
}

void Session::run_steps(bool profile) {
  cudaStream_t s = ctx_->stream();
  if (graph_allowed_ && !profile && ctx_->cfg().cuda_graph && !ctx_->cfg().verify && replay_graph()) return;
  for (auto& st : steps_) {
    if (profile) {
      if (!st.ev0) {
        OXB_CUDA(cudaEventCreate(&st.ev0));
        OXB_CUDA(cudaEventCreate(&st.ev1));
      }
      OXB_CUDA(cudaEventRecord(st.ev0, s));
    }
    st.launch(s);
    st.launches += 1;
    if (profile) OXB_CUDA(cudaEventRecord(st.ev1, s));
  }
  OXB_CUDA(cudaGetLastError());
}

static void write_result_shape(const Value& v, oxb200_result* r) {
  r->rank = (uint32_t)v.shape.size();
  for (size_t d = 0; d < v.shape.size() && d < OXB200_MAX_RANK; ++d) r->shape[d] = (uint64_t)v.shape[d];
  r->len = (uint64_t)v.numel();
}

void Session::download(oxb200_result* fetches, uint32_t n) {
  download_async(fetches, n);
  finish_download();
}

void Session::finish_download() {
  sync();
  int flag = check_error_flag();
  if (flag)
    raise(OXB200_FAILED, flag == 20 ? "Gather: an index is out of range (device code %d); results are not valid" : "a tensor-core kernel gave up on a bounded wait (code %d); results are not valid", flag);
}

void Session::download_async(oxb200_result* fetches, uint32_t n) {
  if (n != outputs_.size()) raise(OXB200_FAILED, "run: %u fetch slots for %zu graph outputs", n, outputs_.size());
  // validate everything first, then copy: a rejected write leaves the caller's buffers untouched
  // (write_node_outputs, root crate src/session/run/dispatch.rs:335-455)
  for (uint32_t i = 0; i < n; ++i) {
    const Value& v = values_[output_staging_[i].second];
    if (fetches[i].lanes && fetches[i].cap < (uint64_t)v.numel())
      raise(OXB200_FAILED, "run: fetch buffer for '%s' holds %llu lanes, %lld needed", outputs_[i].c_str(), (unsigned long long)fetches[i].cap, (long long)v.numel());
  }
  for (uint32_t i = 0; i < n; ++i) {
    const Value& v = values_[output_staging_[i].second];
    write_result_shape(v, &fetches[i]);
    if (fetches[i].lanes && v.numel() > 0) {
      OXB_CUDA(cudaMemcpyAsync(fetches[i].lanes, v.ptr, (size_t)v.numel() * 4, cudaMemcpyDeviceToHost, ctx_->stream()));
      ctx_->counters.downloads += 1;
      ctx_->counters.download_bytes += (uint64_t)v.numel() * 4;
    }
  }
}

void Session::fetch_value(const std::string& name, oxb200_result* out) {
  Value* v = find_value(name);
  if (!v) raise(OXB200_FAILED, "fetch_value: '%s' is not a value of the planned graph", name.c_str());
  if (!v->ptr) raise(OXB200_FAILED, "fetch_value: '%s' has no device storage (fused away)", name.c_str());
  write_result_shape(*v, out);
  if (!out->lanes) return;
  if (out->cap < (uint64_t)v->numel()) raise(OXB200_FAILED, "fetch_value: buffer too small for '%s'", name.c_str());
  int64_t n = v->numel();
  if (n == 0) return;
  // convert to f32 lanes in the logical order through a temporary
  void* tmp = ctx_->alloc_device((size_t)n * 4);
  k::Dims4 d{1, 1, 1, 1};
  if (v->shape.size() == 4) d = k::Dims4{v->shape[0], v->shape[1], v->shape[2], v->shape[3]};
  else d = k::Dims4{n, 1, 1, 1};
  k::TensorRef src{v->ptr, v->dt, v->shape.size() == 4 ? v->layout : Layout::PLAIN, d};
  k::TensorRef dst{tmp, DT::F32, Layout::PLAIN, d};
  k::convert(src, dst, ctx_->stream());
  OXB_CUDA(cudaMemcpyAsync(out->lanes, tmp, (size_t)n * 4, cudaMemcpyDeviceToHost, ctx_->stream()));
  sync();
  ctx_->free_device(tmp);
  ctx_->counters.downloads += 1;
  ctx_->counters.download_bytes += (uint64_t)n * 4;
}

// ---- pipelined runs ---------------------------------------------------------------------------
void Session::rebind_input(int value_index, void* ptr) {
  values_[value_index].ptr = ptr;
  for (Value& v : values_) {  // values that share the input's storage (Reshape, Flatten, Identity)
    int root = v.alias_of;
    while (root >= 0 && values_[root].alias_of >= 0) root = values_[root].alias_of;
    if (root == value_index) v.ptr = ptr;
  }
}

void Session::prepare_pipeline() {
  if (pipe_ready_) return;
  // uploads and downloads have a stream each: a download waits for its run, and an upload queued behind it
  // in the same stream would wait for that run too instead of overlapping it
  OXB_CUDA(cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking));
  OXB_CUDA(cudaStreamCreateWithFlags(&down_stream_, cudaStreamNonBlocking));
  // A second input buffer is only safe when no step has the input's address built into a tensor map:
  // the tensor-core steps are the ones that do, so none of them may read an input (or an alias of one).
  pipe_double_ = external_bind_.empty();
  for (const Step& st : steps_) {
    if (st.family != 0) continue;
    for (int r : st.reads) {
      int root = r;
      while (values_[root].alias_of >= 0) root = values_[root].alias_of;
      for (auto& in : input_staging_)
        if (in.second == root) pipe_double_ = false;
    }
  }
  for (int f = 0; f < 2; ++f) {
    Flight& fl = flight_[f];
    OXB_CUDA(cudaEventCreateWithFlags(&fl.up, cudaEventDisableTiming));
    OXB_CUDA(cudaEventCreateWithFlags(&fl.done, cudaEventDisableTiming));
    OXB_CUDA(cudaEventCreateWithFlags(&fl.down, cudaEventDisableTiming));
    for (auto& in : input_staging_) {
      void* p = values_[in.second].ptr;
      if (f == 1 && pipe_double_) OXB_CUDA(cudaMalloc(&p, std::max<size_t>((size_t)values_[in.second].numel() * dt_size(values_[in.second].dt), 256)));
      fl.in_dev.push_back(p);
    }
    for (auto& out : output_staging_) {
      float* p = nullptr;
      OXB_CUDA(cudaMallocHost(&p, std::max<size_t>((size_t)values_[out.second].numel() * 4, 4)));
      fl.out_host.push_back(p);
      void* d = nullptr;
      OXB_CUDA(cudaMalloc(&d, std::max<size_t>((size_t)values_[out.second].numel() * 4, 256)));
      fl.out_dev.push_back(d);
    }
    OXB_CUDA(cudaMallocHost(&fl.err_host, sizeof(int)));
  }
  pipe_ready_ = true;
}

void Session::submit(const oxb200_operand* feeds, uint32_t n, bool profile) {
  prepare_pipeline();
  Flight& fl = flight_[submit_idx_];
  Flight& prev = flight_[submit_idx_ ^ 1];
  if (fl.busy) raise(OXB200_FAILED, "submit: two runs are already in flight; collect one first");
  cudaStream_t main = ctx_->stream();
  // without a second input buffer the upload must wait until the previous run has read the inputs
  // validate every feed before the first input is re-pointed: a rejected submission leaves the plan as it was
  std::vector<const void*> srcs(input_staging_.size(), nullptr);
  for (size_t i = 0; i < input_staging_.size(); ++i) {
    const auto& in = input_staging_[i];
    const oxb200_operand* f = nullptr;
    for (uint32_t k2 = 0; k2 < n; ++k2)
      if (feeds[k2].name && in.first == feeds[k2].name) f = &feeds[k2];
    if (!f) raise(OXB200_FAILED, "submit: no feed for graph input '%s'", in.first.c_str());
    srcs[i] = feed_lanes(*f, values_[in.second], in.first.c_str());
  }
  if (!pipe_double_ && prev.busy) OXB_CUDA(cudaStreamWaitEvent(copy_stream_, prev.done, 0));
  for (size_t i = 0; i < input_staging_.size(); ++i) {
    const auto& in = input_staging_[i];
    Value& v = values_[in.second];
    OXB_CUDA(cudaMemcpyAsync(fl.in_dev[i], srcs[i], (size_t)v.numel() * dt_size(v.dt), cudaMemcpyHostToDevice, copy_stream_));
    ctx_->counters.uploads += 1;
    ctx_->counters.upload_bytes += (uint64_t)v.numel() * dt_size(v.dt);
    rebind_input(in.second, fl.in_dev[i]);
  }
  OXB_CUDA(cudaEventRecord(fl.up, copy_stream_));
  OXB_CUDA(cudaStreamWaitEvent(main, fl.up, 0));
  run_steps(profile);
  // the outputs move to this slot's own device buffers (a device-to-device copy, microseconds), so that the next
  // run may overwrite the arena while the download is still crossing PCIe
  for (size_t i = 0; i < output_staging_.size(); ++i) {
    const Value& v = values_[output_staging_[i].second];
    if (v.numel() > 0) OXB_CUDA(cudaMemcpyAsync(fl.out_dev[i], v.ptr, (size_t)v.numel() * 4, cudaMemcpyDeviceToDevice, main));
  }
  OXB_CUDA(cudaEventRecord(fl.done, main));
  OXB_CUDA(cudaStreamWaitEvent(down_stream_, fl.done, 0));
  for (size_t i = 0; i < output_staging_.size(); ++i) {
    const Value& v = values_[output_staging_[i].second];
    if (v.numel() > 0) OXB_CUDA(cudaMemcpyAsync(fl.out_host[i], fl.out_dev[i], (size_t)v.numel() * 4, cudaMemcpyDeviceToHost, down_stream_));
    ctx_->counters.downloads += 1;
    ctx_->counters.download_bytes += (uint64_t)v.numel() * 4;
  }
  OXB_CUDA(cudaMemcpyAsync(fl.err_host, err_flag_, sizeof(int), cudaMemcpyDeviceToHost, down_stream_));
  OXB_CUDA(cudaEventRecord(fl.down, down_stream_));
  fl.busy = true;
  submit_idx_ ^= 1;
}

void Session::collect(oxb200_result* fetches, uint32_t n) {
  Flight& fl = flight_[collect_idx_];
  if (!fl.busy) raise(OXB200_FAILED, "collect: no run is in flight");
  if (n != outputs_.size()) raise(OXB200_FAILED, "collect: %u fetch slots for %zu graph outputs", n, outputs_.size());
  for (uint32_t i = 0; i < n; ++i) {
    const Value& v = values_[output_staging_[i].second];
    if (fetches[i].lanes && fetches[i].cap < (uint64_t)v.numel())
      raise(OXB200_FAILED, "collect: fetch buffer for '%s' holds %llu lanes, %lld needed", outputs_[i].c_str(), (unsigned long long)fetches[i].cap, (long long)v.numel());
  }
  OXB_CUDA(cudaEventSynchronize(fl.down));
  ctx_->counters.fences += 1;
  fl.busy = false;
  collect_idx_ ^= 1;
  if (*fl.err_host != 0 || fl.poisoned) {
    // The error word is shared by the runs in flight: let the other run finish before the word is cleared (its
    // kernels may still write it, and its own snapshot may already hold this run's code), and fail it as well.
    const int flag = *fl.err_host, zero = 0;
    fl.poisoned = false;
    Flight& other = flight_[collect_idx_];
    OXB_CUDA(cudaStreamSynchronize(ctx_->stream()));
    OXB_CUDA(cudaStreamSynchronize(down_stream_));
    if (other.busy) other.poisoned = true;
    OXB_CUDA(cudaMemcpy(err_flag_, &zero, sizeof(int), cudaMemcpyHostToDevice));
    for (auto* p : umma_plans_) k::umma_plan_reset_after_error(p);
    for (auto* c : umma_chains_) k::umma_chain_reset_after_error(c);
    raise(OXB200_FAILED, "a kernel reported code %d during a pipelined run (or the run before it failed while this one was in flight); results are not valid", flag);
  }
  for (uint32_t i = 0; i < n; ++i) {
    const Value& v = values_[output_staging_[i].second];
    write_result_shape(v, &fetches[i]);
    if (fetches[i].lanes && v.numel() > 0) std::memcpy(fetches[i].lanes, fl.out_host[i], (size_t)v.numel() * 4);
  }
}

void Session::bind_external(const std::string& name, void* ptr, DT dt, Layout layout) { external_bind_[name] = {ptr, {dt, layout}}; }

// ---- device I/O binding -------------------------------------------------------------------------
bool Session::input_in_tensor_map(int value_index) const {
  // the tensor-core steps build their operands' addresses into tensor maps at plan time
  for (const Step& st : steps_) {
    if (st.family != 0) continue;
    for (int r : st.reads) {
      int root = r;
      while (values_[root].alias_of >= 0) root = values_[root].alias_of;
      if (root == value_index) return true;
    }
  }
  return false;
}

void Session::bind_input_device(const std::string& name, const void* ptr, DT dt, uint64_t len) {
  if (in_flight() > 0) raise(OXB200_FAILED, "bind_input_device: pipelined runs are in flight; collect them first");
  for (size_t i = 0; i < input_staging_.size(); ++i) {
    if (input_staging_[i].first != name) continue;
    const Value& v = values_[input_staging_[i].second];
    if (external_bind_.count(name)) raise(OXB200_FAILED, "bind_input_device: '%s' is a resident dispatch operand", name.c_str());
    if (dt != v.dt) raise(OXB200_FAILED, "bind_input_device: '%s' was planned as %s, the buffer is %s", name.c_str(), dt_name(v.dt), dt_name(dt));
    if ((int64_t)len != v.numel()) raise(OXB200_FAILED, "bind_input_device: '%s' has %lld elements, the buffer %llu", name.c_str(), (long long)v.numel(), (unsigned long long)len);
    if (!ptr || ((uintptr_t)ptr & 15) != 0) raise(OXB200_FAILED, "bind_input_device: the buffer of '%s' must be a 16-byte aligned device address", name.c_str());
    if (own_in_ptr_.empty())
      for (auto& in : input_staging_) own_in_ptr_.push_back(values_[in.second].ptr);
    bound_in_[(int)i] = ptr;
    return;
  }
  raise(OXB200_FAILED, "bind_input_device: '%s' is not an input of the planned graph", name.c_str());
}

void Session::bind_output_device(const std::string& name, void* ptr, uint64_t cap) {
  for (size_t i = 0; i < output_staging_.size(); ++i) {
    if (output_staging_[i].first != name) continue;
    const Value& v = values_[output_staging_[i].second];
    if (cap < (uint64_t)v.numel()) raise(OXB200_FAILED, "bind_output_device: '%s' has %lld lanes, the buffer holds %llu", name.c_str(), (long long)v.numel(), (unsigned long long)cap);
    if (!ptr || ((uintptr_t)ptr & 3) != 0) raise(OXB200_FAILED, "bind_output_device: the buffer of '%s' must be a 4-byte aligned device address", name.c_str());
    bound_out_[(int)i] = {ptr, cap};
    return;
  }
  raise(OXB200_FAILED, "bind_output_device: '%s' is not an output of the planned graph", name.c_str());
}

void Session::output_device_ptr(const std::string& name, void** ptr, uint64_t* len) {
  for (size_t i = 0; i < output_staging_.size(); ++i) {
    if (output_staging_[i].first != name) continue;
    const Value& v = values_[output_staging_[i].second];
    if (ptr) *ptr = v.ptr;
    if (len) *len = (uint64_t)v.numel();
    return;
  }
  raise(OXB200_FAILED, "output_device_ptr: '%s' is not an output of the planned graph", name.c_str());
}

void Session::clear_bindings() {
  if (!own_in_ptr_.empty())
    for (size_t i = 0; i < input_staging_.size(); ++i) rebind_input(input_staging_[i].second, own_in_ptr_[i]);
  bound_in_.clear();
  bound_out_.clear();
}

// A bound input is read in place when no tensor map holds its buffer's address; otherwise its lanes are copied
// device-to-device into the buffer the maps were built for (no host traffic either way).
void Session::apply_input_bindings() {
  for (auto& kv : bound_in_) {
    const int vi = input_staging_[kv.first].second;
    Value& v = values_[vi];
    if (input_in_tensor_map(vi)) {
      if (v.ptr != own_in_ptr_[kv.first]) rebind_input(vi, own_in_ptr_[kv.first]);
      OXB_CUDA(cudaMemcpyAsync(v.ptr, kv.second, (size_t)v.numel() * dt_size(v.dt), cudaMemcpyDeviceToDevice, ctx_->stream()));
    } else {
      rebind_input(vi, const_cast<void*>(kv.second));
    }
  }
}

void Session::run_bound(const oxb200_operand* feeds, uint32_t n, oxb200_result* fetches, uint32_t nf, bool profile) {
  if (in_flight() > 0) raise(OXB200_FAILED, "run_bound: pipelined runs are in flight; collect them first");
  if (fetches && nf != outputs_.size()) raise(OXB200_FAILED, "run_bound: %u fetch slots for %zu graph outputs", nf, outputs_.size());
  // unbound inputs come from the host as in run()
  for (size_t i = 0; i < input_staging_.size(); ++i) {
    if (bound_in_.count((int)i)) continue;
    const auto& in = input_staging_[i];
    if (external_bind_.count(in.first)) continue;
    const oxb200_operand* f = nullptr;
    for (uint32_t k2 = 0; k2 < n; ++k2)
      if (feeds && feeds[k2].name && in.first == feeds[k2].name) f = &feeds[k2];
    if (!f) raise(OXB200_FAILED, "run_bound: graph input '%s' is neither bound nor fed", in.first.c_str());
    Value& v = values_[in.second];
    const void* src = feed_lanes(*f, v, in.first.c_str());
    OXB_CUDA(cudaMemcpyAsync(v.ptr, src, (size_t)v.numel() * dt_size(v.dt), cudaMemcpyHostToDevice, ctx_->stream()));
    ctx_->counters.uploads += 1;
    ctx_->counters.upload_bytes += (uint64_t)v.numel() * dt_size(v.dt);
  }
  apply_input_bindings();
  run_steps(profile);
  for (auto& kv : bound_out_) {
    const Value& v = values_[output_staging_[kv.first].second];
    if (v.numel() > 0 && kv.second.first != v.ptr)
      OXB_CUDA(cudaMemcpyAsync(kv.second.first, v.ptr, (size_t)v.numel() * 4, cudaMemcpyDeviceToDevice, ctx_->stream()));
  }
  if (fetches) {
    for (uint32_t i = 0; i < nf; ++i) {
      const Value& v = values_[output_staging_[i].second];
      if (fetches[i].lanes && fetches[i].cap < (uint64_t)v.numel())
        raise(OXB200_FAILED, "run_bound: fetch buffer for '%s' holds %llu lanes, %lld needed", outputs_[i].c_str(), (unsigned long long)fetches[i].cap, (long long)v.numel());
    }
    for (uint32_t i = 0; i < nf; ++i) {
      const Value& v = values_[output_staging_[i].second];
      write_result_shape(v, &fetches[i]);
      if (fetches[i].lanes && v.numel() > 0) {
        OXB_CUDA(cudaMemcpyAsync(fetches[i].lanes, v.ptr, (size_t)v.numel() * 4, cudaMemcpyDeviceToHost, ctx_->stream()));
        ctx_->counters.downloads += 1;
        ctx_->counters.download_bytes += (uint64_t)v.numel() * 4;
      }
    }
  }
  finish_download();
}

}  // namespace oxb
