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

void Context::register_weight(const std::string& name, const float* lanes, uint64_t len, const uint64_t* shape, uint32_t rank) {
  HostTensor t;
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
  }
  return flag;
}

void Session::upload(const oxb200_operand* feeds, uint32_t n) {
  for (auto& in : input_staging_) {
    const oxb200_operand* f = nullptr;
    for (uint32_t i = 0; i < n; ++i)
      if (feeds[i].name && in.first == feeds[i].name) f = &feeds[i];
    if (!f) raise(OXB200_FAILED, "run: no feed for graph input '%s'", in.first.c_str());
    Value& v = values_[in.second];
    if (external_bind_.count(in.first)) continue;  // bound to a value that already lives on the device
    if (!f->lanes) raise(OXB200_FAILED, "run: feed '%s' has no host lanes", in.first.c_str());
    if ((int64_t)f->len != v.numel()) raise(OXB200_FAILED, "run: feed '%s' has %llu lanes, the plan expects %lld", in.first.c_str(), (unsigned long long)f->len, (long long)v.numel());
    if (f->rank != v.shape.size()) raise(OXB200_FAILED, "run: feed '%s' rank differs from the planned shape", in.first.c_str());
    for (uint32_t d = 0; d < f->rank; ++d)
      if ((int64_t)f->shape[d] != v.shape[d]) raise(OXB200_FAILED, "run: feed '%s' shape differs from the planned shape", in.first.c_str());
    OXB_CUDA(cudaMemcpyAsync(v.ptr, f->lanes, (size_t)v.numel() * 4, cudaMemcpyHostToDevice, ctx_->stream()));
    ctx_->counters.uploads += 1;
    ctx_->counters.upload_bytes += (uint64_t)v.numel() * 4;
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
  if (flag) raise(OXB200_FAILED, "a tensor-core kernel gave up on a bounded wait (code %d); results are not valid", flag);
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
      if (f == 1 && pipe_double_) OXB_CUDA(cudaMalloc(&p, std::max<size_t>((size_t)values_[in.second].numel() * 4, 256)));
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
  if (!pipe_double_ && prev.busy) OXB_CUDA(cudaStreamWaitEvent(copy_stream_, prev.done, 0));
  for (size_t i = 0; i < input_staging_.size(); ++i) {
    const auto& in = input_staging_[i];
    const oxb200_operand* f = nullptr;
    for (uint32_t k2 = 0; k2 < n; ++k2)
      if (feeds[k2].name && in.first == feeds[k2].name) f = &feeds[k2];
    Value& v = values_[in.second];
    if (!f || !f->lanes) raise(OXB200_FAILED, "submit: no host lanes for graph input '%s'", in.first.c_str());
    if ((int64_t)f->len != v.numel()) raise(OXB200_FAILED, "submit: feed '%s' has %llu lanes, the plan expects %lld", in.first.c_str(), (unsigned long long)f->len, (long long)v.numel());
    OXB_CUDA(cudaMemcpyAsync(fl.in_dev[i], f->lanes, (size_t)v.numel() * 4, cudaMemcpyHostToDevice, copy_stream_));
    ctx_->counters.uploads += 1;
    ctx_->counters.upload_bytes += (uint64_t)v.numel() * 4;
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
  if (*fl.err_host != 0) {
    const int flag = *fl.err_host, zero = 0;
    OXB_CUDA(cudaMemcpy(err_flag_, &zero, sizeof(int), cudaMemcpyHostToDevice));
    OXB_CUDA(cudaStreamSynchronize(ctx_->stream()));
    for (auto* p : umma_plans_) k::umma_plan_reset_after_error(p);
    raise(OXB200_FAILED, "a kernel reported code %d during a pipelined run; results are not valid", flag);
  }
  for (uint32_t i = 0; i < n; ++i) {
    const Value& v = values_[output_staging_[i].second];
    write_result_shape(v, &fetches[i]);
    if (fetches[i].lanes && v.numel() > 0) std::memcpy(fetches[i].lanes, fl.out_host[i], (size_t)v.numel() * 4);
  }
}

void Session::bind_external(const std::string& name, void* ptr, DT dt, Layout layout) { external_bind_[name] = {ptr, {dt, layout}}; }

}  // namespace oxb
