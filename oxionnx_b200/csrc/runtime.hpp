// Host runtime of the oxb200 execution provider: context, weight residency, the planner that
// turns a node list into device steps over a lifetime-planned arena, and the run loop.
#pragma once

#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "common.hpp"
#include "kernels.hpp"

namespace oxb {

struct HostTensor {
  std::vector<float> data;
  std::vector<int64_t> shape;
  // Element type the tensor was declared with where it came from (an ONNX initializer, a typed operand); F32 is
  // the reference's dtype-erased default.  The quantised operators' y_zero_point reads it to resolve the
  // saturation range exactly (SatRange::for_dtype, quant_ops/mod.rs:216-222); a float contraction whose weight
  // is declared FLOAT16 / BFLOAT16 runs with 16-bit operands.
  DT declared = DT::F32;
  int64_t numel() const { return prod(shape); }
};

// Attributes (oxionnx-core src/graph.rs:696-733), the five kinds the hot path uses.
struct AttrMap {
  std::map<std::string, int64_t> ints;
  std::map<std::string, float> floats;
  std::map<std::string, std::string> strings;
  std::map<std::string, std::vector<int64_t>> int_lists;
  std::map<std::string, std::vector<float>> float_lists;
  int64_t i(const std::string& k, int64_t d) const {
    auto it = ints.find(k);
    return it == ints.end() ? d : it->second;
  }
  float f(const std::string& k, float d) const {
    auto it = floats.find(k);
    return it == floats.end() ? d : it->second;
  }
  std::string s(const std::string& k) const {
    auto it = strings.find(k);
    return it == strings.end() ? std::string() : it->second;
  }
  std::vector<int64_t> int_list(const std::string& k) const {
    auto it = int_lists.find(k);
    return it == int_lists.end() ? std::vector<int64_t>() : it->second;
  }
  bool has(const std::string& k) const {
    return ints.count(k) || floats.count(k) || strings.count(k) || int_lists.count(k) || float_lists.count(k);
  }
  std::vector<std::string> names() const;
};

struct NodeDef {
  std::string op, name;
  std::vector<std::string> inputs, outputs;
  AttrMap attrs;
};

// A value of the planned graph.
struct Value {
  std::string name;
  std::vector<int64_t> shape;  // logical (ONNX) shape
  DT dt = DT::F32;
  Layout layout = Layout::PLAIN;
  const HostTensor* host = nullptr;  // contents known at plan time (initializer or dispatch operand)
  bool is_graph_input = false, is_graph_output = false;
  bool external = false;  // storage owned elsewhere (resident dispatch operand, staging buffer)
  int producer = -1;      // step index that writes it (-1: input / constant)
  int last_use = -1;      // last step index that reads it
  int alias_of = -1;      // shares the storage of another value
  size_t bytes = 0;
  int slot = -1;
  void* ptr = nullptr;
  // produced by a per-tensor QuantizeLinear of the f32 value q_src in step q_step (planner use:
  // a consumer that repacks the tensor anyway may quantise on the way and drop that step)
  int q_src = -1, q_step = -1;
  float q_scale = 1.f, q_zp = 0.f, q_lo = 0.f, q_hi = 255.f;
  // set on the output of a per-tensor DequantizeLinear of an 8-bit rank-4 value: a consumer that can read the
  // 8-bit lanes itself may drop that step (dq_step) and read dq_src
  // when set: the step that writes this value also merges the value's minimum and maximum into these two ordered
  // keys (the scratch of the DynamicQuantizeLinear that reads it, which then skips its own first pass)
  void* minmax_keys = nullptr;
  int dq_src = -1, dq_step = -1;
  float dq_scale = 1.f, dq_zp = 0.f;
  int64_t numel() const { return prod(shape); }
};

struct Step {
  std::string node_name, op_type, kernel;
  int family = 2;  // 0 tcgen05, 1 direct CUDA-core, 2 glue
  double work = 0;
  bool work_is_bytes = true;
  // algorithmic bytes of one launch: every value the step reads and writes once, plus `param_bytes` (a
  // contraction's packed weights); filled when the plan is finalised
  double param_bytes = 0, bytes = 0;
  std::vector<int> reads, writes;  // value indices
  std::function<void(cudaStream_t)> launch;
  std::function<void()> finalize;  // runs once after the arena is laid out (builds tensor maps)
  float last_ms = -1.f;
  uint64_t launches = 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
};

struct DeviceBuffer {
  void* ptr = nullptr;
  size_t bytes = 0;
};

class Context;

// One planned graph (a whole session, or the one-node graph of a dispatch).
class Session {
 public:
  explicit Session(Context* ctx) : ctx_(ctx) {}
  ~Session();
  // inputs: name -> shape (host data unknown) ; consts: name -> host tensor (known now)
  void plan(const std::vector<NodeDef>& nodes, const std::vector<std::pair<std::string, std::vector<int64_t>>>& inputs,
            const std::map<std::string, const HostTensor*>& volatile_consts, const std::vector<std::string>& outputs);
  void upload(const oxb200_operand* feeds, uint32_t n);
  void run_steps(bool profile);
  void download(oxb200_result* fetches, uint32_t n);
  void download_async(oxb200_result* fetches, uint32_t n);  // enqueue the copies
  void finish_download();                                    // one fence + the kernels' error word
  void fetch_value(const std::string& name, oxb200_result* out);
  void sync();
  std::vector<Step>& steps() { return steps_; }
  const std::vector<std::string>& output_names() const { return outputs_; }
  size_t arena_bytes() const { return arena_.bytes; }
  size_t arena_slots() const { return n_slots_; }
  // Bind a graph input to storage that already lives on the device (resident dispatch operand).
  void bind_external(const std::string& name, void* ptr, DT dt, Layout layout);
  // Declared element type of a graph input (before plan()): 8-bit inputs are stored and fed as 8-bit lanes.
  void declare_input_type(const std::string& name, DT dt) { input_types_[name] = dt; }
  // Device I/O binding (after plan()): inputs read from, outputs also written to, caller-owned device buffers.
  void bind_input_device(const std::string& name, const void* ptr, DT dt, uint64_t len);
  void bind_output_device(const std::string& name, void* ptr, uint64_t cap);
  void output_device_ptr(const std::string& name, void** ptr, uint64_t* len);
  void clear_bindings();
  // run_with_binding: uploads the unbound inputs, runs, copies bound outputs device-to-device, downloads the
  // fetches that have host lanes; one fence
  void run_bound(const oxb200_operand* feeds, uint32_t n, oxb200_result* fetches, uint32_t nf, bool profile);
  // After a run, detach the storage of an output so it can outlive the session.
  Value* find_value(const std::string& name);
  int check_error_flag();
  // Pipelined runs: submit() enqueues the upload of one set of feeds (on a copy stream, into the input buffer
  // that is not being read), the steps, and the download of the outputs into pinned staging; collect() waits
  // for the oldest submission and hands its outputs over.  At most two submissions are in flight.
  void submit(const oxb200_operand* feeds, uint32_t n, bool profile);
  void collect(oxb200_result* fetches, uint32_t n);
  int in_flight() const { return (flight_[0].busy ? 1 : 0) + (flight_[1].busy ? 1 : 0); }

 private:
  friend class Planner;
  Context* ctx_;
  std::vector<Value> values_;
  std::unordered_map<std::string, int> index_;
  std::vector<Step> steps_;
  std::vector<std::string> outputs_;
  std::vector<std::pair<std::string, int>> input_staging_;  // graph input name -> value index of the raw f32 upload
  std::vector<std::pair<std::string, int>> output_staging_; // graph output name -> value index of the f32 PLAIN copy
  DeviceBuffer arena_;
  std::vector<DeviceBuffer> owned_;  // staging + parameter buffers
  std::vector<k::UmmaPlan*> umma_plans_;
  std::vector<k::UmmaChain*> umma_chains_;
  std::vector<k::UmmaAttentionPlan*> umma_attentions_;
  size_t n_slots_ = 0;
  int* err_flag_ = nullptr;
  std::map<std::string, std::pair<void*, std::pair<DT, Layout>>> external_bind_;
  std::map<std::string, DT> input_types_;
  // device bindings: input index -> caller's buffer (copied into the input's own buffer when a tensor map holds
  // that buffer's address, read in place otherwise); output index -> caller's buffer and capacity
  std::map<int, const void*> bound_in_;
  std::map<int, std::pair<void*, uint64_t>> bound_out_;
  std::vector<void*> own_in_ptr_;  // the session's own buffer of each graph input (what an unbound input reads)
  bool input_in_tensor_map(int value_index) const;
  void apply_input_bindings();
  std::shared_ptr<void> planner_;  // keeps the objects the step closures refer to alive
  struct Flight {
    bool busy = false;
    bool poisoned = false;           // the other run in flight failed while this one was running: its results are not trusted
    cudaEvent_t up = nullptr, done = nullptr, down = nullptr;
    std::vector<void*> in_dev;       // this slot's device buffer per graph input
    std::vector<float*> out_host;    // pinned staging per graph output
    std::vector<void*> out_dev;      // device copy of each output, so that the next run need not wait for the download
    int* err_host = nullptr;         // pinned copy of the kernels' error word
  };
  Flight flight_[2];
  int submit_idx_ = 0, collect_idx_ = 0;
  cudaStream_t copy_stream_ = nullptr, down_stream_ = nullptr;  // uploads; downloads
  bool pipe_ready_ = false, pipe_double_ = false;
  void prepare_pipeline();
  void rebind_input(int value_index, void* ptr);
  // CUDA-graph replay of the step list (graph_cache.rs of the reference's provider: off unless
  // OXIONNX_CUDA_GRAPH is set, never together with shadow verification, a failed capture demotes its key
  // for good).  A recording stores device addresses, so the key is every address that can differ between
  // two runs of one plan: the graph inputs' buffers.  Everything else a step touches (arena, weights,
  // parameter vectors, the error word) is owned by the session or the context and never moves.
  struct GraphSlot {
    std::vector<void*> key;
    cudaGraphExec_t exec = nullptr;
    bool warmed = false, poisoned = false;
    uint64_t d_kernel = 0, d_umma = 0, d_simt = 0, d_glue = 0;  // launches one replay stands for
  };
  std::vector<GraphSlot> graphs_;
  bool graph_allowed_ = false;
  bool replay_graph();
  bool capture_graph(GraphSlot& g);

 public:
  void allow_graph(bool on) { graph_allowed_ = on; }
};

class Context {
 public:
  Context(int device, const oxb200_config& cfg);
  ~Context();
  int device() const { return device_; }
  cudaStream_t stream() const { return stream_; }
  const oxb200_config& cfg() const { return cfg_; }
  void set_profile(int on) { cfg_.profile = on ? 1 : 0; }
  void set_graph_capture(int on) { cfg_.cuda_graph = on ? 1 : 0; }
  // device bytes held for reuse: packed weight forms (resident weights) of this context
  uint64_t cached_bytes() const;
  void make_current();

  void register_weight(const std::string& name, const float* lanes, uint64_t len, const uint64_t* shape, uint32_t rank, DT declared = DT::F32);
  const HostTensor* weight(const std::string& name) const;
  bool weight_resident(const std::string& name) const;

  // Device copy of a packed form of a weight, created on first use and kept for the context's
  // life (ResidentWeights, oxionnx-cuda src/residency.rs; identity = name + form).
  void* resident_form(const std::string& name, const std::string& form, size_t bytes, const std::function<void(void*)>& fill_host,
                      bool cacheable);
  void* alloc_device(size_t bytes);
  void free_device(void* p);
  void release_caches();
  void free_temp_forms();

  oxb200_counters counters{};
  std::string last_error;
  std::unique_ptr<Session> session;  // the planned session of oxb200_session_plan
  cudaEvent_t run_ev0 = nullptr, run_ev1 = nullptr;
  float last_run_ms = -1.f;
  std::mutex mu;

 private:
  int device_;
  oxb200_config cfg_;
  cudaStream_t stream_ = nullptr;
  std::unordered_map<std::string, HostTensor> weights_;
  std::map<std::pair<std::string, std::string>, DeviceBuffer> forms_;
  std::set<std::string> resident_names_;
  std::vector<void*> temp_forms_;
};

// Device tensor handed across the ABI (CudaDeviceTensor).
struct DeviceTensorHandle {
  // handles that alias one allocation share this count; the last one released frees the memory
  std::shared_ptr<int> owners = std::make_shared<int>(0);
  void* ptr = nullptr;
  size_t bytes = 0;
  DT dt = DT::F32;
  Layout layout = Layout::PLAIN;
  std::vector<int64_t> shape;
};

// Pure predicates.
bool is_supported_op(const std::string& op);
bool accepts_resident_slot(const std::string& op, uint32_t slot);

}  // namespace oxb
