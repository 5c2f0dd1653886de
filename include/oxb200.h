/*
 * oxb200 -- C ABI of the B200 (sm_100a) execution provider for OxiONNX's dense-contraction
 * hot path: Conv, Gemm/MatMul, QLinearConv, QLinearMatMul, MatMulInteger, ConvInteger and
 * their quantise / dequantise / normalise glue.
 *
 * The entry points mirror, one for one, the Rust interface of the reference's CUDA
 * execution provider (crate oxionnx-cuda of cool-japan/oxionnx v0.1.7); each declaration
 * cites the reference item it replaces.  Conventions kept from the reference:
 *
 *  - Tensors cross the boundary as flat f32 lanes plus a shape (oxionnx-core
 *    src/tensor/types.rs:355).  Quantised values are integers carried in f32 lanes.
 *  - Three-way outcome (oxionnx-cuda src/error.rs:75-111, root crate
 *    src/session/run/sequential.rs:994-1032): DECLINED = "not mine, let the next provider
 *    try" (normal); FAILED = an error, the caller logs it and falls back; VERIFY_MISMATCH =
 *    the device result was proved wrong against the shadow check, the run must fail.
 *  - "Necessary, not sufficient": oxb200_is_supported_op()==0 guarantees a decline; 1 may
 *    still decline (oxionnx-cuda src/lib.rs:184-195).  Unknown attributes decline.
 *  - Malformed quantised inputs (non-finite lanes, zero scales, mis-sized zero points)
 *    decline so that the CPU operator raises its own typed error.
 *  - No exceptions, aborts or panics cross this boundary; every failure is a status plus a
 *    message readable through oxb200_last_error().
 *  - No CPU fallback exists inside the library: if no CUDA device or driver is present,
 *    oxb200_ctx_create fails.
 */
#ifndef OXB200_H
#define OXB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define OXB200_MAX_RANK 8

typedef struct oxb200_ctx oxb200_ctx;       /* replaces oxionnx_cuda::CudaContext (src/context.rs:219) */
typedef struct oxb200_tensor oxb200_tensor; /* replaces oxionnx_cuda::CudaDeviceTensor (src/activation.rs:85) */

/* Outcome of a dispatch: Result<Option<CudaDispatchOutcome>, OnnxError> flattened
 * (oxionnx-cuda src/activation.rs:221-245, src/lib.rs:561). */
enum {
  OXB200_OK_HOST = 0,         /* Ok(Some(Host(..)))   */
  OXB200_OK_DEVICE = 1,       /* Ok(Some(Device(..))) */
  OXB200_DECLINED = 2,        /* Ok(None)             */
  OXB200_FAILED = 3,          /* Err(e)               */
  OXB200_VERIFY_MISMATCH = 4  /* Err(e) with is_verify_mismatch(e) (src/error.rs:106) */
};

/* CudaOutputPlacement (oxionnx-cuda src/activation.rs:221) */
enum { OXB200_PLACE_HOST = 0, OXB200_PLACE_DEVICE = 1 };

/* One attribute of Attributes (oxionnx-core src/graph.rs:696-705). */
enum { OXB200_ATTR_INT = 0, OXB200_ATTR_FLOAT = 1, OXB200_ATTR_STRING = 2, OXB200_ATTR_INTS = 3, OXB200_ATTR_FLOATS = 4 };
typedef struct {
  const char* name;
  int32_t kind;
  int64_t i;
  float f;
  const char* s;
  const int64_t* ints;
  const float* floats;
  uint64_t len;
} oxb200_attr;

/* Node (oxionnx-core src/graph.rs:851): op, name, inputs ("" = omitted), outputs, attrs. */
typedef struct {
  const char* op_type;
  const char* name;
  const char* const* inputs;
  uint32_t n_inputs;
  const char* const* outputs;
  uint32_t n_outputs;
  const oxb200_attr* attrs;
  uint32_t n_attrs;
} oxb200_node;

/* Element types a typed buffer may have (DType, oxionnx-core src/dtype.rs:8-24; the subset this path stores). */
enum { OXB200_DT_F32 = 0, OXB200_DT_U8 = 1, OXB200_DT_I8 = 2, OXB200_DT_I32 = 3, OXB200_DT_F16 = 5, OXB200_DT_BF16 = 6 };

/* InputBinding (oxionnx-cuda src/activation.rs:285): a host tensor (f32 lanes) or a value
 * that already lives on the device.  A graph input that was declared with an 8-bit type
 * (oxb200_value_info.dtype) is fed through `typed` instead of `lanes`: `len` elements of
 * `dtype` in the logical (row-major) order, a quarter of the bytes of f32 lanes
 * (TypedTensor feeds of Session::run_typed, root crate src/session/run/entry.rs). */
typedef struct {
  const char* name;
  const float* lanes; /* host f32 lanes, NULL when `resident` or `typed` is set */
  uint64_t len;
  const uint64_t* shape;
  uint32_t rank;
  oxb200_tensor* resident;
  int32_t dtype;      /* OXB200_DT_* of `typed`; ignored when `typed` is NULL */
  const void* typed;  /* typed host lanes, or NULL */
} oxb200_operand;

/* One output of a dispatch or a fetch of a run. */
typedef struct {
  float* lanes;  /* caller-owned destination for host results (may be NULL when only a device result is wanted) */
  uint64_t cap;  /* capacity of `lanes` in elements */
  uint64_t len;  /* out: number of elements of the result */
  uint64_t shape[OXB200_MAX_RANK];
  uint32_t rank;
  oxb200_tensor* resident; /* out: device tensor when the outcome is OK_DEVICE */
} oxb200_result;

/* Declared shape and element type of a graph input (TensorInfo, oxionnx-core src/graph.rs:862).
 * dtype 0 (f32 lanes) is the reference's dtype-erased convention; U8 / I8 declare a quantised
 * input whose feeds arrive as typed 8-bit lanes and whose saturation is exact per type
 * (SatRange::for_dtype, oxionnx-ops src/registry/quant_ops/mod.rs:216-222). */
typedef struct {
  const char* name;
  const uint64_t* shape;
  uint32_t rank;
  int32_t dtype;
} oxb200_value_info;

/* Context options.  Zero-initialise, set struct_size, then override.  The environment
 * variables of the reference keep their names and truthiness rule (oxionnx-cuda
 * src/context.rs:40-45,179-192) and are read by oxb200_config_from_env(). */
typedef struct {
  uint32_t struct_size;
  int32_t verify;             /* OXIONNX_CUDA_VERIFY: shadow-verify hook enabled */
  int32_t strict;             /* OXIONNX_CUDA_STRICT */
  int32_t residency;          /* OXIONNX_CUDA_RESIDENCY (default 1) */
  int32_t cuda_graph;         /* OXIONNX_CUDA_GRAPH: replay a planned session as one CUDA graph */
  int32_t kernel_path;        /* 0 auto (tcgen05 where eligible), 1 force the direct CUDA-core kernels */
  int32_t keep_intermediates; /* 1: every value keeps a private arena slot (per-node inspection) */
  int32_t profile;            /* 1: record per-node CUDA-event timings during runs */
  int32_t requant_f64;        /* 1: requantise with the two-pass f64 form even where the one-FMA form is proven exact;
                                 2: the one-FMA form, but never its packed 16-bit saturation */
  int32_t split_k_max;        /* most slices a long reduction may be split into (0: default 8, 1: never split) */
  int32_t cta_pairs;          /* 0 the tile model decides, 1 never pair CTAs (cta_group::2), 2 pair wherever the shape allows */
  int32_t float_precision;    /* float contractions (Conv, Gemm, MatMul on the tensor cores): 0 TF32 operands (f32 storage),
                                 1 f16 operands, 2 bf16 operands; accumulation is f32 in every case, results are f32 lanes.
                                 The reference's counterpart is its mixed-precision session (src/session/mixed_precision) */
  int32_t reserved[4];
} oxb200_config;

/* CacheCounters (oxionnx-cuda src/residency.rs:141-240) plus arena figures. */
typedef struct {
  uint64_t uploads, upload_bytes;
  uint64_t downloads, download_bytes;
  uint64_t fences;
  uint64_t weight_uploads, weight_bytes_resident;
  uint64_t arena_bytes, arena_peak_bytes, arena_slots;
  uint64_t kernel_launches;
  uint64_t umma_launches, simt_launches, glue_launches;
  uint64_t dispatches, declines, failures;
  uint64_t graph_captures, graph_replays, graph_poisoned; /* graph_cache.rs: recordings made, replays, keys demoted */
} oxb200_counters;

/* ---- pure predicates (no device) ---------------------------------------------------- */

/* oxionnx_cuda::is_supported_op (src/lib.rs:217).  Adds the INT8 family the reference's
 * own CUDA provider never claimed. */
int oxb200_is_supported_op(const char* op_type);
/* oxionnx_cuda::accepts_resident_slot (src/lib.rs:419) */
int oxb200_accepts_resident_slot(const char* op_type, uint32_t slot);
/* decide_placement (root crate src/execution_providers.rs:352-387).  policy: 0 CpuOnly,
 * 1 Auto{gpu_threshold_bytes}, 2 Manual with `manual_pin` (0 unmapped, 1 pinned to CPU,
 * 2 pinned to this provider).  Returns 1 when the node goes to this provider. */
int oxb200_decide_placement(int policy, uint64_t gpu_threshold_bytes, int manual_pin, const char* op_type, uint64_t output_bytes);
/* is_verify_mismatch (src/error.rs:106): does the message carry the proved-wrong marker? */
int oxb200_is_verify_mismatch(const char* message);
/* env_flag truthiness (src/context.rs:179-192) and config assembly from the environment */
int oxb200_env_truthy(const char* value);
void oxb200_config_from_env(oxb200_config* cfg);

/* ---- context ------------------------------------------------------------------------- */

int oxb200_device_count(void);
/* CudaContext::try_new_with (src/context.rs:362-467): one context, one stream, one device.
 * A process may hold several contexts, on one device or on several (one per GPU for a batch split over
 * GPUs); calls on different contexts may run on different host threads at the same time, calls on one
 * context are serialised by the context's own lock. */
int oxb200_ctx_create(int device_ordinal, const oxb200_config* cfg, oxb200_ctx** out);
void oxb200_ctx_destroy(oxb200_ctx* ctx);
const char* oxb200_last_error(const oxb200_ctx* ctx); /* ctx may be NULL: last error of the calling thread */
/* CudaContext::cache_counters (src/context.rs:394-430) */
void oxb200_get_counters(const oxb200_ctx* ctx, oxb200_counters* out);
/* CudaContext::release_device_caches */
int oxb200_release_device_caches(oxb200_ctx* ctx);
/* Switches the per-node CUDA-event timing of planned runs (oxb200_config.profile) on or off for later runs;
 * the reference has no counterpart (its profiler wraps whole nodes on the host, src/session/profiling.rs). */
int oxb200_set_profile(oxb200_ctx* ctx, int on);

/* Peak rate of the tensor pipe on the context's device for one contraction kind (0 = kind::i8, 1 = kind::tf32,
 * 2 = kind::f16 with f16 operands, 3 = with bf16 operands): every SM issues a long run of tcgen05.mma
 * instructions on operands that are never refilled, and the call returns operations (two per multiply-add)
 * per second.  It is what the benchmark's roofline fractions are quoted against beside the cuBLAS-derived
 * figures; the reference has no counterpart.  Takes a few milliseconds. */
int oxb200_probe_tensor_peak(oxb200_ctx* ctx, int32_t kind, double* ops_per_second);

/* Page-locked host memory for feeds and fetches (the reference's pinned staging,
 * src/residency.rs:1147-1312, handed to the caller so no extra host copy is needed). */
void* oxb200_host_alloc(size_t bytes);
void oxb200_host_free(void* p);

/* ---- weights ------------------------------------------------------------------------- */

/* The `weights: &HashMap<String,Tensor>` argument of try_cuda_dispatch_resident
 * (src/lib.rs:561): initializers are registered once, are invariant for the context's
 * life, and are uploaded/packed on first use by a planned session or a dispatch
 * (initializer_id, src/dispatch_helpers.rs:21-64). The lanes are copied. */
int oxb200_weight_register(oxb200_ctx* ctx, const char* name, const float* lanes, uint64_t len, const uint64_t* shape, uint32_t rank);
/* The same with the element type the initializer was declared with in the model (TensorProto.data_type,
 * oxionnx-proto src/types.rs:9-24).  The lanes are still f32; the type is kept beside them and is what lets a
 * quantised operator whose y_zero_point is a uint8 / int8 initializer saturate to exactly that type
 * (SatRange::for_dtype, oxionnx-ops src/registry/quant_ops/mod.rs:216-222; pinned by the reference's
 * tests/qlinear_run_typed_e2e.rs:91-134) instead of the value-based union range. */
int oxb200_weight_register_typed(oxb200_ctx* ctx, const char* name, const float* lanes, uint64_t len, const uint64_t* shape, uint32_t rank, int32_t dtype);
/* CudaContext::is_weight_resident */
int oxb200_is_weight_resident(const oxb200_ctx* ctx, const char* name);

/* ---- per-node dispatch --------------------------------------------------------------- */

/* try_cuda_dispatch_resident (src/lib.rs:561) / try_cuda_dispatch (src/lib.rs:354).
 * `operands` are positionally aligned with node->inputs; an operand whose name is a
 * registered weight may pass lanes == NULL.  `results` has node->n_outputs entries. */
int oxb200_dispatch(oxb200_ctx* ctx, const oxb200_node* node, const oxb200_operand* operands, uint32_t n_operands, int want_placement,
                    oxb200_result* results, uint32_t n_results);

/* shadow_verify (oxionnx-cuda src/reference.rs:115-119,198-240): the caller owns the CPU
 * operators and hands the CPU result of the node just dispatched; a difference beyond
 * ATOL 1e-4 / RTOL 1e-3 is "proved wrong".  Returns OK_HOST, or VERIFY_MISMATCH under
 * strict mode / FAILED otherwise, with the reference's marker in the message. */
int oxb200_shadow_verify(oxb200_ctx* ctx, const char* op_type, const float* device_lanes, const float* cpu_lanes, uint64_t len);

/* CudaDeviceTensor::{shape,len,read_back} (src/activation.rs:116-208) and
 * CudaContext::recycle_activation (src/context.rs:394). */
int oxb200_tensor_shape(const oxb200_tensor* t, uint64_t* shape, uint32_t* rank, uint64_t* len);
int oxb200_tensor_read_back(oxb200_ctx* ctx, const oxb200_tensor* t, float* dst_lanes, uint64_t cap);
void oxb200_tensor_release(oxb200_ctx* ctx, oxb200_tensor* t);
/* CudaDeviceTensor::alias (src/activation.rs:150-163): another handle to the same allocation under another shape
 * of the same element count (what Reshape / Flatten of a resident value become).  DECLINED -- the reference's
 * None -- when the counts differ, or when the tensor is stored channels-last and the new shape would read its
 * bytes in another order.  The allocation lives until the last handle to it is released. */
int oxb200_tensor_alias(oxb200_ctx* ctx, const oxb200_tensor* t, const uint64_t* shape, uint32_t rank, oxb200_tensor** out);
/* CudaDeviceTensor::reserved_bytes (src/activation.rs:116-148): device bytes of the allocation behind the handle. */
uint64_t oxb200_tensor_reserved_bytes(const oxb200_tensor* t);
/* CudaContext::streams_unified (src/context.rs:384): every launch and copy of a dispatch or a run rides one queue
 * (always 1 here; the pipelined submit / collect pair orders its copy streams against it with events). */
int oxb200_streams_unified(const oxb200_ctx* ctx);
/* CudaContext::cached_device_bytes (src/context.rs:445): device bytes held for reuse (packed weight forms). */
uint64_t oxb200_cached_device_bytes(oxb200_ctx* ctx);
/* CudaContext::set_graph_capture / graph_capture_enabled (src/context.rs:416-424): whether later runs of a planned
 * session replay its step list as a CUDA graph; recordings already made are kept.  Never on under verification. */
int oxb200_set_graph_capture(oxb200_ctx* ctx, int on);
int oxb200_graph_capture_enabled(const oxb200_ctx* ctx);

/* ---- planned, device-resident session run --------------------------------------------- */

/* What Session::build_from_graph + StaticRunPlan::build + MemoryPlan::compute become
 * (root crate src/session/loading.rs:181, src/session/run/plan.rs:77,
 * src/memory/types.rs:347-452): shapes and device dtypes are inferred for every value,
 * weights are packed and uploaded, kernels are selected and every intermediate gets a
 * lifetime-planned slot of the device arena.  `nodes` must be topologically sorted.
 * Returns OK_DEVICE, or DECLINED/FAILED naming the first node the provider cannot take. */
int oxb200_session_plan(oxb200_ctx* ctx, const oxb200_node* nodes, uint32_t n_nodes, const oxb200_value_info* inputs, uint32_t n_inputs,
                        const char* const* outputs, uint32_t n_outputs);
/* Session::run (root crate src/session/run/entry.rs:92): host feeds in, host fetches out;
 * every intermediate stays in HBM.  Copies are asynchronous on the context's stream and
 * the call returns after one fence. */
int oxb200_run(oxb200_ctx* ctx, const oxb200_operand* feeds, uint32_t n_feeds, oxb200_result* fetches, uint32_t n_fetches);
/* Pipelined form of oxb200_run for throughput: submit enqueues the upload of one set of feeds (host lanes,
 * ideally page-locked) on a copy stream, the run, and the download of the outputs, and returns at once; collect
 * waits for the oldest submission and writes its outputs.  Up to two submissions may be in flight, so the copy
 * of the next batch overlaps the run of the current one.  The reference has no counterpart (its run is
 * synchronous, src/session/run/sequential.rs:468). */
int oxb200_run_submit(oxb200_ctx* ctx, const oxb200_operand* feeds, uint32_t n_feeds);
int oxb200_run_collect(oxb200_ctx* ctx, oxb200_result* fetches, uint32_t n_fetches);
/* Device time of the last oxb200_run in milliseconds, taken with CUDA events on the context's
 * stream from before the first host-to-device copy to after the last device-to-host copy. */
float oxb200_last_run_ms(const oxb200_ctx* ctx);

/* ---- device I/O binding -------------------------------------------------------------- */

/* IoBinding::bind_input / bind_output and Session::run_with_binding (root crate
 * src/io_binding.rs:42-58, src/session/run/entry.rs:109-139) extended to device memory, which
 * the reference's binding (host tensors only) cannot hold: a graph input or output of the
 * planned session is bound to a device buffer, so that consecutive runs exchange no bytes with
 * the host.
 *   bind_input_device   the input is read from `device_ptr` (`len` elements of the input's
 *                       declared dtype, logical row-major order, 16-byte aligned) by every
 *                       following run until it is bound again or the bindings are cleared;
 *                       the buffer stays the caller's and must outlive those runs.
 *   bind_output_device  the output's f32 lanes (logical order) are also written to
 *                       `device_ptr` (capacity `cap` elements) at the end of every run.
 *   output_device_ptr   the library-owned device buffer that holds an output's f32 lanes after
 *                       a run; it keeps its address for the life of the plan, so it can be bound
 *                       as the input of another plan or of the next run.
 *   run_bound           one run that touches the host only for inputs that are not bound
 *                       (`feeds` may be NULL when every input is bound) and fetches that are not
 *                       NULL; with everything bound it moves no bytes across PCIe and returns
 *                       after one fence.
 *   clear_bindings      forgets every binding; later runs upload and download as before. */
int oxb200_bind_input_device(oxb200_ctx* ctx, const char* name, const void* device_ptr, int32_t dtype, uint64_t len);
int oxb200_bind_output_device(oxb200_ctx* ctx, const char* name, void* device_ptr, uint64_t cap);
int oxb200_output_device_ptr(oxb200_ctx* ctx, const char* name, void** device_ptr, uint64_t* len);
int oxb200_run_bound(oxb200_ctx* ctx, const oxb200_operand* feeds, uint32_t n_feeds, oxb200_result* fetches, uint32_t n_fetches);
int oxb200_clear_bindings(oxb200_ctx* ctx);
/* The same run split for measurement: stage feeds, run the planned launches `iters`
 * times with everything resident (no host traffic), read fetches. */
int oxb200_upload_feeds(oxb200_ctx* ctx, const oxb200_operand* feeds, uint32_t n_feeds);
int oxb200_run_resident(oxb200_ctx* ctx, uint32_t iters, float* elapsed_ms);
int oxb200_download_fetches(oxb200_ctx* ctx, oxb200_result* fetches, uint32_t n_fetches);
/* Read any planned value after a run (needs keep_intermediates=1 for intermediates). */
int oxb200_fetch_value(oxb200_ctx* ctx, const char* name, oxb200_result* out);

/* Plan introspection (NodeProfile, root crate src/session/types.rs:18-27): one record per
 * planned step. */
typedef struct {
  const char* node_name;
  const char* op_type;
  const char* kernel;   /* which kernel family runs it */
  double work;          /* algorithmic ops (contractions) or bytes (glue) per launch */
  int32_t work_is_bytes;
  float last_ms;        /* CUDA-event time of the last profiled run (profile=1), else -1 */
  uint64_t launches;
  double bytes;         /* algorithmic bytes per launch: every operand and result once, plus a contraction's packed weights */
} oxb200_step_info;
uint32_t oxb200_plan_step_count(const oxb200_ctx* ctx);
int oxb200_plan_step_info(const oxb200_ctx* ctx, uint32_t index, oxb200_step_info* out);

/* ---- ONNX models ------------------------------------------------------------------------ */

/* What oxionnx_proto::load and the optimizer become on the host side of this provider (oxionnx-proto
 * src/model.rs:45-355, src/reader.rs, src/parser.rs; root crate src/optimizer/mod.rs:134-167): a model file is
 * parsed (protobuf wire format, no external dependency) into topologically sorted nodes, initializers as f32
 * lanes with their declared element types, and graph inputs / outputs; `optimize` runs the reference's fusions
 * for this path in its order -- MatMul+Add -> Gemm, Conv+BatchNormalization fold
 * (src/optimizer/fusion/conv/batchnorm.rs:17-188), Conv+Relu / Conv+Clip (relu.rs:69-179), Conv+Clip(0,6)
 * (relu6.rs:30), Mul(x, Sigmoid(x)) -> SiLU, the InstanceNorm-style chain -> OxiInstanceNorm
 * (src/optimizer/fusion/instance_norm.rs:199-268), Conv+Add+Relu -> ConvAddRelu (conv/add_relu.rs:27-156) --
 * and `session_plan_model` registers the initializers as the context's weights and plans the graph.  Features
 * the provider does not take (external data files, subgraph attributes, sparse initializers, string tensors)
 * are DECLINED with a message. */
typedef struct oxb200_model oxb200_model;
int oxb200_model_load(const void* bytes, uint64_t len, oxb200_model** out);
int oxb200_model_load_file(const char* path, oxb200_model** out);
void oxb200_model_free(oxb200_model* model);
/* level 0: nothing; 1: the passes above.  `removed` (optional) receives the number of nodes fused away. */
int oxb200_model_optimize(oxb200_model* model, int32_t level, uint32_t* removed);
/* One pass by the reference's function name ("fuse_conv_batchnorm", "fuse_conv_relu", "fuse_conv_clip_to_conv_relu6",
 * "fuse_instance_norm", "fuse_matmul_add", "fuse_mul_sigmoid_to_silu", "fuse_conv_add_relu"). */
int oxb200_model_run_pass(oxb200_model* model, const char* pass, uint32_t* removed);
/* Views into the model; they stay valid until the model is optimised again or freed.  A symbolic or missing input
 * dimension reads as UINT64_MAX; an input's dtype is an OXB200_DT_* code, or -1 for a type the boundary does not take. */
uint32_t oxb200_model_node_count(const oxb200_model* model);
int oxb200_model_node(oxb200_model* model, uint32_t index, oxb200_node* out);
uint32_t oxb200_model_input_count(const oxb200_model* model);
int oxb200_model_input(oxb200_model* model, uint32_t index, oxb200_value_info* out);
uint32_t oxb200_model_output_count(const oxb200_model* model);
const char* oxb200_model_output_name(const oxb200_model* model, uint32_t index);
uint32_t oxb200_model_initializer_count(const oxb200_model* model);
int oxb200_model_initializer(oxb200_model* model, uint32_t index, oxb200_operand* out); /* name, f32 lanes, shape, declared dtype */
/* Session::from_file + build (root crate src/session/loading.rs:181): the model's initializers become the
 * context's weights (typed), its graph is planned.  `shapes` supplies the concrete shape of every input that has
 * a symbolic dimension (and may override the others). */
int oxb200_session_plan_model(oxb200_ctx* ctx, oxb200_model* model, const oxb200_value_info* shapes, uint32_t n_shapes);

/* ---- allocation-free entry point -------------------------------------------------------- */

/* DynamicQuantizeLinear for hosts that are not allowed to allocate device memory while running
 * (a frame loop whose memory was fixed at start-up, another runtime's arena, a sandboxed plug-in).
 * This entry point has no counterpart in the reference.  It computes exactly what the
 * DynamicQuantizeLinear node of oxb200_dispatch computes, but everything it touches is either
 * passed in by the caller or part of the library image: it calls no cudaMalloc, no cudaFree and
 * no other allocating routine.
 *   x_device        n f32 lanes on the device, 16-byte aligned (the kernels read four lanes per load)
 *   y_device        n u8 lanes on the device (output), 4-byte aligned (four lanes per store)
 *   scale_zp_device 2 f32 lanes on the device (output: y_scale, y_zero_point), 4-byte aligned
 * A pointer that misses its alignment (a slice of a larger buffer at an odd offset) is rejected with
 * OXB200_FAILED before anything is launched.
 *   cuda_stream     a cudaStream_t of device `device_ordinal` (NULL: the default stream)
 * The reduction scratch is a 256-byte array inside the library, present on every GPU that loads
 * it until the process exits.  At most 2^28 lanes per call; larger inputs are rejected with
 * OXB200_FAILED and a message.  The first call for a device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current), so make that first call before any stream
 * capture.  All calls share the array: each call resets it on its stream first, and calls that
 * overlap on one GPU race on it -- serialise them.  Returns OXB200_OK_DEVICE once the work is
 * enqueued; the message of a failure is read with oxb200_last_error(NULL). */
int oxb200_dynamic_quantize_linear_noalloc(int device_ordinal, const float* x_device, uint64_t n, uint8_t* y_device, float* scale_zp_device,
                                           void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* OXB200_H */
