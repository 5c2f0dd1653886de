// Launch interface of the device kernels (glue, direct CUDA-core contractions, tcgen05
// contractions).  Everything here is host-callable and enqueues work on a stream; nothing
// synchronises.
#pragma once

#include "common.hpp"

namespace oxb {
namespace k {

// Canonical 4-D view used by the element-wise kernels.  Any tensor is viewed as logical
// [N, C, H, W]: rank-4 activations directly, a per-axis operation on another rank as
// (outer, axis extent, inner, 1), everything else as a flat run in N.
struct Dims4 {
  int64_t N, C, H, W;
  int64_t numel() const { return N * C * H * W; }
};

struct TensorRef {
  void* ptr;
  DT dt;
  Layout layout;
  Dims4 d;
};

// ---- layout / dtype conversion --------------------------------------------------------
// Copies `src` to `dst` element by element converting memory order and storage type
// (integers <-> f32 lanes are exact for every value the path stores; i32 -> f32 rounds to
// nearest even above 2^24 exactly like the reference's `as f32`).
void convert(const TensorRef& src, const TensorRef& dst, cudaStream_t s);

// ---- quantisation glue ------------------------------------------------------------------
// y = clamp(rne(x / scale[ch]) + zp[ch], lo, hi); f32 division and rounding, no FMA.
// scale/zp are device f32 arrays of length 1 (per tensor) or C (per channel of the view).
void quantize_linear(const TensorRef& x, const TensorRef& y, const float* scale, int64_t n_scale, const float* zp, int64_t n_zp, float lo,
                     float hi, cudaStream_t s);
// Same arithmetic with host-known per-tensor parameters and identical memory order on both
// sides: 16 lanes per thread through 16-byte accesses.  Fails if the operand is not eligible
// (callers check quantize_linear_scalar_ok first).
// f32 lanes -> f16 / bf16 lanes (round to nearest even), same memory order: the operand copy a 16-bit float
// contraction reads.  6 B per element.
void convert_f32_to_half(const float* src, void* dst, DT dst_dt, int64_t n, cudaStream_t s);
// y = x rounded to TF32 (cvt.rna), lane by lane: the operand copy of a TF32 contraction whose input was not rounded
// by its producer (a graph input).  8 B per element.
void round_to_tf32_copy(const float* src, float* dst, int64_t n, cudaStream_t s);
bool quantize_linear_scalar_ok(const TensorRef& x, const TensorRef& y);
void quantize_linear_scalar(const TensorRef& x, const TensorRef& y, float scale, float zp, float lo, float hi, cudaStream_t s);
// y = (x - zp[ch]) * scale[ch], two separately rounded f32 operations.
void dequantize_linear(const TensorRef& x, const TensorRef& y, const float* scale, int64_t n_scale, const float* zp, int64_t n_zp,
                       cudaStream_t s);
// DynamicQuantizeLinear: params[0] = y_scale, params[1] = y_zero_point (f32 lanes on the
// device); `scratch` is 2 floats used for the min/max reduction.
// `have_minmax`: the producer of x has already merged x's extrema into the scratch keys; only the second pass runs.
void dynamic_quantize_linear(const TensorRef& x, const TensorRef& y, float* params, float* scratch, cudaStream_t s, bool have_minmax = false);
// Puts a freshly allocated scratch block (at least 12 bytes) into the state dynamic_quantize_linear expects.
void dynamic_quantize_scratch_init(float* scratch);

// The residual join of a quantised network in one pass:
//   y = Q( relu?( DQ(a) + DQ(b) ) )  with per-tensor parameters,
// performing the same f32 operations in the same order as the separate DequantizeLinear, Add,
// Relu and QuantizeLinear nodes (subtract, multiply, add, max, divide, round-half-even, add,
// clamp; none fused), so the lanes are bit-identical while the f32 intermediates never reach
// memory: 3 bytes of traffic per element instead of 27.  a, b and y are 8-bit tensors of the
// same shape and memory order.
struct ResidualParams {
  float a_scale, a_zp, b_scale, b_zp, y_scale, y_zp, lo, hi;
  int relu;
  // set by residual_requant_prepare(): 1 when the division-free lane gives the reference's result for every one of
  // the 256 x 256 input pairs (checked on the host, pair by pair); 2 when the pairwise form (f32x2 arithmetic, ReLU
  // folded into the lower clamp bound, packed 16-bit clamp) does so too; 0 otherwise (the IEEE division runs)
  int proven_fast;
  float y_rcp;
};
// Decides once, at plan time, whether the fast kernel may be used for these parameters.
void residual_requant_prepare(ResidualParams& rp, DT a_dt, DT b_dt);
void residual_requant(const void* a, DT a_dt, const void* b, DT b_dt, void* y, DT y_dt, int64_t n, const ResidualParams& rp, cudaStream_t s);

// ---- element-wise -----------------------------------------------------------------------
enum BinOp { BIN_ADD = 0, BIN_SUB = 1, BIN_MUL = 2, BIN_DIV = 3 };
enum UnOp { UN_RELU = 0, UN_TANH = 1, UN_SIGMOID = 2, UN_SILU = 3, UN_COPY = 4, UN_GELU_ERF = 5, UN_GELU_TANH = 6, UN_ERF = 7 };
// out = op(a, b) with numpy broadcasting expressed through per-axis extents of 1 in the
// views; optional fused relu afterwards; round_tf32 rounds the f32 result to TF32
// (round-to-nearest, ties away) for a following tensor-core contraction.
void binary(const TensorRef& a, const TensorRef& b, const TensorRef& out, int op, int relu_after, int round_tf32, cudaStream_t s);
void unary(const TensorRef& x, const TensorRef& y, int op, cudaStream_t s);
// y = x >= 0 ? x : x * slope[c or 0]
void prelu(const TensorRef& x, const TensorRef& y, const float* slope, int64_t n_slope, cudaStream_t s);

// ---- pooling / normalisation ------------------------------------------------------------
struct PoolShape {
  int kh, kw, sh, sw, pt, pl, dh, dw, P, Q;
};
void max_pool(const TensorRef& x, const TensorRef& y, const PoolShape& ps, cudaStream_t s);
// Sequential f32 sum over the plane in (h, w) order, then one division: the order the
// reference's global_avg_pool uses, so the result is bit-identical.
void global_avg_pool(const TensorRef& x, const TensorRef& y, int round_tf32, cudaStream_t s);
// The same sum over an 8-bit NHWC tensor dequantised on the fly with per-tensor parameters: (x - zp) * scale per
// lane, added in (h, w) order, i.e. DequantizeLinear followed by GlobalAveragePool without the f32 tensor between them.
void global_avg_pool_dequant(const TensorRef& x, const TensorRef& y, float scale, float zp, int round_tf32, cudaStream_t s);
// OxiInstanceNorm over (n, c) planes, two-pass variance about the mean; optional fused
// per-sample modulation y = norm * scale[n,c] + shift[n,c] (both may be NULL).
void instance_norm(const TensorRef& x, const TensorRef& y, float eps, const float* scale_nc, const float* shift_nc, int relu, int round_tf32,
                   cudaStream_t s);

// ---- spatial glue -----------------------------------------------------------------------
// mode 0 nearest, 1 linear; coord 0 half_pixel, 1 pytorch_half_pixel, 2 asymmetric,
// 3 align_corners; nearest_rule 0 round_prefer_floor, 1 floor, 2 ceil, 3 round_prefer_ceil
// `round_tf32`: interpolated lanes (linear mode) are rounded to TF32 when they feed a contraction.
void resize(const TensorRef& x, const TensorRef& y, int mode, int coord, int nearest_rule, float scale_h, float scale_w, int round_tf32, cudaStream_t s);
// mode 0 constant, 1 reflect, 2 edge (spatial and channel pads of a rank-4 view)
void pad(const TensorRef& x, const TensorRef& y, int mode, float value, int pn, int pc, int ph, int pw, cudaStream_t s);
// Copies `x` into the channel range [c_off, c_off + x.C) of `y` (Concat on the channel axis)
// or, axis 0/2/3, the matching range of that axis.
void concat_into(const TensorRef& x, const TensorRef& y, int axis, int64_t offset, cudaStream_t s);
// Transformer glue (f32, logical row-major order).  gather_rows: out[i, :] = table[idx[i], :] with index lanes
// as f32 (negative counts from the end; out of range records code 20 in *err).  transpose_perm: y of shape yd
// reads x through the strides xstride (the input stride of each output axis).  softmax_rows / layer_norm_rows:
// over the last axis of a [rows, n] view.
void gather_rows(const float* table, const float* idx, float* out, int64_t n_idx, int64_t rows, int64_t inner, int* err, cudaStream_t s);
void transpose_perm(const void* x, void* y, const Dims4& yd, const Dims4& xstride, cudaStream_t s);
// softmax_rows optionally applies x * scale[0] and + mask[row / rows_per_mask][:] first (fused Mul / Add producers).
void softmax_rows(const float* x, float* y, int64_t rows, int64_t n, const float* scale, const float* mask, int64_t rows_per_mask, int round_tf32,
                  cudaStream_t s);
// `x2`, when given, is added to `x` lane by lane first (the residual Add in front of the normalisation).
void layer_norm_rows(const float* x, float* y, int64_t rows, int64_t n, const float* scale, const float* bias, float eps, cudaStream_t s,
                     unsigned int* minmax_keys = nullptr, const float* x2 = nullptr);
// Slice with unit steps over logical (row-major) axes padded to four: y[i] = x[i + start], dims as (N, C, H, W).
void slice_rows(const void* x, void* y, DT dt, const Dims4& xd, const Dims4& yd, const Dims4& start, cudaStream_t s);

// Space-to-depth packing for stride-2 convolutions over very few channels (the 3-channel
// stem): dst[n][y][x][(bh*2+bw)*C + c] = src[n][c][2y+bh][2x+bw] - sub, channels padded with
// zeros up to c_pad, so that the convolution becomes a stride-1 one over 4*C channels whose
// rows are long enough for the tensor-core path.  src may be channels-first f32 lanes (a graph
// input) or a channels-last activation; dst is channels-last [N, H/2, W/2, c_pad].
void s2d_pack(const TensorRef& src, void* dst, DT dst_dt, int c_pad, int sub, cudaStream_t s);

// The same packing laid out for row windows: dst is [N][H/2][wp][16] with `pad_left` zero pixels
// in front of every row and zeros behind it, 16 lanes per pixel (4*C values, then zeros).  A
// window of s consecutive pixels is then s*16 contiguous lanes, which the tensor-core kernel
// reads as the "channels" of one filter-row tap (ConvShape::x_pixel_stride).  When `quantize` is
// set the source is f32 and each value is first quantised exactly as QuantizeLinear does,
// clamp(round_half_even(x / scale) + zp, lo, hi); `sub` is subtracted last.
struct S2dQuant {
  int quantize = 0;
  float scale = 1.f, zp = 0.f, lo = 0.f, hi = 255.f;
};
// `pair_top` >= 0 selects the row-pair form for 8-bit destinations: dst is [N][rows_phys][wp][32], physical row j
// holding the packed blocks of image rows j - pair_top and j - pair_top + 1 (zeros outside the image), so that a
// window of S2p pixels is 128 contiguous bytes covering two filter rows.
void s2d_window_pack(const TensorRef& src, void* dst, DT dst_dt, int pad_left, int wp, int sub, const S2dQuant& q, int pair_top, int rows_phys,
                     cudaStream_t s);
// The row-window layout for a stride-1 convolution over up to four f32 channels: [N][H][wp][4].
void window_pack_f32(const TensorRef& src, void* dst, int pad_left, int wp, cudaStream_t s);

// ---- contractions -----------------------------------------------------------------------
struct ConvShape {
  int N, C, H, W;     // input (per group channels = C / group)
  int OC, R, S;       // filter
  int P, Q;           // output spatial
  int sh, sw, pt, pl, pb, pr, dh, dw, group;
  // Tensor-core path only.  When non-zero, consecutive W positions of the stored activation are
  // x_pixel_stride elements apart (less than C: neighbouring positions overlap) and a stored row
  // holds x_row_pixels of them; zero means the dense layout (C and W).
  int x_pixel_stride = 0, x_row_pixels = 0;
  int64_t M() const { return (int64_t)N * P * Q; }
  int64_t K() const { return (int64_t)(C / group) * R * S; }
  double ops() const { return 2.0 * (double)M() * (double)OC * (double)K(); }
};

enum EpiMode { EPI_F32 = 0, EPI_REQUANT = 1, EPI_INT32 = 2, EPI_DEQUANT = 3 };

struct Epilogue {
  int mode = EPI_F32;
  // EPI_F32: out = act(acc + bias_f[oc]); act 0 none, 1 relu, 2 clip, 3 silu, 4 prelu (per-channel slope)
  const float* bias_f = nullptr;
  const float* slope = nullptr;  // act 4: [OC] padded like the bias
  int act = 0;
  float clip_lo = 0.f, clip_hi = 0.f;
  int round_tf32 = 0;
  // EPI_F32 with a fused residual: out = act((acc + bias_f[oc]) + residual[m * OC + oc]); the two
  // additions round as the separate Conv and Add nodes do
  const float* residual = nullptr;
  // integer modes.  Direct kernels subtract zero points per element; the tensor-core kernel
  // computes raw = sum(x*w) and applies acc = raw + bias_i[oc] - x_zp * wsum[oc].
  const int32_t* bias_i = nullptr;
  const float* bias_if = nullptr;  // tensor-core kernel: the folded integer bias as f32 lanes (every entry below 2^24), or null
  const int32_t* wsum = nullptr;
  int x_zp = 0;
  const float* x_zp_dev = nullptr;  // when set, the zero point is read from this device f32 lane
  const int32_t* x_zp_rows = nullptr;  // direct kernels: per-row zero point of a matmul A operand (length M)
  const int32_t* w_zp = nullptr;    // direct kernels: per-oc (n_w_zp == OC) or single
  int n_w_zp = 0;
  // EPI_REQUANT: q = clamp(rne(f64(acc) * f64(combined[oc]) + y_zp), lo, hi)
  const float* combined = nullptr;
  int64_t acc_abs_bound = 0;  // when > 0: no |raw + bias - x_zp * wsum| of this layer can exceed it (from the weights)
  int combined_fma_ok = 0;  // every combined[oc] is 0 or has 2^-21 <= |c| <= 2^40: the one-FMA requantisation is exact
  double q_abs_bound = 0;   // when > 0: no |acc * combined[oc] + y_zp| of this layer can exceed it (from acc_abs_bound and the scales)
  int y_zp = 0;
  int lo = 0, hi = 255;
  int relu_fused = 0;  // integer: clamp below at max(lo, 0) (a following Relu node)
  // EPI_DEQUANT (MatMulInteger -> Cast -> Mul(x_scale * w_scale[oc]) -> Add(bias[oc]) [-> Gelu], the chain a
  // dynamically quantised linear is exported as): out = f32(acc) * (x_scale * w_scale[oc]) + bias[oc], every
  // product and sum rounded separately as the unfused nodes do; dq_act 1 = exact Gelu, 2 = tanh Gelu
  const float* dq_w_scale = nullptr;      // [OC], padded like the other parameter vectors
  const float* dq_x_scale_dev = nullptr;  // one device lane (a DynamicQuantizeLinear scale)
  const float* dq_bias = nullptr;         // [OC], padded
  int dq_act = 0;
  DT out_dt = DT::F32;
  // tensor-core kernel, f32 outputs: two ordered u32 keys into which the kernel merges the extrema of what it writes
  // (the scratch of a DynamicQuantizeLinear that reads the output next), or null
  unsigned int* minmax_keys = nullptr;
};

// Direct CUDA-core convolution (and matmul as a 1x1 convolution): general geometry
// (groups, dilations, asymmetric pads), any zero points, i64 accumulation.
// x: NHWC (or PLAIN when x_plain_nchw, used by the stem to read a graph input directly),
// w: packed [R][S][C/group][OC] in w_dt, out: NHWC [M, OC].
void conv_direct(const void* x, DT x_dt, int x_plain_nchw, const void* w, DT w_dt, void* out, const ConvShape& cs, const Epilogue& e,
                 cudaStream_t s);

// Batched plain f32 matmul C[b] = A[b] (MxK) * B[b] (KxN) with optional broadcast of either
// side (stride 0), used for activation x activation products.
void matmul_f32_direct(const float* a, const float* b, float* c, int64_t batch, int64_t M, int64_t K, int64_t N, int64_t a_bstride,
                       int64_t b_bstride, cudaStream_t s);

// Batched TF32 products over strided windows of row-major f32 matrices (see umma_plan_create_batched).
struct BatchedGemm {
  const void* a = nullptr;
  int64_t a_rows = 0, a_cols = 0;
  const void* b = nullptr;  // [N][K] per item, K contiguous
  int64_t b_rows = 0, b_cols = 0;
  void* out = nullptr;
  int64_t o_rows = 0, o_cols = 0;
  int outer = 1, inner = 1;  // items = outer * inner
  int M = 0, N = 0, K = 0;   // per item
  int a_rb = 0, a_rh = 0, a_ch = 0, b_rb = 0, b_rh = 0, b_ch = 0, o_rb = 0, o_rh = 0, o_ch = 0;
  const float* zero_bias = nullptr;  // at least align_up(N, 256) zeros
  int round_tf32 = 0;
  unsigned int* minmax_keys = nullptr;  // as Epilogue::minmax_keys
};
struct UmmaPlan;
UmmaPlan* umma_plan_create_batched(const BatchedGemm& g, std::string* why);

// True when the driver accepts an im2col tensor map whose W stride is shorter than its channel
// extent (overlapping positions), which the row-window stem layout needs.
bool umma_overlapping_positions_ok();

// tcgen05 implicit-GEMM plan (tensor maps are built once at plan time).
struct UmmaPlan;
// kind: 0 = i8 (A u8/s8, B s8/u8, s32 accumulate), 1 = tf32 (f32 storage, f32 accumulate), 2 = f16, 3 = bf16
// (16-bit storage, f32 accumulate).  Returns nullptr with `why` filled when the shape is not eligible.
// Choices a context may override (oxb200_config): `requant_f64` 1 keeps the two-pass f64 requantisation even where
// the one-FMA form is proven, 2 keeps the one-FMA form without the packed 16-bit saturation; `split_k_max` bounds the slices of a split reduction (0: the default of 8, 1: never
// split); `cta_pairs` 0 lets the tile model decide, 1 never pairs CTAs, 2 pairs them wherever the shape allows.
struct UmmaTuning {
  int requant_f64 = 0;
  int split_k_max = 0;
  int cta_pairs = 0;
};
UmmaPlan* umma_plan_create(const void* x, DT x_dt, const void* w_packed, DT w_dt, void* out, const ConvShape& cs, const Epilogue& e, int kind,
                           const UmmaTuning& tune, std::string* why);
void umma_plan_destroy(UmmaPlan* p);
// After a launch that gave up (error word set): puts a split-K plan's arrival counters back to zero, so that the
// next launch does not inherit a half-counted tile.  A no-op for plans that do not split K.
void umma_plan_reset_after_error(UmmaPlan* p);
void umma_launch(const UmmaPlan* p, int* err_flag, cudaStream_t s);
const char* umma_plan_desc(const UmmaPlan* p);
// Re-point a plan at new buffers (arena moved) is not supported: plans are rebuilt.

// A chain of quantised linear layers over at most 64 rows as one cooperative tcgen05 kernel: layer i reads
// [rows][K] 8-bit lanes at `x`, multiplies by the packed [N][K] 8-bit weights at `w`, requantises
// (q = clamp(rne(f64(acc + bias_i[ch]) * f64(combined[ch]) + y_zp), lo, hi)) and writes [rows][N] 8-bit lanes at
// `out`, which must be layer i+1's `x`.  Returns nullptr with `why` filled when the chain is not eligible (then
// every layer runs as its own plan).
struct UmmaChainLayer {
  const void* x = nullptr;
  DT x_dt = DT::U8;
  const void* w = nullptr;
  DT w_dt = DT::I8;
  void* out = nullptr;
  int K = 0, N = 0;
  const int32_t* bias_i = nullptr;
  const float* combined = nullptr;
  int y_zp = 0, lo = 0, hi = 255;
  int fma_exact = 0;  // every combined[ch] is 0 or within [2^-21, 2^40]: fma(acc, c, 1.5 * 2^23 + zp) is the exact requantisation for |acc| < 2^24
};
// Optional ends of a chain: `head_x` (f32 [rows][K of the first layer], 16-byte aligned) makes the first layer
// quantise its own input, q = clamp(rint(x / scale) + zp, lo, hi), instead of reading 8-bit rows; `tail_out`
// (f32 [rows][N of the last layer]) also receives (q - zp) * scale of the last layer's rows.
struct UmmaChainEnds {
  const float* head_x = nullptr;
  float head_scale = 1.f, head_zp = 0.f, head_lo = 0.f, head_hi = 255.f;
  float* tail_out = nullptr;
  float tail_scale = 1.f, tail_zp = 0.f;
  int tail_signed = 0;
};
struct UmmaChain;
UmmaChain* umma_chain_create(const UmmaChainLayer* layers, int n_layers, int rows, const UmmaChainEnds& ends, std::string* why);
void umma_chain_destroy(UmmaChain* c);
// After a launch that gave up: clears the arrival counters and the grid barrier's counter.
void umma_chain_reset_after_error(UmmaChain* c);
// false when the driver refused the cooperative launch (nothing ran): the caller runs the layers one by one
// `head_x`: where the f32 rows of a quantising head are for this launch (a graph input's buffer may change from run
// to run); ignored by a chain without one.
bool umma_chain_launch(const UmmaChain* c, int* err_flag, const float* head_x, cudaStream_t s);
const char* umma_chain_desc(const UmmaChain* c);

// One attention layer's f32 side as one tensor-core kernel (scores, scale + mask + softmax, context) for sequences
// of 128 positions and heads of 64 lanes.  q, k: [B * S, H * D] f32 matrices whose heads are column windows;
// vt: V transposed per head, [B * H * D, S]; out: [o_rows, o_cols] f32 where head (b, h) starts at row
// b * o_rb + h * o_rh and column h * o_ch; scale: one device lane or null; mask: [B][S] additive lanes or null.
struct FusedAttention {
  const float* q = nullptr;
  const float* k = nullptr;
  const float* vt = nullptr;
  float* out = nullptr;
  int64_t o_rows = 0, o_cols = 0;
  int o_rb = 0, o_rh = 0, o_ch = 0;
  int B = 0, H = 0, S = 0, D = 0;
  const float* scale = nullptr;
  const float* mask = nullptr;
  int round_probs = 1;                  // the probabilities feed a TF32 product
  unsigned int* minmax_keys = nullptr;  // as Epilogue::minmax_keys, for the context
};
struct UmmaAttentionPlan;
UmmaAttentionPlan* umma_attention_create(const FusedAttention& a, std::string* why);
void umma_attention_destroy(UmmaAttentionPlan* p);
void umma_attention_launch(const UmmaAttentionPlan* p, int* err_flag, cudaStream_t s);
const char* umma_attention_desc(const UmmaAttentionPlan* p);

// Packed weight size helpers for the tensor-core path: weights are laid out [OC][R*S*Cpad]
// (K-major rows), Cpad = C rounded up to the channel block.
int umma_channel_block(int C, int kind);  // 0 when C is not eligible
inline int umma_elem_bytes(int kind) { return kind == 0 ? 1 : (kind == 1 ? 4 : 2); }
bool umma_available();                    // driver entry point for tensor-map encoding found
// Issue-rate probe: operations per second the tensor pipe reaches for `kind` (0 i8, 1 tf32, 2 f16, 3 bf16) on the
// current device with nothing to wait for; `err_flag` is a device word that records a wait that ran out.
double umma_probe_peak(int kind, int* err_flag, cudaStream_t s);

}  // namespace k
}  // namespace oxb
