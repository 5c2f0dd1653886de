/*
 * CPU oracle for the dense-contraction hot path of OxiONNX (oxionnx v0.1.7).
 *
 * TEST INFRASTRUCTURE ONLY.  This library restates, on the host, the arithmetic of the
 * reference's registered CPU operators (oxionnx-ops) for the nodes the B200 path
 * implements.  It is the checker the device kernels are compared against and the CPU
 * baseline that is timed next to them; nothing in the shipped device path links,
 * loads or calls it.
 *
 * Parity status:
 *  - integer / quantised operators: exact restatement, pinned against the known-answer
 *    vectors of the reference's own tests (tests/golden/reference_vectors.json).
 *  - float operators (Conv, MatMul, Gemm, OxiInstanceNorm, ...): follow the operator
 *    definitions; the reference's float contraction lives in the third-party crate
 *    matrixmultiply 0.3 (not vendored), so the summation order is "parity unpinned".
 *
 * Convention (same as the reference): every tensor is a flat array of f32 lanes plus a
 * shape; quantised values are integers carried in f32 lanes.
 */
#ifndef OXI_ORACLE_H
#define OXI_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

#define OXO_MAX_RANK 8

/* status codes: 0 ok, negative = the OnnxError variant the reference would raise */
enum {
  OXO_OK = 0,
  OXO_ERR_SHAPE_MISMATCH = -1,   /* OnnxError::ShapeMismatch */
  OXO_ERR_INVALID_MODEL = -2,    /* OnnxError::InvalidModel  */
  OXO_ERR_UNSUPPORTED = -3,      /* OnnxError::Unsupported / UnsupportedOp */
  OXO_ERR_INTERNAL = -4
};

typedef struct {
  float* data;                 /* NULL + present==0: optional input omitted */
  int64_t shape[OXO_MAX_RANK];
  int32_t rank;
  int32_t present;
  int64_t len;                 /* number of lanes in data */
  int32_t dtype;               /* declared element type when it survived to the operator (TypedTensor): OXO_DT_* */
} oxo_tensor;

/* lanes are always f32; dtype only records what the tensor was declared as (oxionnx-core src/dtype.rs:8) */
enum { OXO_DT_UNTYPED = 0, OXO_DT_U8 = 1, OXO_DT_I8 = 2 };

enum { OXO_ATTR_INT = 0, OXO_ATTR_FLOAT = 1, OXO_ATTR_STRING = 2, OXO_ATTR_INTS = 3, OXO_ATTR_FLOATS = 4 };

typedef struct {
  const char* name;
  int32_t kind;
  int64_t i;
  float f;
  const char* s;
  const int64_t* ints;
  const float* floats;
  int64_t len;
} oxo_attr;

/* Run one operator.  Outputs are allocated by the oracle (release with oxo_free_tensor).
 * Returns OXO_OK or an error code; oxo_last_error() then holds the message. */
int oxo_run_node(const char* op_type, const oxo_tensor* inputs, int32_t n_inputs,
                 const oxo_attr* attrs, int32_t n_attrs, oxo_tensor* outputs, int32_t n_outputs);
void oxo_free_tensor(oxo_tensor* t);
const char* oxo_last_error(void);

/* threads == 1: the reference's own threading for the integer operators (none).
 * threads  > 1: the same arithmetic split over independent outputs (bit-identical for
 * the integer operators). */
void oxo_set_threads(int32_t threads);
int32_t oxo_get_threads(void);
/* 0: accumulate float contractions in f64 then round once (tight yardstick, the checker);
 * 1: accumulate in f32, sequentially (closer to what an f32 sgemm produces);
 * 2: the reference's algorithm and threading for float Conv / MatMul / Gemm -- im2col in blocks of at most
 *    64 MiB plus a blocked, packed sgemm with an 8x8 FMA register tile, jobs or row bands over the threads
 *    (oxionnx-ops src/conv/conv2d.rs:246-546, src/math_typed.rs:45): the TIMED CPU baseline, checked against
 *    mode 0 to 1e-5. */
void oxo_set_float_accum(int32_t mode);

/* scalar helpers exposed for unit tests */
double oxo_round_ties_even_f64(double v);
float oxo_round_ties_even_f32(float v);
float oxo_requantize(int64_t acc, float combined, int32_t zero_point, int64_t lo, int64_t hi);

#ifdef __cplusplus
}
#endif
#endif
