"""Writes tests/golden/reference_vectors.json: the known-answer vectors that the reference
project's own tests hold for the dense-contraction hot path.

The reference is a Rust project and cannot be executed here, so the vectors are
transcribed from its test sources (each case cites file:line inside the oxionnx project).
When REFERENCE_ROOT names a checkout of the reference project the
script checks that every numeric literal sequence of every case really appears in the
cited line range, so a transcription slip cannot go unnoticed.  The JSON file is what the
test-suite reads; it needs no access to the reference tree.

Usage:  REFERENCE_ROOT=<checkout of oxionnx> python tests/golden/make_reference_vectors.py
"""
import json
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "reference_vectors.json")
REF = os.environ.get("REFERENCE_ROOT", "")


def t(data, shape):
    return {"data": [float(v) for v in data], "shape": list(shape)}


def s(v):
    return t([v], [1])


def tt(data, shape, dtype):
    """A typed tensor (TypedTensor with U8 / I8 storage): the declared element type travels with the lanes."""
    return dict(t(data, shape), dtype=dtype)


def iota(n, shape):
    """Written in the source as iota(n, shape) = 0, 1, ..., n-1."""
    return dict(t(range(n), shape), gen={"kind": "iota", "n": n})


def fill(v, n, shape):
    """Written in the source as vec![v; n] / &[v; n]."""
    return dict(t([v] * n, shape), gen={"kind": "fill", "v": v, "n": n})


W2 = "tests/w2_quantized_ops_e2e.rs"
ND = "oxionnx-ops/tests/qlinear_native_dtype_test.rs"
CC = "tests/conformance_conv.rs"
OC = "tests/op_conv_tests.rs"
W1 = "oxionnx-ops/tests/w1_conv_pool.rs"

CASES = [
    dict(name="matmul_integer_u8_with_zero_point", source=f"{W2}:119-144", op="MatMulInteger",
         inputs=[t([11, 7, 3, 10, 6, 2, 9, 5, 1, 8, 4, 0], [4, 3]), t([1, 4, 2, 5, 3, 6], [3, 2]), s(12.0), s(0.0)],
         attrs={}, expected=[t([-38, -83, -44, -98, -50, -113, -56, -128], [4, 2])], exact=True),
    dict(name="matmul_integer_i8_without_zero_points", source=f"{W2}:147-162", op="MatMulInteger",
         inputs=[t([1, 2, 3, 4, 5, 6], [2, 3]), t([-1, 2, 3, -4, 5, 6], [3, 2])],
         attrs={}, expected=[t([20, 12, 41, 24], [2, 2])], exact=True),
    dict(name="qlinear_matmul_u8_node_test", source=f"{W2}:169-197", op="QLinearMatMul",
         inputs=[t([208, 236, 0, 238, 3, 214, 255, 29], [2, 4]), s(0.0066), s(113.0),
                 t([152, 51, 244, 60, 26, 255, 0, 127, 246, 127, 254, 247], [4, 3]), s(0.00705), s(114.0), s(0.0107), s(118.0)],
         attrs={}, expected=[t([168, 115, 255, 1, 66, 151], [2, 3])], exact=True),
    dict(name="qlinear_matmul_i8_symmetric_keeps_negative_outputs", source=f"{W2}:206-232", op="QLinearMatMul",
         inputs=[t([1, -2, 3, 4, 5, -6], [2, 3]), s(0.5), s(0.0), t([-1, 2, 3, -4, 5, 6], [3, 2]), s(0.5), s(0.0), s(1.0), s(3.0)],
         attrs={}, expected=[t([5, 10, -2, -9], [2, 2])], exact=True),
    dict(name="qlinear_matmul_union_range", source=f"{W2}:686-712", op="QLinearMatMul",
         inputs=[t([10, 0, 0, 10], [2, 2]), s(1.0), s(0.0), t([10, -15, 0, 0], [2, 2]), s(1.0), s(0.0), s(1.0), s(100.0)],
         attrs={}, expected=[t([200, -50, 100, 100], [2, 2])], exact=True),
    dict(name="conv_integer_pads0", source=f"{W2}:236-256", op="ConvInteger",
         inputs=[t([2, 3, 4, 5, 6, 7, 8, 9, 10], [1, 1, 3, 3]), t([1, 1, 1, 1], [1, 1, 2, 2]), s(1.0)],
         attrs={"pads": [0, 0, 0, 0]}, expected=[t([12, 16, 24, 28], [1, 1, 2, 2])], exact=True),
    dict(name="conv_integer_pads1", source=f"{W2}:236-275", op="ConvInteger",
         inputs=[t([2, 3, 4, 5, 6, 7, 8, 9, 10], [1, 1, 3, 3]), t([1, 1, 1, 1], [1, 1, 2, 2]), s(1.0)],
         attrs={"pads": [1, 1, 1, 1]},
         expected=[t([1, 3, 5, 3, 5, 12, 16, 9, 11, 24, 28, 15, 7, 15, 17, 9], [1, 1, 4, 4])], exact=True),
    dict(name="conv_integer_mixed_sign_zero_points", source=f"{W2}:278-300", op="ConvInteger",
         inputs=[t([2, 3, 4, 5, 6, 7, 8, 9, 10], [1, 1, 3, 3]), t([1, -1, 2, 3], [1, 1, 2, 2]), s(3.0), s(1.0)],
         attrs={"pads": [0, 0, 0, 0]}, expected=[t([8, 9, 11, 12], [1, 1, 2, 2])], exact=True),
    dict(name="qlinear_conv_node_test", source=f"{W2}:308-345", op="QLinearConv",
         inputs=[t([255, 174, 162, 25, 203, 168, 58, 15, 59, 237, 95, 129, 0, 64, 56, 242, 153, 221, 168, 12, 166, 232, 178, 186, 195,
                    237, 162, 237, 188, 39, 124, 77, 80, 102, 43, 127, 230, 21, 83, 41, 40, 134, 255, 154, 92, 141, 42, 148, 247],
                   [1, 1, 7, 7]),
                 s(0.003692047), s(132.0), t([0], [1, 1, 1, 1]), s(0.0017279458), s(255.0), s(0.0016268126), s(123.0)],
         attrs={},
         expected=[t([0, 81, 93, 230, 52, 87, 197, 240, 196, 18, 160, 126, 255, 191, 199, 13, 102, 34, 87, 243, 89, 23, 77, 69, 60, 18,
                      93, 18, 67, 216, 131, 178, 175, 153, 212, 128, 25, 234, 172, 214, 215, 121, 0, 101, 163, 114, 213, 107, 8],
                     [1, 1, 7, 7])], exact=True),
    dict(name="qlinear_conv_per_channel_scale_and_int32_bias", source=f"{W2}:356-396", op="QLinearConv",
         inputs=[t(list(range(1, 33)), [1, 2, 4, 4]), s(0.02), s(16.0),
                 t([1, -2, 3, 0, 2, 1, -1, 1, 0, 1, 2, -3, 1, 1, 1, 1], [2, 2, 2, 2]), t([0.5, 0.25], [2]), t([0.0, 0.0], [2]),
                 s(0.05), s(100.0), t([50.0, -60.0], [2])],
         attrs={"strides": [1, 1], "pads": [0, 0, 0, 0]},
         expected=[t([107, 108, 109, 111, 112, 113, 115, 116, 117, 95, 95, 96, 96, 97, 97, 98, 98, 99], [1, 2, 3, 3])], exact=True),
    dict(name="qlinear_conv_depthwise_same_upper", source=f"{W2}:401-441", op="QLinearConv",
         inputs=[t(list(range(1, 37)), [1, 4, 3, 3]), s(0.05), s(10.0),
                 t([130, 120, 140, 126, 128, 132, 124, 129, 127, 131, 125, 133, 135, 121, 138, 122], [4, 1, 2, 2]), s(0.4), s(128.0),
                 s(0.1), s(50.0)],
         attrs={"group": 4, "auto_pad": "SAME_UPPER", "kernel_shape": [2, 2]},
         expected=[t([47, 48, 38, 49, 50, 46, 52, 51, 50, 49, 49, 46, 50, 50, 44, 56, 56, 50, 60, 61, 39, 62, 63, 37, 57, 57, 47, 64,
                      65, 124, 67, 67, 134, 49, 49, 86], [1, 4, 3, 3])], exact=True),
    dict(name="qlinear_conv_int8_with_dilations", source=f"{W2}:446-480", op="QLinearConv",
         inputs=[t([-5, 3, 7, -2, 0, 9, 4, -8, 6, 1, -3, 2, 8, -6, 5, 0], [1, 1, 4, 4]), s(0.5), s(0.0), t([2, -1, 1, 3], [1, 1, 2, 2]),
                 s(0.5), s(0.0), s(0.25), s(-5.0)],
         attrs={"dilations": [2, 2], "pads": [0, 0, 0, 0]}, expected=[t([-25, 10, 14, 15], [1, 1, 2, 2])], exact=True),
    dict(name="qlinear_conv_rejects_zero_output_scale", source=f"{W2}:485-540", op="QLinearConv",
         inputs=[t([1, 2, 3, 4], [1, 1, 2, 2]), s(0.1), s(0.0), t([1], [1, 1, 1, 1]), s(0.1), s(0.0), s(0.0), s(0.0)],
         attrs={}, error_contains="scale is zero"),
    dict(name="dynamic_quantize_linear_matches_reference", source=f"{W2}:542-571", op="DynamicQuantizeLinear",
         inputs=[t([0.0, 2.0, -3.0, -2.5, 1.34, 0.5], [6])], attrs={},
         expected=[t([153, 255, 0, 26, 221, 179], [6]), t([0.019607844], []), t([153], [])], exact=[True, 1e-9, True]),
    dict(name="dynamic_quantize_linear_2d_preserves_shape", source=f"{W2}:574-606", op="DynamicQuantizeLinear",
         inputs=[t([1.5, 2.5, 3.5, -1.0, -2.0, 0.0], [2, 3])], attrs={},
         expected=[t([163, 209, 255, 47, 0, 93], [2, 3]), t([0.02156863], []), t([93], [])], exact=[True, 1e-8, True]),
    dict(name="matmul_integer_rejects_mis_sized_zero_point", source=f"{W2}:717-748", op="MatMulInteger",
         inputs=[t([1, 2, 3, 4, 5, 6], [2, 3]), t([1, 2, 3, 4, 5, 6], [3, 2]), t([1, 2, 3], [3])],
         attrs={}, error_contains="a_zero_point has 3 entries"),
    # The registered DynamicQuantizeLinear agrees with the library helper on non-degenerate
    # inputs (dynamic.rs:210-233), so the helper's pinned vectors pin the operator too.
    dict(name="dynamic_quantize_zero_point_added_after_rounding", source="oxionnx-ops/src/quantized/tests/dynamic.rs:141-153",
         op="DynamicQuantizeLinear", inputs=[t([-128.0, -127.5, 0.0, 24.5, 25.5, 127.0], [6])], attrs={},
         expected=[t([0.0, 0.0, 128.0, 152.0, 154.0, 255.0], [6]), t([1.0], []), t([128], [])], exact=True),
    dict(name="dynamic_quantize_zero_point_ties_to_even", source="oxionnx-ops/src/quantized/tests/dynamic.rs:192-203",
         op="DynamicQuantizeLinear", inputs=[t([-0.5, 254.5], [2])], attrs={},
         expected=[t([0.0, 254.0], [2]), t([1.0], []), t([0], [])], exact=True),
    dict(name="quantize_linear_per_channel_axis0", source="oxionnx-ops/tests/w1_indexing_quant.rs:421-441", op="QuantizeLinear",
         inputs=[t([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], [2, 3]), t([1.0, 10.0], [2])], attrs={"axis": 0},
         expected=[t([1.0, 2.0, 3.0, 0.0, 0.0, 1.0], [2, 3])], exact=True),
    dict(name="quantize_linear_per_channel_axis1", source="oxionnx-ops/tests/w1_indexing_quant.rs:444-456", op="QuantizeLinear",
         inputs=[t([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], [2, 3]), t([1.0, 2.0, 4.0], [3])], attrs={"axis": 1},
         expected=[t([1.0, 1.0, 1.0, 4.0, 2.0, 2.0], [2, 3])], exact=True),
    dict(name="quantize_linear_per_channel_zero_point", source="oxionnx-ops/tests/w1_indexing_quant.rs:459-469", op="QuantizeLinear",
         inputs=[t([5.0, 15.0, 7.0, 3.0], [2, 2]), t([1.0, 1.0], [2]), t([2.0, 100.0], [2])], attrs={"axis": 0},
         expected=[t([7.0, 17.0, 107.0, 103.0], [2, 2])], exact=True),
    dict(name="dequantize_linear_per_channel_axis0", source="oxionnx-ops/tests/w1_indexing_quant.rs:472-482", op="DequantizeLinear",
         inputs=[t([10.0, 20.0, 30.0, 40.0], [2, 2]), t([2.0, 0.5], [2]), t([1.0, 2.0], [2])], attrs={"axis": 0},
         expected=[t([18.0, 38.0, 14.0, 19.0], [2, 2])], exact=True),
    dict(name="gemm_alpha_beta_full_bias", source="oxionnx-ops/tests/w2_perf_matmul.rs:170-181", op="Gemm",
         inputs=[t([1, 2, 3, 4, 5, 6], [2, 3]), t([1, 0, 1, 0, 1, 0, 1, 1, 1], [3, 3]), t([1, 2, 3, 4, 5, 6], [2, 3])],
         attrs={"alpha": 2.0, "beta": 0.5}, expected=[t([8.5, 11.0, 9.5, 22.0, 24.5, 23.0], [2, 3])], exact=1e-5),
    dict(name="gemm_c_1xn", source="oxionnx-ops/tests/w2_perf_matmul.rs:213-236", op="Gemm",
         inputs=[t([1, 0, 0, 1, 1, 1], [3, 2]), t([2, 3, 4, 5], [2, 2]), t([10, 20], [1, 2])],
         attrs={"alpha": 1.0, "beta": 1.0}, expected=[t([12, 23, 14, 25, 16, 28], [3, 2])], exact=1e-5),
    dict(name="gemm_stride_table_nn", source="oxionnx-ops/tests/w2_perf_matmul.rs:110-120", op="Gemm",
         inputs=[t([1, 2, 3, 4, 5, 6], [3, 2]), t([1, 2, 3, 4, 5, 6, 7, 8], [2, 4])], attrs={"alpha": 1.0, "beta": 0.0},
         expected=[t([11, 14, 17, 20, 23, 30, 37, 44, 35, 46, 57, 68], [3, 4])], exact=1e-5),
    dict(name="gemm_stride_table_tt", source="oxionnx-ops/tests/w2_perf_matmul.rs:110-120", op="Gemm",
         inputs=[t([1, 3, 5, 2, 4, 6], [2, 3]), t([1, 5, 2, 6, 3, 7, 4, 8], [4, 2])],
         attrs={"alpha": 1.0, "beta": 0.0, "transA": 1, "transB": 1},
         expected=[t([11, 14, 17, 20, 23, 30, 37, 44, 35, 46, 57, 68], [3, 4])], exact=1e-5),
    dict(name="matmul_m1_numpy", source="oxionnx-ops/tests/w2_perf_matmul.rs:265-280", op="MatMul",
         inputs=[t([-1.486, -0.003, 0.406, -1.885, -1.408], [1, 5]),
                 t([1.713, -1.718, -1.481, 1.793, 0.488, -0.524, 0.046, 0.651, -0.899, -1.448, 1.152, 0.681, 0.05, 1.267, 0.196], [5, 3])],
         attrs={}, expected=[t([0.126859, -1.139666, 0.277691], [1, 3])], exact=1e-4),
    dict(name="matmul_batched_m1_numpy", source="oxionnx-ops/tests/w2_perf_matmul.rs:283-316", op="MatMul",
         inputs=[t([0.962, -0.591, 0.107, -0.033, -0.293, 0.183], [2, 1, 3]),
                 t([-0.529, 0.604, 0.735, -0.742, -0.066, -0.446, -0.834, 0.792, -0.14, -0.705, 0.347, -0.596, 0.803, -0.566, -0.934,
                    -0.598, -0.309, -0.062, 0.812, 0.395, -0.321, -0.966, -0.68, 0.993], [2, 3, 4])],
         attrs={}, expected=[t([-0.484872, 0.769199, 1.237093, -1.245648, 0.005295, -0.139934, -0.331534, 0.085718], [2, 1, 4])],
         exact=1e-4),
    # ---- typed execution: the declared type of y_zero_point fixes the saturation range exactly ----
    dict(name="typed_qlinear_matmul_f32_zero_point_union", source=f"{ND}:164-174", op="QLinearMatMul",
         inputs=[t([10, 0, 0, 10], [2, 2]), s(1.0), s(0.0), t([10, -15, 0, 0], [2, 2]), s(1.0), s(0.0), s(1.0), s(100.0)],
         attrs={}, expected=[t([200, -50, 100, 100], [2, 2])], exact=True),
    dict(name="typed_qlinear_matmul_i8_zero_point", source=f"{ND}:178-186", op="QLinearMatMul",
         inputs=[tt([10, 0, 0, 10], [2, 2], "i8"), s(1.0), s(0.0), tt([10, -15, 0, 0], [2, 2], "i8"), s(1.0), s(0.0), s(1.0), tt([100], [1], "i8")],
         attrs={}, expected=[t([127, -50, 100, 100], [2, 2])], exact=True),
    dict(name="typed_qlinear_matmul_u8_zero_point", source=f"{ND}:194-202", op="QLinearMatMul",
         inputs=[tt([10, 0, 0, 10], [2, 2], "u8"), s(1.0), s(0.0), tt([10, -15, 0, 0], [2, 2], "i8"), s(1.0), s(0.0), s(1.0), tt([100], [1], "u8")],
         attrs={}, expected=[t([200, 0, 100, 100], [2, 2])], exact=True),
    dict(name="typed_qlinear_conv_f32_zero_point_union", source=f"{ND}:207-217", op="QLinearConv",
         inputs=[t([10, -15], [1, 1, 1, 2]), s(1.0), s(0.0), t([10], [1, 1, 1, 1]), s(1.0), s(0.0), s(1.0), s(100.0)],
         attrs={}, expected=[t([200, -50], [1, 1, 1, 2])], exact=True),
    dict(name="typed_qlinear_conv_i8_zero_point", source=f"{ND}:220-228", op="QLinearConv",
         inputs=[tt([10, -15], [1, 1, 1, 2], "i8"), s(1.0), s(0.0), tt([10], [1, 1, 1, 1], "i8"), s(1.0), s(0.0), s(1.0), tt([100], [1], "i8")],
         attrs={}, expected=[t([127, -50], [1, 1, 1, 2])], exact=True),
    dict(name="typed_qlinear_conv_u8_zero_point", source=f"{ND}:231-239", op="QLinearConv",
         inputs=[tt([10, -15], [1, 1, 1, 2], "i8"), s(1.0), s(0.0), tt([10], [1, 1, 1, 1], "i8"), s(1.0), s(0.0), s(1.0), tt([100], [1], "u8")],
         attrs={}, expected=[t([200, 0], [1, 1, 1, 2])], exact=True),
    # the same table through Session::run_typed (typed graph inputs)
    dict(name="run_typed_qlinear_matmul_u8", source="tests/qlinear_run_typed_e2e.rs:63-104", op="QLinearMatMul",
         inputs=[tt([10, 0, 0, 10], [2, 2], "u8"), s(1.0), s(0.0), tt([10, -15, 0, 0], [2, 2], "i8"), s(1.0), s(0.0), s(1.0), tt([100], [1], "u8")],
         attrs={}, expected=[t([200.0, 0.0, 100.0, 100.0], [2, 2])], exact=True),
    dict(name="run_typed_qlinear_matmul_i8", source="tests/qlinear_run_typed_e2e.rs:63-119", op="QLinearMatMul",
         inputs=[tt([10, 0, 0, 10], [2, 2], "u8"), s(1.0), s(0.0), tt([10, -15, 0, 0], [2, 2], "i8"), s(1.0), s(0.0), s(1.0), tt([100], [1], "i8")],
         attrs={}, expected=[t([127.0, -50.0, 100.0, 100.0], [2, 2])], exact=True),
    dict(name="run_typed_qlinear_matmul_f32_zero_point_union", source="tests/qlinear_run_typed_e2e.rs:63-134", op="QLinearMatMul",
         inputs=[tt([10, 0, 0, 10], [2, 2], "u8"), s(1.0), s(0.0), tt([10, -15, 0, 0], [2, 2], "i8"), s(1.0), s(0.0), s(1.0), s(100.0)],
         attrs={}, expected=[t([200.0, -50.0, 100.0, 100.0], [2, 2])], exact=True),
    # ---- float Conv and MaxPool: geometry, auto_pad, typed errors ----
    dict(name="conformance_conv2d_1x1", source=f"{CC}:15-54", op="Conv",
         inputs=[t([1, 2, 3, 4, 5, 6, 7, 8], [1, 2, 2, 2]), t([1, 0, 0, 1, 1, 1], [3, 2, 1, 1])],
         attrs={"strides": [1, 1], "pads": [0, 0, 0, 0], "dilations": [1, 1], "group": 1},
         expected=[t([1, 2, 3, 4, 5, 6, 7, 8, 6, 8, 10, 12], [1, 3, 2, 2])], exact=1e-5),
    dict(name="conformance_conv2d_3x3_pad1", source=f"{CC}:57-91", op="Conv",
         inputs=[fill(1.0, 9, [1, 1, 3, 3]), fill(1.0, 9, [1, 1, 3, 3])],
         attrs={"strides": [1, 1], "pads": [1, 1, 1, 1], "dilations": [1, 1], "group": 1},
         expected=[t([4, 6, 4, 6, 9, 6, 4, 6, 4], [1, 1, 3, 3])], exact=1e-5),
    dict(name="conformance_maxpool_2x2", source=f"{CC}:94-125", op="MaxPool", inputs=[t(range(1, 17), [1, 1, 4, 4])],
         attrs={"kernel_shape": [2, 2], "strides": [2, 2], "pads": [0, 0, 0, 0]}, expected=[t([6, 8, 14, 16], [1, 1, 2, 2])], exact=1e-5),
    dict(name="conv2d_dilated", source=f"{OC}:15-44", op="Conv", inputs=[fill(1.0, 25, [1, 1, 5, 5]), fill(1.0, 4, [1, 1, 2, 2])],
         attrs={"strides": [1, 1], "pads": [0, 0, 0, 0], "dilations": [2, 2], "group": 1}, expected=[fill(4.0, 9, [1, 1, 3, 3])], exact=1e-5),
    dict(name="conv2d_grouped", source=f"{OC}:47-76", op="Conv", inputs=[fill(1.0, 36, [1, 4, 3, 3]), fill(1.0, 8, [4, 2, 1, 1])],
         attrs={"strides": [1, 1], "pads": [0, 0, 0, 0], "dilations": [1, 1], "group": 2}, expected=[fill(2.0, 36, [1, 4, 3, 3])], exact=1e-5),
    dict(name="conv2d_stride2", source=f"{OC}:79-109", op="Conv", inputs=[t(range(1, 17), [1, 1, 4, 4]), fill(1.0, 4, [1, 1, 2, 2])],
         attrs={"strides": [2, 2], "pads": [0, 0, 0, 0], "dilations": [1, 1], "group": 1}, expected=[t([14, 22, 46, 54], [1, 1, 2, 2])], exact=1e-5),
    dict(name="conv2d_batch_n", source=f"{OC}:144-170", op="Conv", inputs=[fill(1.0, 36, [4, 1, 3, 3]), fill(1.0, 4, [1, 1, 2, 2])],
         attrs={"strides": [1, 1], "pads": [0, 0, 0, 0], "dilations": [1, 1], "group": 1}, expected=[fill(4.0, 16, [4, 1, 2, 2])], exact=1e-5),
    dict(name="conv_auto_pad_same_upper", source=f"{W1}:89-108", op="Conv", inputs=[iota(25, [1, 1, 5, 5]), fill(1.0, 9, [1, 1, 3, 3])],
         attrs={"auto_pad": "SAME_UPPER"},
         expected=[t([12, 21, 27, 33, 24, 33, 54, 63, 72, 51, 63, 99, 108, 117, 81, 93, 144, 153, 162, 111, 72, 111, 117, 123, 84], [1, 1, 5, 5])],
         exact=1e-4),
    dict(name="conv_auto_pad_same_upper_stride2", source=f"{W1}:110-127", op="Conv", inputs=[iota(36, [1, 1, 6, 6]), fill(1.0, 9, [1, 1, 3, 3])],
         attrs={"auto_pad": "SAME_UPPER", "strides": [2, 2]}, expected=[t([63, 81, 63, 171, 189, 135, 168, 180, 126], [1, 1, 3, 3])], exact=1e-4),
    dict(name="conv_auto_pad_same_lower_stride2", source=f"{W1}:110-139", op="Conv", inputs=[iota(36, [1, 1, 6, 6]), fill(1.0, 9, [1, 1, 3, 3])],
         attrs={"auto_pad": "SAME_LOWER", "strides": [2, 2]}, expected=[t([14, 30, 42, 75, 126, 144, 147, 234, 252], [1, 1, 3, 3])], exact=1e-4),
    dict(name="conv_auto_pad_valid_overrides_pads", source=f"{W1}:142-158", op="Conv", inputs=[iota(25, [1, 1, 5, 5]), fill(1.0, 9, [1, 1, 3, 3])],
         attrs={"auto_pad": "VALID", "pads": [1, 1, 1, 1]}, expected=[t([54, 63, 72, 99, 108, 117, 144, 153, 162], [1, 1, 3, 3])], exact=1e-4),
    dict(name="conv_rejects_unknown_auto_pad", source=f"{W1}:161-174", op="Conv", inputs=[iota(25, [1, 1, 5, 5]), fill(1.0, 9, [1, 1, 3, 3])],
         attrs={"auto_pad": "SAME"}, error_kind="Unsupported"),
    dict(name="conv_zero_stride_is_typed_error", source=f"{W1}:179-192", op="Conv", inputs=[iota(25, [1, 1, 5, 5]), fill(1.0, 9, [1, 1, 3, 3])],
         attrs={"strides": [0, 0]}, error_kind="ShapeMismatch"),
    dict(name="conv_zero_group_is_typed_error", source=f"{W1}:195-208", op="Conv", inputs=[iota(25, [1, 1, 5, 5]), fill(1.0, 9, [1, 1, 3, 3])],
         attrs={"group": 0}, error_kind="ShapeMismatch"),
    dict(name="conv_kernel_larger_than_padded_input", source=f"{W1}:211-227", op="Conv", inputs=[t([1.0], [1, 1, 1, 1]), fill(1.0, 9, [1, 1, 3, 3])],
         attrs={}, error_kind="ShapeMismatch"),
    dict(name="conv_dilation_beyond_input_extent", source=f"{W1}:230-244", op="Conv", inputs=[iota(25, [1, 1, 5, 5]), fill(1.0, 9, [1, 1, 3, 3])],
         attrs={"dilations": [4, 4]}, error_kind="ShapeMismatch"),
    dict(name="conv_negative_pads", source=f"{W1}:247-260", op="Conv", inputs=[iota(25, [1, 1, 5, 5]), fill(1.0, 9, [1, 1, 3, 3])],
         attrs={"pads": [-1, 0, 0, 0]}, error_kind="ShapeMismatch"),
    dict(name="conv_non_4d_input", source=f"{W1}:263-275", op="Conv", inputs=[iota(5, [1, 1, 5]), fill(1.0, 9, [1, 1, 3, 3])],
         attrs={}, error_kind="ShapeMismatch"),
    dict(name="max_pool_ceil_mode_1", source=f"{W1}:280-297", op="MaxPool", inputs=[iota(25, [1, 1, 5, 5])],
         attrs={"kernel_shape": [2, 2], "strides": [2, 2], "ceil_mode": 1}, expected=[t([6, 8, 9, 16, 18, 19, 21, 23, 24], [1, 1, 3, 3])], exact=1e-4),
    dict(name="max_pool_ceil_mode_0", source=f"{W1}:280-309", op="MaxPool", inputs=[iota(25, [1, 1, 5, 5])],
         attrs={"kernel_shape": [2, 2], "strides": [2, 2]}, expected=[t([6, 8, 16, 18], [1, 1, 2, 2])], exact=1e-4),
    dict(name="max_pool_h4_k3_s2_ceil", source=f"{W1}:312-329", op="MaxPool", inputs=[iota(16, [1, 1, 4, 4])],
         attrs={"kernel_shape": [3, 3], "strides": [2, 2], "ceil_mode": 1}, expected=[t([10, 11, 14, 15], [1, 1, 2, 2])], exact=1e-4),
    dict(name="max_pool_h4_k3_s2_floor", source=f"{W1}:312-336", op="MaxPool", inputs=[iota(16, [1, 1, 4, 4])],
         attrs={"kernel_shape": [3, 3], "strides": [2, 2]}, expected=[t([10.0], [1, 1, 1, 1])], exact=1e-4),
    dict(name="max_pool_ceil_mode_drops_window_in_right_padding", source=f"{W1}:339-359", op="MaxPool", inputs=[iota(25, [1, 1, 5, 5])],
         attrs={"kernel_shape": [3, 3], "strides": [3, 3], "pads": [0, 0, 2, 2], "ceil_mode": 1}, expected=[t([12, 14, 22, 24], [1, 1, 2, 2])],
         exact=1e-4),
    dict(name="max_pool_dilations", source=f"{W1}:362-377", op="MaxPool", inputs=[iota(16, [1, 1, 4, 4])],
         attrs={"kernel_shape": [2, 2], "dilations": [2, 2]}, expected=[t([10, 11, 14, 15], [1, 1, 2, 2])], exact=1e-4),
    dict(name="max_pool_auto_pad_same_upper", source=f"{W1}:380-397", op="MaxPool", inputs=[iota(25, [1, 1, 5, 5])],
         attrs={"kernel_shape": [3, 3], "auto_pad": "SAME_UPPER"},
         expected=[t([6, 7, 8, 9, 9, 11, 12, 13, 14, 14, 16, 17, 18, 19, 19, 21, 22, 23, 24, 24, 21, 22, 23, 24, 24], [1, 1, 5, 5])], exact=1e-4),
]


def _numbers(text):
    """All numeric literals of a Rust snippet, as floats (underscores and type suffixes dropped)."""
    text = re.sub(r"//[^\n]*", "", text)
    out = []
    for m in re.finditer(r"(?<![A-Za-z_\d.])-?\d[\d_]*(?:\.[\d_]*)?(?:e-?\d+)?(?:f32|f64|i8|u8|i64|usize)?", text):
        tok = re.sub(r"(f32|f64|i8|u8|i64|usize)$", "", m.group(0)).replace("_", "")
        try:
            out.append(float(tok))
        except ValueError:
            pass
    return out


def _contains_run(hay, needle):
    n = len(needle)
    if n == 0:
        return True
    for i in range(len(hay) - n + 1):
        if all(abs(hay[i + j] - needle[j]) <= 1e-9 * max(1.0, abs(needle[j])) for j in range(n)):
            return True
    return False


def verify_against_reference():
    """Each case's tensors must be findable as literal runs inside the cited lines."""
    problems = []
    for case in CASES:
        path, span = case["source"].rsplit(":", 1)
        lo, hi = (int(v) for v in span.split("-"))
        with open(os.path.join(REF, path)) as fh:
            lines = fh.readlines()
        # a generous window: helpers such as (1..=32) ranges are written as ranges there
        window = "".join(lines[max(lo - 12, 0):hi + 4])
        nums = _numbers(window)
        for tensor in case["inputs"] + case.get("expected", []):
            data = tensor["data"]
            gen = tensor.get("gen")
            if gen:  # written as a generator expression there, not as literals
                if gen["kind"] == "iota":
                    pat = rf"iota\({gen['n']}\b"
                else:
                    pat = rf"\[{gen['v']:.1f}(?:_f32)?; {gen['n']}\]"
                if not re.search(pat, window):
                    problems.append(f"{case['name']}: generator {gen} not found in {case['source']}")
                continue
            if len(data) <= 1:
                continue
            is_range = all(abs(data[i + 1] - data[i] - 1.0) < 1e-12 for i in range(len(data) - 1)) and len(data) > 8
            ok = _contains_run(nums, data)
            if not ok and is_range:
                ok = _contains_run(nums, [data[0], data[-1]])  # written as (a..=b)
            if not ok:
                problems.append(f"{case['name']}: tensor of {len(data)} values not found in {case['source']}")
    return problems


def main():
    if REF and os.path.isdir(REF):
        problems = verify_against_reference()
        if problems:
            print("\n".join(problems))
            sys.exit(1)
        print(f"verified {len(CASES)} cases against {REF}")
    else:
        print("reference tree not present: writing the transcription unverified")
    with open(OUT, "w") as fh:
        json.dump({"reference": "cool-japan/oxionnx v0.1.7", "cases": CASES}, fh, indent=1)
    print(f"wrote {OUT}")


if __name__ == "__main__":
    main()
