"""The ONNX loader and the host-side fusion passes, through the C ABI (oxb200_model_*), without a GPU.

The pass tests are the reference's own, case by case: src/optimizer/fusion/conv/tests.rs (Conv+BatchNormalization
fold with its numbers, Conv+Relu, Conv+Clip, Conv+Clip(0,6), Conv+Add+Relu with its input order and its declines),
src/optimizer/fusion/instance_norm_tests.rs (every spelling of the normalisation chain and every decline),
src/optimizer/fusion/matmul/matmul_add.rs and src/optimizer/fusion/simplify/functions.rs:346 (SiLU).  The loader
tests write models with the package's own ONNX writer and check what oxionnx-proto's loader is specified to
produce: typed tensors decoded to f32 lanes with the declared type kept, Constant nodes folded, initializers
dropped from the graph inputs, symbolic dimensions reported, malformed files rejected with a message.
"""
import numpy as np
import pytest

from oxionnx_b200 import _ffi, models, onnx_io
from oxionnx_b200.graph import Graph, Node
from oxionnx_b200.onnx_io import Model, ModelError


def model_of(nodes, weights=None, outputs=(), inputs=None, shapes=None):
    weights = weights or {}
    produced = {o for n in nodes for o in n.outputs}
    if inputs is None:
        inputs = []
        for n in nodes:
            for i in n.inputs:
                if i and i not in produced and i not in weights and i not in inputs:
                    inputs.append(i)
    shapes = shapes or {}
    g = Graph(nodes=list(nodes), input_names=list(inputs), output_names=list(outputs))
    data = onnx_io.write_onnx(g, weights, {i: (shapes.get(i, (2, 3, 4, 5)), np.float32) for i in inputs},
                              outputs={o: (shapes.get(o, ()), np.float32) for o in outputs})
    return Model.from_bytes(data)


def N(op, name, ins, outs, **attrs):
    return Node(op=op, name=name, inputs=list(ins), outputs=list(outs), attrs=attrs)


# ---- loader -------------------------------------------------------------------------------------
def test_loader_round_trip_of_nodes_attributes_initializers_and_value_infos():
    rng = np.random.default_rng(0)
    weights = {
        "w": rng.standard_normal((4, 3, 3, 3)).astype(np.float32), "zp_u8": np.uint8([131]), "zp_i8": np.int8([-7, 5]),
        "idx": np.int64([0, -1, 7]), "half": np.float16([1.0, -2.5, 0.0999755859375]), "i32": np.int32([[-5, 70000]]), "flag": np.array([True, False]),
        "d": np.float64([3.25]), "u16": np.uint16([65535]), "i16": np.int16([-32768]),
    }
    nodes = [N("Conv", "c0", ["x", "w"], ["y"], pads=[1, 1, 1, 1], strides=[2, 2], group=1, auto_pad="NOTSET", alpha=0.5, scales=[1.0, 2.5])]
    data = onnx_io.write_onnx(Graph(nodes, ["x"], ["y"]), weights, {"x": (("batch", 3, 8, 8), np.float32)}, outputs={"y": ((None, 4, 4, 4), np.float32)},
                              list_initializers_as_inputs=True)
    m = Model.from_bytes(data)
    (node,) = m.nodes()
    assert (node.op, node.name, node.inputs, node.outputs) == ("Conv", "c0", ["x", "w"], ["y"])
    assert node.attrs == {"pads": [1, 1, 1, 1], "strides": [2, 2], "group": 1, "auto_pad": "NOTSET", "alpha": 0.5, "scales": [1.0, 2.5]}
    # initializers listed among the inputs (the pre-IR-4 convention) are not graph inputs
    assert m.inputs() == [("x", (None, 3, 8, 8), _ffi.DT_F32)]
    assert m.output_names() == ["y"]
    ini = m.initializers()
    assert np.array_equal(ini["w"][0], weights["w"]) and ini["w"][1] == _ffi.DT_F32
    assert ini["zp_u8"] == (pytest.approx(np.float32([131])), _ffi.DT_U8) and ini["zp_i8"][1] == _ffi.DT_I8
    assert np.array_equal(ini["zp_i8"][0], np.float32([-7, 5]))
    assert np.array_equal(ini["idx"][0], np.float32([0, -1, 7]))
    assert np.array_equal(ini["half"][0], weights["half"].astype(np.float32)) and ini["half"][1] == _ffi.DT_F16
    assert np.array_equal(ini["i32"][0], np.float32([[-5, 70000]])) and ini["i32"][1] == _ffi.DT_I32
    assert np.array_equal(ini["flag"][0], np.float32([1, 0]))
    assert np.array_equal(ini["d"][0], np.float32([3.25]))
    assert np.array_equal(ini["u16"][0], np.float32([65535])) and np.array_equal(ini["i16"][0], np.float32([-32768]))


def test_loader_folds_constant_nodes_and_sorts_topologically():
    # Constant nodes become initializers; a file whose nodes are out of order is sorted (producers first)
    raw_nodes = [N("Relu", "late", ["s"], ["y"]), N("Add", "early", ["x", "k"], ["s"]), N("Constant", "k_node", [], ["k"], value_floats=[1.0, 2.0, 3.0])]
    m = model_of(raw_nodes, outputs=["y"], inputs=["x"], shapes={"x": (3,)})
    assert [n.name for n in m.nodes()] == ["early", "late"]
    assert np.array_equal(m.initializers()["k"][0], np.float32([1, 2, 3]))


def test_loader_rejects_malformed_files_with_a_message():
    good = onnx_io.write_onnx(Graph([N("Relu", "r", ["x"], ["y"])], ["x"], ["y"]), {"w": np.float32([1, 2, 3])}, {"x": ((1, 3), np.float32)})
    with pytest.raises(ModelError, match="truncated|runs past|empty"):
        Model.from_bytes(good[: len(good) // 2])
    with pytest.raises(ModelError, match="empty"):
        Model.from_bytes(b"")
    with pytest.raises(ModelError, match="no graph"):
        Model.from_bytes(onnx_io._int(1, 8))
    # raw_data whose length disagrees with the shape
    bad_tensor = onnx_io._int(1, 4) + onnx_io._int(2, 1) + onnx_io._str(8, "w") + onnx_io._len(9, b"\0" * 12)
    bad = onnx_io._int(1, 8) + onnx_io._len(7, onnx_io._len(5, bad_tensor))
    with pytest.raises(ModelError, match="raw bytes"):
        Model.from_bytes(bad)
    # a cycle
    with pytest.raises(ModelError, match="cycle"):
        model_of([N("Relu", "a", ["q"], ["p"]), N("Relu", "b", ["p"], ["q"])], inputs=[])


# ---- fuse_conv_batchnorm (src/optimizer/fusion/conv/tests.rs:11-113) -------------------------------
def _bn_weights(conv_w, scale, bias, mean, var, conv_b=None):
    w = {"conv_w": np.float32(conv_w).reshape(1, 1, 1, 1), "bn_scale": np.float32([scale]), "bn_bias": np.float32([bias]), "bn_mean": np.float32([mean]),
         "bn_var": np.float32([var])}
    if conv_b is not None:
        w["conv_b"] = np.float32([conv_b])
    return w


def test_fuse_conv_batchnorm():
    nodes = [N("Conv", "conv", ["x", "conv_w", "conv_b"], ["conv_out"]),
             N("BatchNormalization", "bn", ["conv_out", "bn_scale", "bn_bias", "bn_mean", "bn_var"], ["bn_out"], epsilon=1e-5)]
    m = model_of(nodes, _bn_weights(1.0, 1.0, 0.0, 0.0, 1.0, conv_b=0.0), outputs=["bn_out"])
    assert m.run_pass("fuse_conv_batchnorm") == 1
    (fused,) = m.nodes()
    assert fused.op == "Conv" and fused.outputs == ["bn_out"] and fused.name == "conv_fused_convbn"
    assert fused.inputs == ["x", "conv_out_fused_weight", "conv_out_fused_bias"]
    ini = m.initializers()
    assert "conv_out_fused_weight" in ini and "conv_out_fused_bias" in ini


def test_fuse_conv_batchnorm_no_conv_bias_numbers():
    # tests.rs:47-80: w = 2, gamma = 3, beta = 0.5, mean = 1, var = 4
    nodes = [N("Conv", "conv", ["x", "conv_w"], ["conv_out"]),
             N("BatchNormalization", "bn", ["conv_out", "bn_scale", "bn_bias", "bn_mean", "bn_var"], ["bn_out"], epsilon=1e-5)]
    m = model_of(nodes, _bn_weights(2.0, 3.0, 0.5, 1.0, 4.0), outputs=["bn_out"])
    assert m.run_pass("fuse_conv_batchnorm") == 1
    ini = m.initializers()
    inv_std = np.float32(1.0) / np.sqrt(np.float32(4.0) + np.float32(1e-5))
    assert abs(ini["conv_out_fused_weight"][0].ravel()[0] - 2.0 * 3.0 * inv_std) < 1e-5
    assert abs(ini["conv_out_fused_bias"][0].ravel()[0] - ((0.0 - 1.0) * 3.0 * inv_std + 0.5)) < 1e-5


def test_fuse_conv_batchnorm_multiple_consumers_is_left_alone():
    nodes = [N("Conv", "conv", ["x", "conv_w", "conv_b"], ["conv_out"]),
             N("BatchNormalization", "bn", ["conv_out", "bn_scale", "bn_bias", "bn_mean", "bn_var"], ["bn_out"], epsilon=1e-5),
             N("Relu", "relu", ["conv_out"], ["relu_out"])]
    m = model_of(nodes, _bn_weights(1.0, 1.0, 0.0, 0.0, 1.0, conv_b=0.0), outputs=["bn_out"])
    assert m.run_pass("fuse_conv_batchnorm") == 0 and len(m.nodes()) == 3


def test_generated_names_never_shadow_existing_tensors():
    # graph_utils.rs:192-210: an initializer already called conv_out_fused_weight pushes the new one to _1
    w = _bn_weights(1.0, 1.0, 0.0, 0.0, 1.0)
    w["conv_out_fused_weight"] = np.float32([9.0])
    nodes = [N("Conv", "", ["x", "conv_w"], ["conv_out"]),
             N("BatchNormalization", "bn", ["conv_out", "bn_scale", "bn_bias", "bn_mean", "bn_var"], ["bn_out"]), N("Relu", "keep", ["conv_out_fused_weight"], ["z"])]
    m = model_of(nodes, w, outputs=["bn_out", "z"])
    assert m.run_pass("fuse_conv_batchnorm") == 1
    assert m.nodes()[0].inputs[1] == "conv_out_fused_weight_1"
    assert m.initializers()["conv_out_fused_weight"][0].ravel()[0] == 9.0


def test_package_batchnorm_fold_agrees_with_the_pass():
    """The graph generators of this package fold BatchNorm themselves; their formula must be the pass's (and the
    reference's, batchnorm.rs:134-144)."""
    rng = np.random.default_rng(3)
    cw = rng.standard_normal((6, 4, 3, 3)).astype(np.float32)
    cb = rng.standard_normal(6).astype(np.float32)
    gamma, beta = rng.uniform(0.5, 1.5, 6).astype(np.float32), rng.standard_normal(6).astype(np.float32)
    mean, var = rng.standard_normal(6).astype(np.float32), rng.uniform(0.5, 1.5, 6).astype(np.float32)
    weights = {"conv_w": cw, "conv_b": cb, "bn_scale": gamma, "bn_bias": beta, "bn_mean": mean, "bn_var": var}
    nodes = [N("Conv", "conv", ["x", "conv_w", "conv_b"], ["conv_out"]),
             N("BatchNormalization", "bn", ["conv_out", "bn_scale", "bn_bias", "bn_mean", "bn_var"], ["bn_out"], epsilon=1e-5)]
    m = model_of(nodes, weights, outputs=["bn_out"])
    assert m.run_pass("fuse_conv_batchnorm") == 1
    ini = m.initializers()
    fw, fb = models.fold_batchnorm(cw, cb, gamma, beta, mean, var, 1e-5)
    assert np.array_equal(ini["conv_out_fused_weight"][0], fw) and np.array_equal(ini["conv_out_fused_bias"][0], fb)


# ---- fuse_conv_relu / relu6 (tests.rs:115-245) -----------------------------------------------------
def test_fuse_conv_relu():
    m = model_of([N("Conv", "conv", ["x", "w", "b"], ["conv_out"]), N("Relu", "relu", ["conv_out"], ["relu_out"])])
    assert m.run_pass("fuse_conv_relu") == 1
    (f,) = m.nodes()
    assert f.op == "Conv" and f.outputs == ["relu_out"] and f.attrs["activation"] == "relu" and f.name == "conv_fused_activation"


def test_fuse_conv_clip_as_relu_and_general_clip():
    m = model_of([N("Conv", "conv", ["x", "w"], ["conv_out"]), N("Clip", "clip", ["conv_out"], ["clip_out"], min=0.0, max=float("inf"))])
    assert m.run_pass("fuse_conv_relu") == 1
    assert m.nodes()[0].attrs["activation"] == "relu" and m.nodes()[0].outputs == ["clip_out"]
    m = model_of([N("Conv", "conv", ["x", "w"], ["conv_out"]), N("Clip", "clip", ["conv_out"], ["clip_out"], min=0.0, max=6.0)])
    assert m.run_pass("fuse_conv_relu") == 1
    a = m.nodes()[0].attrs
    assert a["activation"] == "clip" and a["activation_min"] == 0.0 and a["activation_max"] == 6.0
    # opset-11 spelling: the bounds are constant inputs
    m = model_of([N("Conv", "conv", ["x", "w"], ["conv_out"]), N("Clip", "clip", ["conv_out", "lo", "hi"], ["clip_out"])],
                 {"lo": np.float32([-1.0]), "hi": np.float32([2.5])})
    assert m.run_pass("fuse_conv_relu") == 1
    a = m.nodes()[0].attrs
    assert a["activation"] == "clip" and a["activation_min"] == -1.0 and a["activation_max"] == 2.5
    # an inverted range is not fused
    m = model_of([N("Conv", "conv", ["x", "w"], ["conv_out"]), N("Clip", "clip", ["conv_out"], ["clip_out"], min=3.0, max=1.0)])
    assert m.run_pass("fuse_conv_relu") == 0


def test_fuse_conv_relu_no_fusion_multiple_consumers_or_graph_output():
    m = model_of([N("Conv", "conv", ["x", "w"], ["conv_out"]), N("Relu", "relu", ["conv_out"], ["relu_out"]), N("Add", "add", ["conv_out", "other"], ["add_out"])])
    assert m.run_pass("fuse_conv_relu") == 0 and len(m.nodes()) == 3
    m = model_of([N("Conv", "conv", ["x", "w"], ["conv_out"]), N("Relu", "relu", ["conv_out"], ["y"])], outputs=["y", "conv_out"])
    assert m.run_pass("fuse_conv_relu") == 0
    # a Conv that already carries an activation takes no second one
    m = model_of([N("Conv", "conv", ["x", "w"], ["conv_out"], activation="relu"), N("Relu", "relu", ["conv_out"], ["y"])])
    assert m.run_pass("fuse_conv_relu") == 0


def test_fuse_conv_clip_to_conv_relu6():
    m = model_of([N("Conv", "conv", ["x", "w"], ["conv_out"]), N("Clip", "clip", ["conv_out"], ["clip_out"], min=0.0, max=6.0)])
    assert m.run_pass("fuse_conv_clip_to_conv_relu6") == 1
    (f,) = m.nodes()
    assert f.op == "Conv" and f.attrs["activation"] == "clip" and f.attrs["activation_min"] == 0.0 and f.attrs["activation_max"] == 6.0
    assert f.outputs == ["clip_out"] and f.name == "conv_fused_relu6"
    m = model_of([N("Conv", "conv", ["x", "w"], ["conv_out"]), N("Clip", "clip", ["conv_out"], ["clip_out"], min=0.0, max=1.0)])
    assert m.run_pass("fuse_conv_clip_to_conv_relu6") == 0  # wrong range
    m = model_of([N("Relu", "relu", ["x"], ["relu_out"]), N("Clip", "clip", ["relu_out"], ["clip_out"], min=0.0, max=6.0)])
    assert m.run_pass("fuse_conv_clip_to_conv_relu6") == 0  # not a Conv
    m = model_of([N("Conv", "conv", ["x", "w"], ["conv_out"]), N("Clip", "clip", ["conv_out"], ["clip_out"], min=0.0, max=6.0),
                  N("Add", "add", ["conv_out", "other"], ["add_out"])])
    assert m.run_pass("fuse_conv_clip_to_conv_relu6") == 0  # two consumers


# ---- fuse_conv_add_relu (tests.rs:519-639) -----------------------------------------------------------
def test_fuse_conv_add_relu_input_order_and_attributes():
    for add_inputs in (["conv_out", "residual"], ["residual", "conv_out"]):
        m = model_of([N("Conv", "conv", ["x", "w", "b"], ["conv_out"], pads=[1, 1, 1, 1]), N("Add", "add", add_inputs, ["add_out"]),
                      N("Relu", "relu", ["add_out"], ["relu_out"])])
        assert m.run_pass("fuse_conv_add_relu") == 2
        (f,) = m.nodes()
        assert f.op == "ConvAddRelu" and f.inputs == ["x", "w", "b", "residual"] and f.outputs == ["relu_out"]
        assert f.attrs["fused_ops"] == "Add,Relu" and f.attrs["pads"] == [1, 1, 1, 1] and f.name == "conv_fused_conv_add_relu"
    m = model_of([N("Conv", "conv", ["x", "w"], ["conv_out"]), N("Add", "add", ["conv_out", "residual"], ["add_out"]), N("Relu", "relu", ["add_out"], ["relu_out"])])
    assert m.run_pass("fuse_conv_add_relu") == 2
    assert m.nodes()[0].inputs[2] == "" and m.nodes()[0].inputs[3] == "residual"  # the bias slot stays, empty


def test_fuse_conv_add_relu_declines():
    base = [N("Conv", "conv", ["x", "w", "b"], ["conv_out"]), N("Add", "add", ["conv_out", "residual"], ["add_out"]), N("Relu", "relu", ["add_out"], ["relu_out"])]
    m = model_of(base + [N("Relu", "extra", ["conv_out"], ["extra_out"])])
    assert m.run_pass("fuse_conv_add_relu") == 0 and m.nodes()[0].op == "Conv"
    m = model_of(base + [N("Sigmoid", "extra", ["add_out"], ["extra_out"])])
    assert m.run_pass("fuse_conv_add_relu") == 0
    m = model_of(base[:2] + [N("Sigmoid", "sigmoid", ["add_out"], ["sig_out"])])
    assert m.run_pass("fuse_conv_add_relu") == 0


def test_fuse_conv_add_relu_keeps_the_graph_sorted_when_the_residual_comes_later():
    # main-branch conv first, shortcut conv second (a ResNet projection block): the fused node needs the shortcut
    nodes = [N("Conv", "main", ["x", "w1"], ["m"]), N("Conv", "short", ["x", "w2"], ["s"]), N("Add", "add", ["m", "s"], ["a"]), N("Relu", "relu", ["a"], ["y"])]
    m = model_of(nodes, outputs=["y"])
    assert m.run_pass("fuse_conv_add_relu") == 2
    names = [n.name for n in m.nodes()]
    assert names == ["short", "main_fused_conv_add_relu"]


# ---- fuse_matmul_add, SiLU ---------------------------------------------------------------------------
def test_fuse_matmul_add_to_gemm():
    w = {"b": np.zeros((8, 5), np.float32), "bias": np.zeros(5, np.float32)}
    m = model_of([N("MatMul", "mm", ["a", "b"], ["p"]), N("Add", "add", ["p", "bias"], ["y"])], w, outputs=["y"], shapes={"a": (3, 8)})
    assert m.run_pass("fuse_matmul_add") == 1
    (f,) = m.nodes()
    assert f.op == "Gemm" and f.inputs == ["a", "b", "bias"] and f.outputs == ["y"] and f.name == "mm_fused_gemm"
    assert f.attrs == {"alpha": 1.0, "beta": 1.0, "transA": 0, "transB": 0}
    # a rank-3 A is not a Gemm
    m = model_of([N("MatMul", "mm", ["a", "b"], ["p"]), N("Add", "add", ["p", "bias"], ["y"])], w, outputs=["y"], shapes={"a": (2, 3, 8)})
    assert m.run_pass("fuse_matmul_add") == 0
    # a rank-2 bias is not folded
    w2 = dict(w, bias=np.zeros((1, 5), np.float32))
    m = model_of([N("MatMul", "mm", ["a", "b"], ["p"]), N("Add", "add", ["p", "bias"], ["y"])], w2, outputs=["y"], shapes={"a": (3, 8)})
    assert m.run_pass("fuse_matmul_add") == 0


def test_fuse_mul_sigmoid_to_silu():
    for mul_inputs in (["x", "s"], ["s", "x"]):
        m = model_of([N("Sigmoid", "sig", ["x"], ["s"]), N("Mul", "mul", mul_inputs, ["y"])], outputs=["y"])
        assert m.run_pass("fuse_mul_sigmoid_to_silu") == 1
        (f,) = m.nodes()
        assert f.op == "SiLU" and f.inputs == ["x"] and f.outputs == ["y"] and f.name == "mul_fused_silu"
    m = model_of([N("Sigmoid", "sig", ["x"], ["s"]), N("Mul", "mul", ["z", "s"], ["y"])], outputs=["y"])
    assert m.run_pass("fuse_mul_sigmoid_to_silu") == 0  # the other operand is not the sigmoid's input


# ---- fuse_instance_norm (src/optimizer/fusion/instance_norm_tests.rs) -------------------------------
def chain(pow_square=False, reciprocal=True, swap_mul=False, swap_eps=False, axes=(2, 3), keepdims=1, eps=1e-8, axes_as_input=False, rank4=True,
          extra=(), sub_reversed=False, mean_of="X", square_other=False, exponent=2.0, numerator=1.0, eps_constant=True):
    """make_chain (instance_norm_tests.rs:49-124): X -> ... -> norm."""
    w = {"two": np.float32([exponent]), "one": np.float32([numerator])}
    if eps_constant:
        w["eps"] = np.float32([eps])

    def rm(name, src, dst):
        if axes_as_input:
            w["axes"] = np.int64(list(axes))
            return N("ReduceMean", name, [src, "axes"], [dst], keepdims=keepdims)
        return N("ReduceMean", name, [src], [dst], axes=list(axes), keepdims=keepdims)

    nodes = [rm("rm_mean", mean_of, "mean"), N("Sub", "sub", ["mean", "X"] if sub_reversed else ["X", "mean"], ["diff"])]
    if pow_square:
        nodes.append(N("Pow", "pow", ["diff", "two"], ["sq"]))
    else:
        nodes.append(N("Mul", "square", ["diff", "other" if square_other else "diff"], ["sq"]))
    nodes.append(rm("rm_var", "sq", "var"))
    nodes.append(N("Add", "add_eps", ["eps", "var"] if swap_eps else ["var", "eps"], ["vare"]))
    nodes.append(N("Sqrt", "sqrt", ["vare"], ["std"]))
    if reciprocal is None:
        nodes.append(N("Div", "norm_div", ["diff", "std"], ["norm"]))
    else:
        nodes.append(N("Reciprocal", "recip", ["std"], ["rstd"]) if reciprocal else N("Div", "recip", ["one", "std"], ["rstd"]))
        nodes.append(N("Mul", "norm_mul", ["rstd", "diff"] if swap_mul else ["diff", "rstd"], ["norm"]))
    nodes.extend(extra)
    shape = (2, 3, 4, 5) if rank4 else (2, 3, 7)
    shapes = {n: shape for n in ("X", "other", "Y")}
    inputs = ["X"] + (["other"] if square_other or mean_of == "other" else []) + ([] if eps_constant else ["eps"])
    return nodes, w, shapes, inputs


def fuse(spec_kwargs, outputs=("norm",)):
    nodes, w, shapes, inputs = chain(**spec_kwargs)
    m = model_of(nodes, w, outputs=list(outputs), inputs=inputs, shapes=shapes)
    removed = m.run_pass("fuse_instance_norm")
    return removed, m.nodes()


@pytest.mark.parametrize("spec", [dict(), dict(reciprocal=False), dict(reciprocal=None), dict(pow_square=True), dict(swap_mul=True, swap_eps=True),
                                  dict(axes=(-2, -1)), dict(axes_as_input=True), dict(eps=1.0)],
                         ids=["reciprocal + mul-self", "div-one reciprocal", "direct div", "pow square", "commuted operands", "negative axes",
                              "opset-18 axes input", "large epsilon"])
def test_instance_norm_chain_variants_fuse(spec):
    removed, nodes = fuse(spec)
    assert len(nodes) == 1 and nodes[0].op == "OxiInstanceNorm"
    assert nodes[0].inputs == ["X"] and nodes[0].outputs == ["norm"]
    assert nodes[0].attrs["epsilon"] == pytest.approx(spec.get("eps", 1e-8))
    assert removed == (6 if spec.get("reciprocal", True) is None else 7)
    assert nodes[0].name == "rm_mean_fused_instancenorm"  # the fused node takes the earliest chain node's place


def test_instance_norm_rank_3_fuses_over_the_single_spatial_axis():
    removed, nodes = fuse(dict(axes=(2,), rank4=False))
    assert len(nodes) == 1 and nodes[0].op == "OxiInstanceNorm"


def test_instance_norm_leaves_the_runtime_affine_nodes_outside():
    extra = [N("Mul", "scale_mul", ["scale", "norm"], ["scaled"]), N("Add", "shift_add", ["scaled", "shift"], ["biased"])]
    nodes, w, shapes, inputs = chain(extra=extra)
    m = model_of(nodes, w, outputs=["biased"], inputs=inputs + ["scale", "shift"], shapes=shapes)
    assert m.run_pass("fuse_instance_norm") == 7
    assert [n.op for n in m.nodes()] == ["OxiInstanceNorm", "Mul", "Add"]


@pytest.mark.parametrize("spec,outputs", [
    (dict(axes=(1, 2, 3)), ("norm",)),                                   # the reduction includes the channel axis
    (dict(axes=(3,)), ("norm",)),                                        # partial spatial reduction
    (dict(keepdims=0), ("norm",)),
    (dict(extra=(N("Relu", "spy", ["std"], ["spied"]),)), ("norm", "spied")),   # an intermediate has a second consumer
    (dict(), ("norm", "var")),                                           # an intermediate is a graph output
    (dict(square_other=True), ("norm",)),                                # the square multiplies two different tensors
    (dict(pow_square=True, exponent=3.0), ("norm",)),
    (dict(reciprocal=False, numerator=2.0), ("norm",)),                  # Div(2, std) is not a reciprocal
    (dict(eps_constant=False), ("norm",)),                               # epsilon is a run-time tensor
    (dict(eps=-1e-3), ("norm",)),
    (dict(sub_reversed=True), ("norm",)),                                # mean - X
    (dict(mean_of="other"), ("norm",)),                                  # the mean is taken of another tensor
], ids=["channel axis reduced", "partial reduction", "keepdims 0", "extra consumer", "graph output inside", "square of two tensors", "exponent 3",
        "numerator 2", "run-time epsilon", "negative epsilon", "reversed subtraction", "mean of another tensor"])
def test_instance_norm_chain_declines(spec, outputs):
    removed, nodes = fuse(spec, outputs)
    assert removed == 0 and all(n.op != "OxiInstanceNorm" for n in nodes)


def test_instance_norm_declines_when_rank_is_unknown():
    nodes, w, _, inputs = chain()
    # the input carries no shape: nothing tells the matcher that axes [2, 3] are all the spatial axes
    g = Graph(nodes=nodes, input_names=[], output_names=["norm"])
    m = Model.from_bytes(onnx_io.write_onnx(g, w, {}, outputs={"norm": ((), np.float32)}))
    assert m.run_pass("fuse_instance_norm") == 0


def test_two_independent_chains_fuse_separately():
    n1, w, shapes, _ = chain()

    def rename(node, suffix):
        keep = {"eps", "one", "two", "axes"}
        return Node(node.op, node.name + suffix, [i if i in keep else i + suffix for i in node.inputs], [o + suffix for o in node.outputs], dict(node.attrs))

    nodes = [rename(n, "_a") for n in n1] + [rename(n, "_b") for n in n1]
    shapes = {"X_a": (2, 3, 4, 5), "X_b": (2, 3, 4, 5)}
    m = model_of(nodes, w, outputs=["norm_a", "norm_b"], inputs=["X_a", "X_b"], shapes=shapes)
    assert m.run_pass("fuse_instance_norm") == 14
    assert [n.op for n in m.nodes()] == ["OxiInstanceNorm", "OxiInstanceNorm"]


# ---- the whole pipeline ---------------------------------------------------------------------------------
def test_optimize_runs_the_passes_in_the_reference_order_on_a_residual_block():
    rng = np.random.default_rng(1)
    c = 8
    w = {}
    nodes = []

    def conv_bn(name, src, relu):
        w[f"{name}_w"] = rng.standard_normal((c, c, 3, 3)).astype(np.float32)
        for k, v in (("s", rng.uniform(0.5, 1.5, c)), ("b", rng.standard_normal(c)), ("m", rng.standard_normal(c)), ("v", rng.uniform(0.5, 1.5, c))):
            w[f"{name}_{k}"] = v.astype(np.float32)
        nodes.append(N("Conv", name, [src, f"{name}_w"], [f"{name}_c"], pads=[1, 1, 1, 1]))
        nodes.append(N("BatchNormalization", f"{name}_bn", [f"{name}_c", f"{name}_s", f"{name}_b", f"{name}_m", f"{name}_v"], [f"{name}_n"], epsilon=1e-5))
        if relu:
            nodes.append(N("Relu", f"{name}_relu", [f"{name}_n"], [f"{name}_r"]))
            return f"{name}_r"
        return f"{name}_n"

    a = conv_bn("c1", "x", True)
    b = conv_bn("c2", a, False)
    nodes.append(N("Add", "add", [b, "x"], ["sum"]))
    nodes.append(N("Relu", "out_relu", ["sum"], ["y"]))
    m = model_of(nodes, w, outputs=["y"], inputs=["x"], shapes={"x": (1, c, 6, 6)})
    assert m.optimize(1) == 5
    got = m.nodes()
    assert [n.op for n in got] == ["Conv", "ConvAddRelu"]
    assert got[0].attrs["activation"] == "relu" and got[0].name == "c1_fused_convbn_fused_activation"
    assert got[1].inputs[3] == "x" and got[1].inputs[1] == "c2_c_fused_weight" and got[1].inputs[2] == "c2_c_fused_bias"


def test_optimised_network_has_the_value_of_the_unfused_one():
    """Every pass at once on a small network (BN folds, Conv+Relu, Conv+Add+Relu, SiLU, Conv+Clip, the
    normalisation chain, MatMul+Add): the CPU oracle run over the optimised graph agrees with the unfused graph."""
    from test_gpu_onnx import oracle_unfused, residual_net
    rng = np.random.default_rng(11)
    graph, weights = residual_net(rng)
    m = Model.from_bytes(onnx_io.write_onnx(graph, weights, {"x": (("N", 3, 16, 16), np.float32)}))
    assert m.optimize(1) == 16
    fused_graph, fused_weights = m.to_graph()
    assert [n.op for n in fused_graph.nodes] == ["Conv", "Conv", "ConvAddRelu", "Conv", "SiLU", "Conv", "OxiInstanceNorm", "Mul", "Add",
                                                 "GlobalAveragePool", "Flatten", "Gemm"]
    x = rng.standard_normal((2, 3, 16, 16)).astype(np.float32)
    want = oracle_unfused(graph, weights, {"x": x})
    got = oracle_unfused(fused_graph, fused_weights, {"x": x})
    for name in want:
        assert np.max(np.abs(got[name] - want[name])) <= 2e-5 * np.max(np.abs(want[name])), name
