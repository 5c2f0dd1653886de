"""ONNX files end to end on the B200: write a model, load it with Session.from_file (the loader and the fusion
passes run in the library), run it, and compare with the CPU oracle run over the UNFUSED graph -- so a pass that
changed the network's value, a fused node the planner misreads, or an epilogue that differs from the separate
operators all show up.  Plus per-node parity of the fused-node forms the passes emit: ConvAddRelu, Conv with a
SiLU or PRelu epilogue.

Float tolerance: |a-b| <= 2e-3 * (max|b| + |b|), the TF32 tolerance of the path; the quantised model is bit-exact.
"""
import numpy as np
import pytest

import oracle
from oxionnx_b200 import onnx_io, session as S
from oxionnx_b200.graph import Graph, Node

pytestmark = pytest.mark.gpu

RTOL = 2e-3


def close(got, want, what=""):
    want = np.asarray(want, np.float32)
    bound = RTOL * float(np.max(np.abs(want))) + RTOL * np.abs(want)
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert got.shape == want.shape, f"{what}: {got.shape} vs {want.shape}"
    assert np.all(err <= bound), f"{what}: max err {err.max()} over bound, {int(np.sum(err > bound))} lanes off"


def N(op, name, ins, outs, **attrs):
    return Node(op=op, name=name, inputs=list(ins), outputs=list(outs), attrs=attrs)


def residual_net(rng, c=32, classes=10):
    """stem conv + BN + relu; a residual block (conv-BN-relu, conv-BN, add, relu); x * sigmoid(x) after a 1x1
    conv; the spelled-out instance normalisation; global pool, flatten, MatMul + Add head."""
    w, nodes = {}, []

    def conv_bn(name, src, cin, cout, k, pad, stride=1):
        w[f"{name}_w"] = (rng.standard_normal((cout, cin, k, k)) * np.sqrt(2.0 / (cin * k * k))).astype(np.float32)
        w[f"{name}_s"] = rng.uniform(0.5, 1.5, cout).astype(np.float32)
        w[f"{name}_b"] = (rng.standard_normal(cout) * 0.1).astype(np.float32)
        w[f"{name}_m"] = (rng.standard_normal(cout) * 0.1).astype(np.float32)
        w[f"{name}_v"] = rng.uniform(0.5, 1.5, cout).astype(np.float32)
        nodes.append(N("Conv", name, [src, f"{name}_w"], [f"{name}_c"], pads=[pad] * 4, strides=[stride, stride], kernel_shape=[k, k]))
        nodes.append(N("BatchNormalization", f"{name}_bn", [f"{name}_c", f"{name}_s", f"{name}_b", f"{name}_m", f"{name}_v"], [f"{name}_n"], epsilon=1e-5))
        return f"{name}_n"

    s = conv_bn("stem", "x", 3, c, 3, 1)
    nodes.append(N("Relu", "stem_relu", [s], ["stem_r"]))
    a = conv_bn("b1", "stem_r", c, c, 3, 1)
    nodes.append(N("Relu", "b1_relu", [a], ["b1_r"]))
    b = conv_bn("b2", "b1_r", c, c, 3, 1)
    nodes.append(N("Add", "join", [b, "stem_r"], ["sum"]))
    nodes.append(N("Relu", "join_relu", ["sum"], ["blk"]))
    # 1x1 conv with bias, then x * sigmoid(x)
    w["pw_w"] = (rng.standard_normal((c, c, 1, 1)) * np.sqrt(1.0 / c)).astype(np.float32)
    w["pw_b"] = (rng.standard_normal(c) * 0.1).astype(np.float32)
    nodes.append(N("Conv", "pw", ["blk", "pw_w", "pw_b"], ["pw_o"]))
    nodes.append(N("Sigmoid", "sig", ["pw_o"], ["sig_o"]))
    nodes.append(N("Mul", "swish", ["pw_o", "sig_o"], ["sw"]))
    # Conv + Clip(0, 6)
    w["c6_w"] = (rng.standard_normal((c, c, 3, 3)) * np.sqrt(2.0 / (c * 9))).astype(np.float32)
    nodes.append(N("Conv", "c6", ["sw", "c6_w"], ["c6_o"], pads=[1, 1, 1, 1]))
    nodes.append(N("Clip", "c6_clip", ["c6_o"], ["c6_r"], min=0.0, max=6.0))
    # instance normalisation spelled as primitive operators, with a runtime scale and shift after it
    w["eps"] = np.float32([1e-5])
    w["gamma"] = rng.uniform(0.5, 1.5, (1, c, 1, 1)).astype(np.float32)
    w["beta"] = (rng.standard_normal((1, c, 1, 1)) * 0.1).astype(np.float32)
    nodes += [N("ReduceMean", "in_mean", ["c6_r"], ["mu"], axes=[2, 3], keepdims=1), N("Sub", "in_sub", ["c6_r", "mu"], ["d"]),
              N("Mul", "in_sq", ["d", "d"], ["d2"]), N("ReduceMean", "in_var", ["d2"], ["var"], axes=[2, 3], keepdims=1),
              N("Add", "in_eps", ["var", "eps"], ["ve"]), N("Sqrt", "in_sqrt", ["ve"], ["sd"]), N("Div", "in_div", ["d", "sd"], ["nrm"]),
              N("Mul", "in_scale", ["nrm", "gamma"], ["scaled"]), N("Add", "in_shift", ["scaled", "beta"], ["inorm"])]
    nodes.append(N("GlobalAveragePool", "gap", ["inorm"], ["pooled"]))
    nodes.append(N("Flatten", "flat", ["pooled"], ["feat"], axis=1))
    w["fc_w"] = (rng.standard_normal((c, classes)) * np.sqrt(1.0 / c)).astype(np.float32)
    w["fc_b"] = (rng.standard_normal(classes) * 0.1).astype(np.float32)
    nodes.append(N("MatMul", "fc", ["feat", "fc_w"], ["fc_o"]))
    nodes.append(N("Add", "fc_add", ["fc_o", "fc_b"], ["logits"]))
    return Graph(nodes, ["x"], ["logits", "inorm"]), w


def oracle_unfused(graph, weights, feeds):
    """The oracle has no ReduceMean / Sqrt / Clip operators of its own (they are not on the path); the unfused
    reference value of those few nodes is computed here in f32 numpy, everything else by the oracle."""
    env = dict(weights)
    env.update(feeds)
    f32 = np.float32
    for n in graph.nodes:
        ins = [env[i] if i else None for i in n.inputs]
        if n.op == "ReduceMean":
            x = ins[0].astype(np.float64)
            env[n.outputs[0]] = x.mean(axis=tuple(n.attrs["axes"]), keepdims=bool(n.attrs.get("keepdims", 1))).astype(f32)
        elif n.op == "Sqrt":
            env[n.outputs[0]] = np.sqrt(ins[0]).astype(f32)
        elif n.op == "Clip":
            env[n.outputs[0]] = np.clip(ins[0], f32(n.attrs["min"]), f32(n.attrs["max"])).astype(f32)
        else:
            outs = oracle.run_node(n.op, ins, n.attrs, n_outputs=len(n.outputs))
            for name, val in zip(n.outputs, outs):
                env[name] = val
    return {o: env[o] for o in graph.output_names}


def test_model_file_loads_fuses_and_runs_like_the_unfused_graph(tmp_path):
    rng = np.random.default_rng(11)
    graph, weights = residual_net(rng)
    path = str(tmp_path / "residual.onnx")
    onnx_io.write_onnx(graph, weights, {"x": (("N", 3, 16, 16), np.float32)}, path, outputs={"logits": (("N", 10), np.float32), "inorm": (("N", 32, 16, 16), np.float32)})
    x = rng.standard_normal((4, 3, 16, 16)).astype(np.float32)
    want = oracle_unfused(graph, weights, {"x": x})

    sess = S.Session.from_file(path)
    ops = [n.op for n in sess.graph.nodes]
    # every pattern of the file is fused: 3 BN folds, 2 Conv+Relu, Conv+Add+Relu, SiLU, Conv+Clip(0,6), the chain, MatMul+Add
    assert ops == ["Conv", "Conv", "ConvAddRelu", "Conv", "SiLU", "Conv", "OxiInstanceNorm", "Mul", "Add", "GlobalAveragePool", "Flatten", "Gemm"], ops
    assert sess.graph.nodes[5].attrs["activation"] == "clip"
    got = sess.run({"x": x})
    close(got["inorm"], want["inorm"], "instance-normalised feature map")
    close(got["logits"], want["logits"], "logits")
    # a second batch size replans from the symbolic dimension
    x2 = rng.standard_normal((2, 3, 16, 16)).astype(np.float32)
    got2 = sess.run({"x": x2})
    close(got2["logits"], oracle_unfused(graph, weights, {"x": x2})["logits"], "logits at batch 2")
    sess.close()

    # optimisation off: the file's own nodes run (BatchNormalization is not on this provider's list -> typed refusal)
    plain = S.Session.from_file(path, optimization_level=0)
    assert [n.op for n in plain.graph.nodes] == [n.op for n in graph.nodes]
    with pytest.raises(S.Declined, match="BatchNormalization"):
        plain.run({"x": x})
    plain.close()


def test_quantised_model_file_keeps_typed_initializers(tmp_path):
    """A QLinearConv whose zero points are uint8 / int8 tensors in the file: the declared types choose the
    saturation range (oxionnx-ops quant_ops run_typed), and the result is the oracle's bit for bit."""
    rng = np.random.default_rng(5)
    c_in, c_out = 16, 32
    weights = {"x_scale": np.float32([0.02]), "x_zp": np.uint8([128]), "w": rng.integers(-127, 128, (c_out, c_in, 3, 3)).astype(np.int8),
               "w_scale": rng.uniform(0.001, 0.01, c_out).astype(np.float32), "w_zp": np.zeros(c_out, np.int8), "y_scale": np.float32([0.05]),
               "y_zp": np.uint8([3]), "bias": rng.integers(-500, 500, c_out).astype(np.int32)}
    nodes = [N("QuantizeLinear", "q", ["x", "x_scale", "x_zp"], ["xq"]),
             N("QLinearConv", "qc", ["xq", "x_scale", "x_zp", "w", "w_scale", "w_zp", "y_scale", "y_zp", "bias"], ["yq"], pads=[1, 1, 1, 1]),
             N("DequantizeLinear", "dq", ["yq", "y_scale", "y_zp"], ["y"])]
    graph = Graph(nodes, ["x"], ["y", "yq"])
    path = str(tmp_path / "q.onnx")
    onnx_io.write_onnx(graph, weights, {"x": ((2, c_in, 12, 12), np.float32)}, path)
    x = (rng.standard_normal((2, c_in, 12, 12)) * 1.5).astype(np.float32)
    sess = S.Session.from_file(path)
    got = sess.run({"x": x})
    _, typed = sess._model.to_graph()
    assert typed["x_zp"].dtype == np.uint8 and typed["w"].dtype == np.int8
    want = oracle.run_graph(graph, weights, {"x": x})
    assert np.array_equal(got["yq"], want["yq"]) and np.array_equal(got["y"], want["y"])
    assert got["yq"].min() >= 0 and got["yq"].max() <= 255
    sess.close()


# ---- the fused-node forms, node by node --------------------------------------------------------------
@pytest.fixture(scope="module")
def ctx():
    c = S.CudaContext(0)
    yield c
    c.close()


def dispatch(ctx, op, inputs, attrs):
    names = [f"in{i}" if x is not None else "" for i, x in enumerate(inputs)]
    node = Node(op=op, name="n0", inputs=names, outputs=["out0"], attrs=dict(attrs))
    out = S.try_cuda_dispatch(node, {}, {n: x for n, x in zip(names, inputs) if n}, ctx)
    assert out is not None, ctx.last_error()
    return out[0]


@pytest.mark.parametrize("shape", [(2, 64, 14, 14, 64, 3, 1, 1), (1, 32, 9, 9, 48, 1, 1, 0), (2, 3, 17, 17, 8, 3, 2, 1), (1, 256, 14, 14, 256, 3, 1, 1)],
                         ids=["3x3 64->64", "1x1 32->48", "3-channel stride 2 (direct kernel)", "3x3 256->256"])
@pytest.mark.parametrize("bias", [True, False], ids=["bias", "no bias"])
def test_conv_add_relu_node(ctx, shape, bias):
    n, c, h, w_, oc, k, stride, pad = shape
    rng = np.random.default_rng(n * 1000 + c + oc)
    x = rng.standard_normal((n, c, h, w_)).astype(np.float32)
    wt = (rng.standard_normal((oc, c, k, k)) / np.sqrt(c * k * k)).astype(np.float32)
    b = rng.standard_normal(oc).astype(np.float32) if bias else None
    attrs = dict(pads=[pad] * 4, strides=[stride, stride], fused_ops="Add,Relu")
    conv = oracle.run_node("Conv", [x, wt, b], dict(pads=[pad] * 4, strides=[stride, stride]))[0]
    res = rng.standard_normal(conv.shape).astype(np.float32)
    want = oracle.run_node("ConvAddRelu", [x, wt, b, res], attrs)[0]
    got = dispatch(ctx, "ConvAddRelu", [x, wt, b, res], attrs)
    close(got, want, "ConvAddRelu")
    assert got.min() >= 0.0 and np.array_equal(got == 0, want == 0) or np.mean((got == 0) != (want == 0)) < 1e-3


def test_conv_add_relu_rejects_a_residual_of_the_wrong_shape(ctx):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((1, 8, 6, 6)).astype(np.float32)
    wt = rng.standard_normal((8, 8, 3, 3)).astype(np.float32)
    res = rng.standard_normal((1, 8, 5, 5)).astype(np.float32)
    node = Node(op="ConvAddRelu", name="n0", inputs=["a", "b", "", "r"], outputs=["o"], attrs=dict(pads=[1, 1, 1, 1], fused_ops="Add,Relu"))
    assert S.try_cuda_dispatch(node, {}, {"a": x, "b": wt, "r": res}, ctx) is None
    assert "residual" in ctx.last_error()


@pytest.mark.parametrize("op", ["Silu", "SiLU"])
def test_silu_node(ctx, op):
    rng = np.random.default_rng(8)
    x = (rng.standard_normal((3, 5, 7, 11)) * 4).astype(np.float32)
    got = dispatch(ctx, op, [x], {})
    want = oracle.run_node("Silu", [x], {})[0]
    assert np.all(np.abs(got - want) <= 2e-6 * (1 + np.abs(want)))


def _session_for(graph, weights, shapes):
    return S.SessionBuilder().with_input_shapes(shapes).build_from_graph(graph, weights)


@pytest.mark.parametrize("kind", ["silu", "prelu"])
@pytest.mark.parametrize("geom", [(2, 64, 14, 14, 128, 3, 1), (2, 96, 10, 10, 64, 1, 0)], ids=["3x3 64->128", "1x1 96->64"])
def test_conv_followed_by_silu_or_prelu_runs_in_the_epilogue(kind, geom):
    n, c, h, w_, oc, k, pad = geom
    rng = np.random.default_rng(c + oc)
    x = rng.standard_normal((n, c, h, w_)).astype(np.float32)
    weights = {"w": (rng.standard_normal((oc, c, k, k)) / np.sqrt(c * k * k)).astype(np.float32), "b": rng.standard_normal(oc).astype(np.float32)}
    nodes = [N("Conv", "conv", ["x", "w", "b"], ["c"], pads=[pad] * 4)]
    if kind == "silu":
        nodes.append(N("SiLU", "act", ["c"], ["y"]))
    else:
        weights["slope"] = np.float32([0.17])
        nodes.append(N("PRelu", "act", ["c", "slope"], ["y"]))
    graph = Graph(nodes, ["x"], ["y"])
    want = oracle.run_graph(graph, weights, {"x": x})["y"]
    sess = _session_for(graph, weights, {"x": x.shape})
    got = sess.run({"x": x})["y"]
    close(got, want, f"Conv + {kind}")
    # one contraction launch carries the activation: no separate elementwise step in the plan
    # layout conversions at the graph's edges and the TF32-rounded copy of the graph input aside
    steps = [st for st in sess.steps() if not st["kernel"].startswith(("convert_", "round_to_tf32"))]
    assert [st["op"] for st in steps] == ["Conv"], steps
    sess.close()


def test_model_with_float16_weights_runs_on_the_f16_kind(tmp_path):
    """A model whose convolution weights are FLOAT16 initializers: the declared type survives loading beside the
    f32 lanes and selects 16-bit operands (f32 accumulation) for that contraction, without any context option."""
    rng = np.random.default_rng(21)
    c, oc = 64, 96
    w16 = (rng.standard_normal((oc, c, 3, 3)) / np.sqrt(c * 9)).astype(np.float16)
    weights = {"w": w16, "b": rng.standard_normal(oc).astype(np.float32)}
    graph = Graph([N("Conv", "conv", ["x", "w", "b"], ["y"], pads=[1, 1, 1, 1], activation="relu")], ["x"], ["y"])
    path = str(tmp_path / "half.onnx")
    onnx_io.write_onnx(graph, weights, {"x": ((2, c, 12, 12), np.float32)}, path)
    x = rng.standard_normal((2, c, 12, 12)).astype(np.float32)
    want = oracle.run_node("Conv", [x, w16.astype(np.float32), weights["b"]], dict(pads=[1, 1, 1, 1], activation="relu"))[0]
    sess = S.Session.from_file(path)
    got = sess.run({"x": x})["y"]
    kernels = [st["kernel"] for st in sess.steps()]
    sess.close()
    assert any(k.startswith("umma_f16") for k in kernels), kernels
    rms = float(np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    assert np.all(np.abs(got.astype(np.float64) - want) <= 1e-2 * np.abs(want) + 1e-2 * rms)
