"""Device I/O binding and typed 8-bit feeds of the planned session (the reference's IoBinding and
run_with_binding, root crate src/io_binding.rs:42-58 and src/session/run/entry.rs:109-139, carried over to device
memory; declared input types as in TensorInfo, oxionnx-core src/graph.rs:862).

Checked here, through the C ABI: a run whose input and output are bound to device buffers moves no byte across
PCIe (the context's upload / download counters stand still) and computes what the CPU oracle computes; a graph
input declared u8 is fed with a quarter of the bytes and gives the lanes of the f32-lane form bit for bit.
"""
import ctypes

import numpy as np
import pytest

import oracle
from oxionnx_b200 import models
from oxionnx_b200.graph import Graph, Node
from oxionnx_b200.session import OnnxError, Session

pytestmark = pytest.mark.gpu


def _conv_graph(c=32):
    rng = np.random.default_rng(11)
    weights = {"w": (rng.standard_normal((c, c, 3, 3)) / np.sqrt(9 * c)).astype(np.float32), "b": (rng.standard_normal(c) * 0.1).astype(np.float32)}
    graph = Graph(nodes=[Node("Conv", "conv", ["x", "w", "b"], ["y"], {"pads": [1, 1, 1, 1], "activation": "relu"})], input_names=["x"], output_names=["y"])
    return graph, weights


def _close(got, want):
    bound = 2e-3 * np.abs(want) + 2e-3 * float(np.abs(want).max())
    return bool(np.all(np.abs(got - want) <= bound))


def test_second_run_reads_the_first_runs_output_on_the_device_with_no_host_traffic():
    import torch

    graph, weights = _conv_graph()
    x = np.random.default_rng(12).standard_normal((2, 32, 12, 12)).astype(np.float32)
    sess = Session.builder().build_from_graph(graph, weights)
    stage1 = torch.zeros(x.size, dtype=torch.float32, device="cuda")
    stage2 = torch.zeros(x.size, dtype=torch.float32, device="cuda")
    # run 1: host feed in, output also written to a caller-owned device buffer
    sess.ensure_planned({"x": x})
    sess.bind_output_device("y", stage1.data_ptr(), x.size)
    y1 = sess.run_with_binding({"x": x})["y"]
    oracle.set_threads(4)
    want1, = oracle.run_node("Conv", [x, weights["w"], weights["b"]], graph.nodes[0].attrs)
    assert _close(y1, want1)
    torch.cuda.synchronize()
    assert np.array_equal(stage1.cpu().numpy().reshape(x.shape), y1), "the bound output buffer holds the run's f32 lanes"
    # run 2: that buffer is the input, another device buffer the output; nothing crosses PCIe
    sess.bind_input_device("x", stage1.data_ptr(), np.float32, x.size)
    sess.bind_output_device("y", stage2.data_ptr(), x.size)
    before = sess.cuda_cache_counters()
    assert sess.run_with_binding(fetch=False) is None
    after = sess.cuda_cache_counters()
    for key in ("uploads", "upload_bytes", "downloads", "download_bytes"):
        assert after[key] == before[key], f"{key} moved from {before[key]} to {after[key]} in a fully bound run"
    assert after["kernel_launches"] > before["kernel_launches"]
    torch.cuda.synchronize()
    y2 = stage2.cpu().numpy().reshape(x.shape)
    want2, = oracle.run_node("Conv", [want1, weights["w"], weights["b"]], graph.nodes[0].attrs)
    assert _close(y2, want2)
    # the library-owned output buffer holds the same lanes and keeps its address
    ptr, count = sess.output_device_ptr("y")
    assert ptr != 0 and count == x.size
    assert sess.output_device_ptr("y")[0] == ptr
    # clearing the bindings brings the host path back
    sess.clear_bindings()
    assert _close(sess.run({"x": x})["y"], want1)
    sess.close()


def test_binding_rejects_what_does_not_match_the_plan():
    import torch

    graph, weights = _conv_graph()
    x = np.zeros((1, 32, 8, 8), np.float32)
    sess = Session.builder().build_from_graph(graph, weights)
    sess.ensure_planned({"x": x})
    buf = torch.zeros(x.size, dtype=torch.float32, device="cuda")
    with pytest.raises(OnnxError, match="not an input"):
        sess.bind_input_device("nope", buf.data_ptr(), np.float32, x.size)
    with pytest.raises(OnnxError, match="elements"):
        sess.bind_input_device("x", buf.data_ptr(), np.float32, x.size - 1)
    with pytest.raises(OnnxError, match="planned as f32"):
        sess.bind_input_device("x", buf.data_ptr(), np.uint8, x.size)
    with pytest.raises(OnnxError, match="aligned"):
        sess.bind_input_device("x", buf.data_ptr() + 4, np.float32, x.size)
    with pytest.raises(OnnxError, match="holds"):
        sess.bind_output_device("y", buf.data_ptr(), x.size - 1)
    with pytest.raises(OnnxError, match="neither bound nor fed"):
        sess.run_with_binding()
    sess.close()


def test_u8_declared_input_is_fed_as_bytes_and_gives_the_same_lanes():
    """The reduced-width QLinearConv ResNet in its two spellings: f32 image -> QuantizeLinear -> ..., and the
    already quantised image declared and fed as u8.  Same logits bit for bit, a quarter of the upload."""
    kw = dict(batch=2, image=64, base=16, blocks=(1, 1, 1, 1), classes=40)
    g32, w32, f32, _ = models.build_resnet50_qlinear(**kw)
    g8, w8, f8, _ = models.build_resnet50_qlinear(typed_input=True, **kw)
    feeds32, feeds8 = f32(2, "typed_in"), f8(2, "typed_in")
    assert feeds8["input_q"].dtype == np.uint8
    s32 = Session.builder().build_from_graph(g32, w32)
    s8 = Session.builder().build_from_graph(g8, w8)
    c0 = s8.cuda_cache_counters()
    out8 = s8.run(feeds8)["logits"]
    c1 = s8.cuda_cache_counters()
    out32 = s32.run(feeds32)["logits"]
    assert c1["upload_bytes"] - c0["upload_bytes"] == feeds8["input_q"].size, "one byte per lane crosses PCIe"
    assert np.array_equal(out8, out32)
    oracle.set_threads(8)
    want = oracle.run_graph(g8, w8, feeds8, keep_all=False)["logits"]
    assert np.array_equal(out8, want)
    assert np.unique(want).size > 8
    # f32 lanes for an input that was declared u8 are refused, not reinterpreted
    with pytest.raises(OnnxError, match="declared u8"):
        s8.run({"input_q": feeds8["input_q"].astype(np.float32)})
    # the pipelined call takes typed feeds too
    outs = s8.run_pipelined([feeds8, feeds8, feeds8])
    assert all(np.array_equal(o["logits"], want) for o in outs)
    s8.close()
    s32.close()
