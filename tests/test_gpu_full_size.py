"""The benchmark's networks at their full per-image size against the CPU oracle: the INT8 ResNet-50 (224 x 224,
width 64) bit for bit on every logit and on every quantised tensor a session keeps, the f32 ResNet-50 within 1e-2
of its logits' magnitude (TF32 operands; bf16 operands 3e-2), the InSwapper-shaped generator within 2.5e-2 of its
image's range.  Small batches keep the oracle's share to tens of seconds on the GPU box's host cores.

Two things these sizes show that the reduced networks do not.  (1) The randomly initialised f32 ResNet-50 has no
real normalisation, its activations grow to 1.6e5 by the last block: beyond the range of f16 (65504), so f16
operands overflow on THIS network (the conversion is IEEE: infinity); bf16 has f32's range and is what is checked
here, f16 is checked on the reduced network whose activations fit.  (2) Fifty TF32 layers with an instance
normalisation between most of them drift to 1.7e-2 of the generator's output range although every node, fed the
oracle's inputs, stays inside the rigorous TF32 bound (test_gpu_teacher_forced.py); the bound here is 2.5e-2."""
import os

import numpy as np
import pytest

import oracle
from oxionnx_b200 import models
from oxionnx_b200.session import Session

pytestmark = pytest.mark.gpu


def oracle_threads():
    oracle.set_threads(max(1, min(32, os.cpu_count() or 1)))


def test_int8_resnet50_full_size_is_the_oracle_bit_for_bit():
    graph, weights, feeds, _ = models.build_resnet50_qlinear(batch=2, image=224)
    f = feeds(2)
    oracle_threads()
    ref = oracle.run_graph(graph, weights, f)
    oracle.set_threads(1)
    # the session a user gets: fused residual joins, quantising stem pack, dequantising pool, packed requantisation
    sess = Session.builder().build_from_graph(graph, weights)
    out = sess.run(f)
    assert np.array_equal(out["logits"], ref["logits"])
    kernels = [s["kernel"] for s in sess.steps()]
    assert sum(k.startswith("umma_i8") for k in kernels) == 54, kernels
    sess.close()
    # and node by node: every quantised tensor of the network
    inspect = Session.builder().with_keep_intermediates(True).build_from_graph(graph, weights)
    inspect.run(f)
    checked = 0
    for node in graph.nodes:
        if node.op not in ("QLinearConv", "QuantizeLinear", "MaxPool"):
            continue
        name = node.outputs[0]
        if inspect.has_value(name):
            assert np.array_equal(inspect.fetch_value(name), ref[name]), name
            checked += 1
    assert checked >= 36, checked  # the rest are fused into their consumers even in the inspecting session
    inspect.close()


def test_f32_resnet50_full_size_within_the_float_tolerance():
    graph, weights, feeds, _ = models.build_resnet50_f32(batch=1, image=224)
    f = feeds(1)
    oracle_threads()
    want = oracle.run_graph(graph, weights, f, keep_all=False)["logits"]
    oracle.set_threads(1)
    for precision, bound in (("tf32", 1e-2), ("bf16", 3e-2)):
        sess = Session.builder().with_tuning(float_precision=precision).build_from_graph(graph, weights)
        got = sess.run(f)["logits"]
        sess.close()
        err = float(np.max(np.abs(got.astype(np.float64) - want)) / np.max(np.abs(want)))
        print(f"ResNet-50 f32 at 224 x 224, {precision} operands: final-output error {err:.2e} of the output's magnitude")
        assert err <= bound, (precision, err)
        assert int(np.argmax(got)) == int(np.argmax(want))


def test_inswapper_full_size_within_the_float_tolerance():
    graph, weights, feeds, _ = models.build_inswapper_f32(batch=1)
    f = feeds(1)
    oracle_threads()
    want = oracle.run_graph(graph, weights, f, keep_all=False)["image"]
    oracle.set_threads(1)
    sess = Session.builder().build_from_graph(graph, weights)
    got = sess.run(f)["image"]
    sess.close()
    err = float(np.max(np.abs(got.astype(np.float64) - want)) / np.max(np.abs(want)))
    print(f"InSwapper-shaped generator at 128 x 128: final-output error {err:.2e} of the output's magnitude")
    assert err <= 2.5e-2, err
