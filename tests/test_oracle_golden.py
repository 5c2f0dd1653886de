"""The CPU oracle against the reference's own known-answer vectors
(tests/golden/reference_vectors.json, transcribed from the reference's tests by
file:line) and against closed-form properties of its scalar helpers."""
import json
import os

import numpy as np
import pytest

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
with open(os.path.join(ROOT, "tests", "golden", "reference_vectors.json")) as _fh:
    CASES = json.load(_fh)["cases"]


def _arr(t):
    dtype = {"u8": np.uint8, "i8": np.int8}.get(t.get("dtype"), np.float32)  # a typed tensor keeps its declared type
    return np.asarray(t["data"], dtype=dtype).reshape(t["shape"])


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
@pytest.mark.parametrize("threads", [1, 4])
def test_reference_vector(case, threads):
    oracle.set_threads(threads)
    try:
        ins = [_arr(t) for t in case["inputs"]]
        if "error_kind" in case:  # the OnnxError variant the reference's test matches on
            with pytest.raises(oracle.OracleError) as ei:
                oracle.run_node(case["op"], ins, case["attrs"], n_outputs=1)
            assert ei.value.kind == case["error_kind"], str(ei.value)
            return
        if "error_contains" in case:
            with pytest.raises(oracle.OracleError) as ei:
                oracle.run_node(case["op"], ins, case["attrs"], n_outputs=1)
            assert case["error_contains"] in str(ei.value)
            return
        outs = oracle.run_node(case["op"], ins, case["attrs"], n_outputs=len(case["expected"]))
        exact = case["exact"]
        for i, (got, want) in enumerate(zip(outs, case["expected"])):
            w = _arr(want)
            assert list(got.shape) == want["shape"], f"{case['name']} output {i}: shape"
            rule = exact[i] if isinstance(exact, list) else exact
            if rule is True:
                assert np.array_equal(got, w), f"{case['name']} output {i}: {got} vs {w} ({case['source']})"
            else:
                assert np.all(np.abs(got - w) <= float(rule)), f"{case['name']} output {i}"
    finally:
        oracle.set_threads(1)


def test_round_ties_even_matches_numpy_rint():
    rng = np.random.default_rng(7)
    vals = np.concatenate([rng.normal(0, 300, 2000), np.arange(-20, 20) + 0.5, np.arange(-20, 20, dtype=np.float64)])
    for v in vals:
        assert oracle.round_ties_even_f64(v) == np.rint(v)
        assert oracle.round_ties_even_f32(np.float32(v)) == np.rint(np.float32(v))


def test_requantize_is_f64_product_then_add_then_ties_even():
    rng = np.random.default_rng(11)
    for _ in range(2000):
        acc = int(rng.integers(-2**30, 2**30))
        combined = np.float32(rng.uniform(1e-7, 1e-2))
        zp = int(rng.integers(-128, 256))
        want = np.clip(np.rint(np.float64(acc) * np.float64(combined) + np.float64(zp)), 0, 255)
        assert oracle.requantize(acc, combined, zp, 0, 255) == np.float32(want)


def test_integer_ops_threads_are_bit_identical():
    rng = np.random.default_rng(3)
    x = rng.integers(0, 256, (2, 8, 9, 9)).astype(np.float32)
    w = rng.integers(-127, 128, (6, 4, 3, 3)).astype(np.float32)
    ins = [x, np.float32([0.03]), np.float32([128]), w, rng.uniform(0.001, 0.01, 6).astype(np.float32), np.zeros(6, np.float32),
           np.float32([0.07]), np.float32([0]), rng.integers(-1000, 1000, 6).astype(np.float32)]
    attrs = {"group": 2, "pads": [1, 1, 1, 1], "strides": [2, 1]}
    oracle.set_threads(1)
    a, = oracle.run_node("QLinearConv", ins, attrs)
    oracle.set_threads(4)
    b, = oracle.run_node("QLinearConv", ins, attrs)
    oracle.set_threads(1)
    assert np.array_equal(a, b)


def test_qlinear_conv_equals_dequantised_float_conv_on_exact_grid():
    """Size-independent property: with power-of-two scales every quantity is exact in f32,
    so QLinearConv must equal quantise(conv(dequantise(x), dequantise(w)))."""
    rng = np.random.default_rng(5)
    x = rng.integers(0, 256, (1, 4, 6, 6)).astype(np.float32)
    w = rng.integers(-8, 8, (3, 4, 3, 3)).astype(np.float32)
    xs, ws, ys, xzp, yzp = 0.25, 0.5, 4.0, 128.0, 130.0
    q, = oracle.run_node("QLinearConv", [x, np.float32([xs]), np.float32([xzp]), w, np.float32([ws]), np.float32([0]), np.float32([ys]),
                                         np.float32([yzp])], {"pads": [1, 1, 1, 1]})
    f, = oracle.run_node("Conv", [(x - xzp) * xs, w * ws], {"pads": [1, 1, 1, 1]})
    want = np.clip(np.rint(f.astype(np.float64) / ys) + yzp, 0, 255)
    assert np.array_equal(q, want.astype(np.float32))


def test_conv_geometry_errors_are_typed():
    x = np.zeros((1, 2, 4, 4), np.float32)
    w = np.zeros((2, 3, 3, 3), np.float32)
    with pytest.raises(oracle.OracleError) as ei:
        oracle.run_node("Conv", [x, w], {})
    assert ei.value.kind == "ShapeMismatch"
    with pytest.raises(oracle.OracleError) as ei:
        oracle.run_node("Conv", [x, np.zeros((2, 2, 3, 3), np.float32)], {"auto_pad": "BOGUS"})
    assert ei.value.kind == "Unsupported"


def test_fused_clip_edge_cases():
    """NaN bound = unbounded on that side; inverted range = pass-through
    (oxionnx-ops/src/registry/conv_ops/conv.rs:124-156)."""
    x = np.float32([[[[-3.0, 0.5, 9.0]]]])
    w = np.float32([[[[1.0]]]])
    y, = oracle.run_node("Conv", [x, w], {"activation": "clip", "activation_min": float("nan"), "activation_max": 6.0})
    assert np.array_equal(y.ravel(), np.float32([-3.0, 0.5, 6.0]))
    y, = oracle.run_node("Conv", [x, w], {"activation": "clip", "activation_min": 5.0, "activation_max": 1.0})
    assert np.array_equal(y.ravel(), np.float32([-3.0, 0.5, 9.0]))
    y, = oracle.run_node("Conv", [x, w], {"activation": "relu"})
    assert np.array_equal(y.ravel(), np.float32([0.0, 0.5, 9.0]))
