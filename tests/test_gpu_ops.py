"""Per-operator parity on the B200: every node goes through the C ABI (oxb200_dispatch, the
counterpart of try_cuda_dispatch_resident) and is compared with the CPU oracle on the same
seeded inputs, and with the reference's own known-answer vectors.

Integer and quantised operators: bit-exact.  Float operators: |a-b| <= atol + rtol*|b| with
rtol = 2e-3 (the TF32 tolerance of the path) and atol = 2e-3 * max|b|.
"""
import json
import zlib
import os

import numpy as np
import pytest

import oracle
from oxionnx_b200.graph import Node
from oxionnx_b200 import session as S

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
with open(os.path.join(ROOT, "tests", "golden", "reference_vectors.json")) as _fh:
    CASES = json.load(_fh)["cases"]

RTOL_TF32 = 2e-3


@pytest.fixture(scope="module", params=["auto", "direct"])
def ctx(request):
    c = S.CudaContext(0, kernel_path=request.param)
    yield c
    c.close()


@pytest.fixture(scope="module")
def ctx_auto():
    c = S.CudaContext(0)
    yield c
    c.close()


def _arr(t):
    dtype = {"u8": np.uint8, "i8": np.int8}.get(t.get("dtype"), np.float32)  # a typed tensor keeps its declared type
    return np.asarray(t["data"], dtype=dtype).reshape(t["shape"])


def dispatch(ctx, op, inputs, attrs=None, n_out=1, initializers=()):
    """One node through the dispatch entry; the inputs whose positions `initializers` lists are handed over as weights."""
    names = [f"in{i}" if x is not None else "" for i, x in enumerate(inputs)]
    node = Node(op=op, name="op0", inputs=names, outputs=[f"out{i}" for i in range(n_out)], attrs=dict(attrs or {}))
    inter = {n: x for i, (n, x) in enumerate(zip(names, inputs)) if n and i not in initializers}
    weights = {n: x for i, (n, x) in enumerate(zip(names, inputs)) if n and i in initializers}
    return S.try_cuda_dispatch(node, weights, inter, ctx)


def assert_close_tf32(got, want, what=""):
    want = np.asarray(want, np.float32)
    atol = RTOL_TF32 * float(np.max(np.abs(want))) if want.size else 0.0
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    bound = atol + RTOL_TF32 * np.abs(want)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    assert np.all(err <= bound), f"{what}: max err {err.max()} (bound {bound[np.argmax(err - bound)]}), {np.sum(err > bound)} lanes off"


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_reference_vector_through_abi(ctx, case):
    ins = [_arr(t) for t in case["inputs"]]
    if "error_kind" in case:
        # malformed geometry is not taken: the node falls to the CPU operator, which raises the typed error
        assert dispatch(ctx, case["op"], ins, case["attrs"]) is None
        assert ctx.last_error()
        return
    if "error_contains" in case:
        # malformed quantised nodes decline so that the CPU operator raises its own typed error
        assert dispatch(ctx, case["op"], ins, case["attrs"]) is None
        assert case["error_contains"].split()[-1] in ctx.last_error() or "scale" in ctx.last_error() or "entries" in ctx.last_error()
        return
    outs = dispatch(ctx, case["op"], ins, case["attrs"], n_out=len(case["expected"]))
    assert outs is not None, ctx.last_error()
    exact = case["exact"]
    for i, (got, want) in enumerate(zip(outs, case["expected"])):
        w = _arr(want)
        assert list(got.shape) == want["shape"]
        rule = exact[i] if isinstance(exact, list) else exact
        if rule is True:
            assert np.array_equal(got, w), f"{case['name']} output {i}: {got.ravel()[:8]} vs {w.ravel()[:8]} ({case['source']})"
        else:
            assert np.all(np.abs(got - w) <= float(rule))


QCONV_SHAPES = [
    # N, C, H, W, OC, k, stride, pad, x_zp, relu-ish y_zp
    (2, 32, 9, 9, 32, 1, 1, 0, 128, 128),      # 32-byte channel block, M tail
    (3, 64, 14, 14, 64, 3, 1, 1, 0, 0),        # 64-byte block, 3x3 halo, row wrap inside a tile
    (2, 128, 7, 7, 256, 3, 2, 1, 0, 128),      # stride 2, two channel tiles
    (1, 256, 8, 8, 40, 1, 2, 0, 128, 0),       # 1x1 stride 2 (projection shortcut), ragged OC
    (2, 64, 12, 10, 128, 3, 1, 1, 0, 128),     # non-square
    (5, 64, 16, 16, 64, 3, 1, 1, 128, 0),      # padded with a non-zero zero point: direct kernel
    (2, 3, 20, 20, 16, 7, 2, 3, 128, 0),       # stem geometry: direct kernel
    (1, 512, 4, 4, 1000, 1, 1, 0, 128, 128),   # classifier as a 1x1 convolution
    (2, 1024, 7, 7, 256, 3, 1, 1, 128, 128),   # one row tile, 72 K blocks: K split over several CTAs
    (3, 1024, 9, 9, 96, 3, 1, 1, 0, 0),        # split K with a ragged channel tile and 16-bit lanes
]


@pytest.mark.parametrize("shape", QCONV_SHAPES, ids=[str(s) for s in QCONV_SHAPES])
def test_qlinear_conv_bit_exact(ctx, shape):
    n, c, h, w, oc, k, stride, pad, x_zp, y_zp = shape
    rng = np.random.default_rng(zlib.crc32(repr(shape).encode()))
    if x_zp == 0:
        x = rng.integers(0, 128, (n, c, h, w)).astype(np.float32)
    else:
        x = rng.integers(0, 256, (n, c, h, w)).astype(np.float32)
    wt = rng.integers(-127, 128, (oc, c, k, k)).astype(np.float32)
    ws = rng.uniform(0.001, 0.01, oc).astype(np.float32)
    bias = rng.integers(-1000, 1001, oc).astype(np.float32)
    y_scale = np.float32(0.005 * 73.0 * np.sqrt(c * k * k) * 40 * 0.02 / 40.0)
    ins = [x, np.float32([0.02]), np.float32([x_zp]), wt, ws, np.zeros(oc, np.float32), np.float32([y_scale]), np.float32([y_zp]), bias]
    attrs = {"strides": [stride, stride], "pads": [pad] * 4, "kernel_shape": [k, k]}
    oracle.set_threads(8)
    want, = oracle.run_node("QLinearConv", ins, attrs)
    got = dispatch(ctx, "QLinearConv", ins, attrs)
    assert got is not None, ctx.last_error()
    assert np.array_equal(got[0], want), f"{np.sum(got[0] != want)} of {want.size} lanes differ; first {got[0].ravel()[:6]} vs {want.ravel()[:6]}"
    assert np.unique(want).size > 8, "degenerate test vector"


PAIR_SHAPES = [
    # N, C, H, W, OC, k, stride, pad: shapes the CTA-pair form (tcgen05 cta_group::2, one 256 x 256 tile per two CTAs) must get right
    (2, 256, 16, 16, 256, 3, 1, 1),     # two full pair tiles, 18 K blocks, halo rows
    (3, 128, 11, 13, 512, 3, 1, 1),     # M = 429: the second CTA of the last pair is mostly past the end; two channel tiles
    (1, 256, 9, 9, 320, 1, 1, 0),       # M = 81 (< 128: the odd CTA has no rows at all), ragged second channel tile
    (5, 64, 14, 14, 256, 3, 2, 1),      # stride 2, 64-byte K blocks
    (2, 512, 20, 20, 256, 1, 1, 0),     # plain GEMM form (2-D tiled loads), M = 800
]


@pytest.mark.parametrize("shape", PAIR_SHAPES, ids=[str(s) for s in PAIR_SHAPES])
def test_cta_pair_kernel_matches_oracle_and_lone_cta_kernel(shape):
    """The pair form against the oracle (bit-exact for QLinearConv, TF32 tolerance for Conv) and against the
    one-CTA-per-tile form of the same layer (bit-exact for the integers; the float forms may sum the K blocks
    in different orders, e.g. when the lone-CTA form splits K, so they are held to the tolerance)."""
    n, c, h, w, oc, k, stride, pad = shape
    rng = np.random.default_rng(zlib.crc32(repr(("pair",) + shape).encode()))
    oracle.set_threads(8)
    attrs = {"strides": [stride, stride], "pads": [pad] * 4, "kernel_shape": [k, k]}
    x = rng.integers(0, 128, (n, c, h, w)).astype(np.float32)
    wt = rng.integers(-127, 128, (oc, c, k, k)).astype(np.float32)
    ws = rng.uniform(0.001, 0.01, oc).astype(np.float32)
    bias = rng.integers(-1000, 1001, oc).astype(np.float32)
    y_scale = np.float32(0.005 * 73.0 * np.sqrt(c * k * k) * 0.02)
    qins = [x, np.float32([0.02]), np.float32([0]), wt, ws, np.zeros(oc, np.float32), np.float32([y_scale]), np.float32([128]), bias]
    xf = rng.standard_normal((n, c, h, w)).astype(np.float32)
    wf = (rng.standard_normal((oc, c, k, k)) / np.sqrt(c * k * k)).astype(np.float32)
    bf = rng.standard_normal(oc).astype(np.float32)
    fattrs = dict(attrs, activation="relu")
    results = {}
    for mode in ("always", "never"):
        ctx = S.CudaContext(0, cta_pairs=mode)
        got_q = dispatch(ctx, "QLinearConv", qins, attrs)
        got_f = dispatch(ctx, "Conv", [xf, wf, bf], fattrs)
        assert got_q is not None and got_f is not None, ctx.last_error()
        results[mode] = (got_q[0], got_f[0])
        ctx.close()
    want_q, = oracle.run_node("QLinearConv", qins, attrs)
    want_f, = oracle.run_node("Conv", [xf, wf, bf], fattrs)
    assert np.array_equal(results["always"][0], want_q), f"{np.sum(results['always'][0] != want_q)} of {want_q.size} lanes differ"
    assert np.array_equal(results["never"][0], want_q)
    assert np.unique(want_q).size > 8, "degenerate test vector"
    assert_close_tf32(results["always"][1], want_f, "pair Conv")
    assert_close_tf32(results["never"][1], want_f, "lone-CTA Conv")


def test_cta_pair_kernel_is_the_one_that_runs_when_forced():
    from oxionnx_b200.graph import Graph
    rng = np.random.default_rng(5)
    weights = {"w": rng.integers(-127, 128, (256, 256, 3, 3)).astype(np.float32), "ws": rng.uniform(0.001, 0.01, 256).astype(np.float32),
               "wz": np.zeros(256, np.float32), "b": rng.integers(-1000, 1000, 256).astype(np.float32), "xs": np.float32([0.02]), "z0": np.float32([0]),
               "ys": np.float32([0.5]), "qs": np.float32([0.02])}
    graph = Graph(nodes=[Node("QuantizeLinear", "q", ["x", "qs", "z0"], ["xq"], {}),
                         Node("QLinearConv", "conv", ["xq", "xs", "z0", "w", "ws", "wz", "ys", "z0", "b"], ["yq"], {"pads": [1, 1, 1, 1]}),
                         Node("DequantizeLinear", "dq", ["yq", "ys", "z0"], ["y"], {})], input_names=["x"], output_names=["y"])
    x = np.abs(rng.standard_normal((2, 256, 12, 12))).astype(np.float32)
    outs = {}
    for mode in ("always", "never"):
        sess = S.Session.builder().with_tuning(cta_pairs=mode).build_from_graph(graph, weights)
        outs[mode] = sess.run({"x": x})["y"]
        kernel = [s_["kernel"] for s_ in sess.steps() if s_["node"] == "conv"][0]
        assert ("cta-pair" in kernel) == (mode == "always"), kernel
        sess.close()
    oracle.set_threads(8)
    want = oracle.run_graph(graph, weights, {"x": x}, keep_all=False)["y"]
    assert np.array_equal(outs["always"], want) and np.array_equal(outs["never"], want)


@pytest.mark.parametrize("form", [0, 1, 2], ids=["auto (packed saturation)", "two-pass f64", "one FMA, unpacked"])
@pytest.mark.parametrize("relu", [False, True], ids=["i8 range", "relu"])
def test_every_requantisation_form_of_the_tensor_core_epilogue_is_bit_exact(form, relu):
    """The requantising epilogue has three forms (f32 estimate + f64 second pass; one fused multiply-add per lane;
    the same with the saturation done on packed 16-bit lanes): each, forced through the context's tuning, must
    give the reference's lanes on the same layer, with and without a Relu folded into the saturation."""
    from oxionnx_b200.graph import Graph
    rng = np.random.default_rng(31 + int(relu))
    c, oc = 128, 192
    weights = {"w": rng.integers(-127, 128, (oc, c, 3, 3)).astype(np.float32), "ws": rng.uniform(0.001, 0.01, oc).astype(np.float32),
               "wz": np.zeros(oc, np.float32), "b": rng.integers(-1000, 1000, oc).astype(np.float32), "xs": np.float32([0.02]), "z0": np.float32([0]),
               "yz": np.float32([0 if relu else -3]), "ys": np.float32([0.35]), "qs": np.float32([0.02])}
    nodes = [Node("QuantizeLinear", "q", ["x", "qs", "z0"], ["xq"], {}),
             Node("QLinearConv", "conv", ["xq", "xs", "z0", "w", "ws", "wz", "ys", "yz", "b"], ["yq"], {"pads": [1, 1, 1, 1]})]
    last = "yq"
    if relu:
        nodes.append(Node("Relu", "r", ["yq"], ["yr"], {}))
        last = "yr"
    nodes.append(Node("DequantizeLinear", "dq", [last, "ys", "yz"], ["y"], {}))
    graph = Graph(nodes=nodes, input_names=["x"], output_names=["y"])
    x = np.abs(rng.standard_normal((3, c, 10, 10))).astype(np.float32)
    sess = S.Session.builder().with_tuning(requant_f64=form).build_from_graph(graph, weights)
    got = sess.run({"x": x})["y"]
    sess.close()
    oracle.set_threads(8)
    want = oracle.run_graph(graph, weights, {"x": x}, keep_all=False)["y"]
    assert np.array_equal(got, want), f"{np.sum(got != want)} of {want.size} lanes differ"
    assert np.unique(want).size > 16, "degenerate test vector"


def test_conv_integer_and_matmul_integer_bit_exact(ctx):
    rng = np.random.default_rng(17)
    oracle.set_threads(8)
    x = rng.integers(0, 256, (2, 64, 10, 10)).astype(np.float32)
    w = rng.integers(-127, 128, (96, 64, 3, 3)).astype(np.float32)
    for xzp, pads in ((0.0, [1, 1, 1, 1]), (7.0, [0, 0, 0, 0]), (130.0, [1, 0, 2, 1])):
        ins = [x, w, np.float32([xzp])]
        attrs = {"pads": pads}
        want, = oracle.run_node("ConvInteger", ins, attrs)
        got = dispatch(ctx, "ConvInteger", ins, attrs)
        assert got is not None, ctx.last_error()
        assert np.array_equal(got[0], want)
    a = rng.integers(0, 256, (130, 3072)).astype(np.float32)
    b = rng.integers(-127, 128, (3072, 96)).astype(np.float32)
    for azp in (np.float32([128]), np.float32([0]), None):
        ins = [a, b, azp] if azp is not None else [a, b]
        want, = oracle.run_node("MatMulInteger", ins)
        got = dispatch(ctx, "MatMulInteger", ins)
        assert got is not None, ctx.last_error()
        assert np.array_equal(got[0], want)
    # accumulators above 2^24 are rounded (to nearest even) when stored as f32 lanes, on both sides alike
    bpos = rng.integers(64, 128, (3072, 96)).astype(np.float32)
    want, = oracle.run_node("MatMulInteger", [a, bpos])
    got = dispatch(ctx, "MatMulInteger", [a, bpos])
    assert np.array_equal(got[0], want)
    assert np.abs(want).max() > 2**24 and np.any(want % 2 == 0)
    # per-row a_zero_point and per-column b_zero_point, batched A
    a3 = rng.integers(0, 256, (2, 5, 64)).astype(np.float32)
    b2 = rng.integers(0, 256, (64, 48)).astype(np.float32)
    ins = [a3, b2, rng.integers(0, 256, 5).astype(np.float32), rng.integers(0, 256, 48).astype(np.float32)]
    want, = oracle.run_node("MatMulInteger", ins)
    got = dispatch(ctx, "MatMulInteger", ins)
    assert got is not None, ctx.last_error()
    assert np.array_equal(got[0], want)


def test_qlinear_matmul_bit_exact(ctx):
    rng = np.random.default_rng(23)
    oracle.set_threads(8)
    for (m, k, n, azp, yzp) in ((64, 1024, 256, 128, 128), (200, 128, 72, 0, 0), (7, 96, 33, 113, 118)):
        a = rng.integers(0, 256, (m, k)).astype(np.float32)
        b = rng.integers(-127, 128, (k, n)).astype(np.float32)
        ins = [a, np.float32([0.05]), np.float32([azp]), b, np.float32([0.011]), np.float32([0]), np.float32([0.1 * np.sqrt(k) / 8]), np.float32([yzp])]
        want, = oracle.run_node("QLinearMatMul", ins)
        got = dispatch(ctx, "QLinearMatMul", ins)
        assert got is not None, ctx.last_error()
        assert np.array_equal(got[0], want), f"{(m, k, n)}: {np.sum(got[0] != want)} lanes differ"


REQUANT_EDGE = [
    # name, K, generator, a_scale, b_scale, y_scale, a_zp, y_zp
    ("exact ties, combined 0.5", 32, ("uniform", (0, 8), (-3, 4)), 1.0, 0.5, 1.0, 0, 0),
    ("exact ties, combined 0.125 with zero points", 64, ("uniform", (0, 16), (-7, 8)), 0.25, 0.5, 1.0, 3, 131),
    ("accumulators beyond 2^24", 1024, ("big", 100, 128), 0.001, 0.001, 0.5, 0, 128),
    ("accumulators beyond 2^24, both signs", 2048, ("big_signed", 100, 128), 0.002, 0.001, 1.0, 0, 128),
    ("combined scale below 2^-21 (two-pass variant)", 4096, ("big_signed", 64, 128), 1e-4, 1e-4, 0.05, 0, 128),
    ("combined scale above one", 32, ("uniform", (0, 4), (-2, 3)), 2.0, 1.5, 1.0, 0, 100),
]


def _requant_edge_operands(rng, gen, m, k, n):
    if gen[0] == "uniform":
        return rng.integers(*gen[1], (m, k)).astype(np.float32), rng.integers(*gen[2], (k, n)).astype(np.float32)
    # rows of A at one level each, columns of B of one sign each: |sum| grows to K * 255 * 127
    a = np.clip(rng.integers(128, 256, (m, 1)) + rng.integers(-2, 3, (m, k)), 0, 255).astype(np.float32)
    b = rng.integers(gen[1], gen[2], (k, n)).astype(np.float32)
    if gen[0] == "big_signed":
        b *= rng.choice(np.float32([-1, 1]), (1, n))
    return a, b


@pytest.mark.parametrize("case", REQUANT_EDGE, ids=[c[0] for c in REQUANT_EDGE])
@pytest.mark.parametrize("force_f64", [False, True], ids=["fma", "two-pass"])
def test_requantisation_edge_cases_bit_exact(case, force_f64):
    """The tensor-core epilogue has two requantisation variants (one fused multiply-add per lane
    when the scales allow it, an f32 estimate with an f64 second pass otherwise); both must equal
    the reference's f64 arithmetic on ties, on accumulators that f32 cannot hold exactly and on
    extreme scales (SatRange::requantize, oxionnx-ops/src/registry/quant_ops/mod.rs:229-233)."""
    name, k, gen, a_scale, b_scale, y_scale, a_zp, y_zp = case
    ctx_auto = S.CudaContext(0, requant_f64=force_f64)
    rng = np.random.default_rng(zlib.crc32(name.encode()))
    oracle.set_threads(8)
    m, n = 256, 96
    a, b = _requant_edge_operands(rng, gen, m, k, n)
    ins = [a, np.float32([a_scale]), np.float32([a_zp]), b, np.float32([b_scale]), np.float32([0]), np.float32([y_scale]), np.float32([y_zp])]
    want, = oracle.run_node("QLinearMatMul", ins)
    got = dispatch(ctx_auto, "QLinearMatMul", ins)
    assert got is not None, ctx_auto.last_error()
    ctx_auto.close()
    assert np.array_equal(got[0], want), f"{name}: {np.sum(got[0] != want)} of {want.size} lanes differ"
    assert np.unique(want).size > 4, "degenerate test vector"


def test_quantize_dequantize_dynamic_bit_exact(ctx):
    rng = np.random.default_rng(29)
    x = (rng.standard_normal((4, 6, 10, 12)) * 3).astype(np.float32)
    x.ravel()[:64] = (np.arange(64) - 32) * 0.025 + 0.0125  # exact ties at scale 0.05
    for zp in (np.float32([128]), np.float32([0]), None):
        ins = [x, np.float32([0.05])] + ([zp] if zp is not None else [])
        want, = oracle.run_node("QuantizeLinear", ins)
        got = dispatch(ctx, "QuantizeLinear", ins)
        assert np.array_equal(got[0], want)
    scale_c = rng.uniform(0.01, 0.1, 6).astype(np.float32)
    zp_c = rng.integers(120, 140, 6).astype(np.float32)
    want, = oracle.run_node("QuantizeLinear", [x, scale_c, zp_c], {"axis": 1})
    got = dispatch(ctx, "QuantizeLinear", [x, scale_c, zp_c], {"axis": 1})
    assert np.array_equal(got[0], want)
    q = rng.integers(0, 256, (4, 6, 10, 12)).astype(np.float32)
    want, = oracle.run_node("DequantizeLinear", [q, scale_c, zp_c], {"axis": 1})
    got = dispatch(ctx, "DequantizeLinear", [q, scale_c, zp_c], {"axis": 1})
    assert np.array_equal(got[0], want)
    want, = oracle.run_node("DequantizeLinear", [q, np.float32([0.037]), np.float32([128])])
    got = dispatch(ctx, "DequantizeLinear", [q, np.float32([0.037]), np.float32([128])])
    assert np.array_equal(got[0], want)
    # quotients on and next to every tie k + 0.5 (scale exactly 1, then a scale with a full mantissa), sizes that
    # leave ragged ends for the 512-lane warp tiles, and scales at the ends of the exponent range
    ties = np.concatenate([np.arange(0, 255, 0.5, dtype=np.float32), np.float32([0.0, 255.0])])
    ties = np.concatenate([ties, np.nextafter(ties, np.float32(300)), np.nextafter(ties, np.float32(-300))]).astype(np.float32)
    ties = np.clip(ties, 0, 255).astype(np.float32)
    odd = np.float32(0.7310585975646973)
    wide = (rng.standard_normal(513 * 41 + 3) * 3).astype(np.float32)
    for arr in (x.reshape(24, 120), np.zeros((3, 5), np.float32), np.float32([[-0.5, 254.5]]), (rng.standard_normal((1000, 77)) * 5).astype(np.float32),
                ties.reshape(1, -1), (ties * odd).reshape(1, -1), (ties - np.float32(100.5)).reshape(1, -1), wide.reshape(1, -1),
                (wide * np.float32(1e-36)).reshape(1, -1), (wide * np.float32(1e33)).reshape(1, -1), wide[:2051].reshape(7, 293)):
        want = oracle.run_node("DynamicQuantizeLinear", [arr], n_outputs=3)
        got = dispatch(ctx, "DynamicQuantizeLinear", [arr], n_out=3)
        assert got is not None, ctx.last_error()
        for g, w in zip(got, want):
            assert g.shape == w.shape
            assert np.array_equal(g, w)


FCONV_SHAPES = [
    (2, 8, 12, 12, 16, 3, 1, 1, "relu"),     # 32-byte channel block
    (3, 16, 9, 9, 24, 1, 1, 0, ""),          # 64-byte block, 1x1 GEMM path, ragged OC
    (2, 32, 14, 14, 64, 3, 2, 1, "relu"),    # 128-byte block, stride 2
    (1, 64, 7, 7, 256, 1, 2, 0, ""),         # projection shortcut
    (2, 64, 8, 8, 64, 3, 1, 1, "clip"),
    (2, 3, 32, 32, 16, 7, 2, 3, "relu"),     # stride-2 stem: space-to-depth row windows
    (2, 3, 20, 18, 40, 7, 1, 3, "relu"),     # stride-1 image-space 7x7 with its own padding: four-lane row windows
    (2, 3, 19, 19, 32, 7, 1, 0, ""),         # the same behind an explicit reflect Pad (no padding of its own)
    (1, 4, 12, 12, 16, 3, 1, 1, ""),         # four channels, 3x3 (windows of four pixels)
    (2, 256, 7, 7, 512, 3, 1, 1, "relu"),    # one row tile, 72 K blocks: K split over several CTAs
    (4, 1024, 7, 7, 200, 1, 1, 0, ""),       # split K on the 1x1 GEMM path, ragged channel tile
    (1, 6, 10, 10, 6, 3, 1, 1, ""),          # depthwise-like groups below
]


@pytest.mark.parametrize("shape", FCONV_SHAPES, ids=[str(s) for s in FCONV_SHAPES])
def test_float_conv_within_tf32_tolerance(ctx, shape):
    n, c, h, w, oc, k, stride, pad, act = shape
    rng = np.random.default_rng(zlib.crc32(repr(shape).encode()))
    x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    group = 3 if c == 6 else 1
    wt = (rng.standard_normal((oc, c // group, k, k)) * np.sqrt(2.0 / (c * k * k))).astype(np.float32)
    b = (rng.standard_normal(oc) * 0.1).astype(np.float32)
    attrs = {"strides": [stride, stride], "pads": [pad] * 4, "group": group}
    if act:
        attrs["activation"] = act
    if act == "clip":
        attrs["activation_min"] = 0.0
        attrs["activation_max"] = 0.75
    oracle.set_threads(8)
    want, = oracle.run_node("Conv", [x, wt, b], attrs)
    got = dispatch(ctx, "Conv", [x, wt, b], attrs)
    assert got is not None, ctx.last_error()
    assert_close_tf32(got[0], want, f"Conv {shape}")


def test_gemm_and_matmul_within_tf32_tolerance(ctx):
    rng = np.random.default_rng(31)
    a = rng.standard_normal((32, 2048)).astype(np.float32)
    w = (rng.standard_normal((1000, 2048)) / 45).astype(np.float32)
    bias = rng.standard_normal(1000).astype(np.float32)
    want, = oracle.run_node("Gemm", [a, w, bias], {"transB": 1, "alpha": 1.0, "beta": 1.0})
    got = dispatch(ctx, "Gemm", [a, w, bias], {"transB": 1, "alpha": 1.0, "beta": 1.0})
    assert_close_tf32(got[0], want, "Gemm transB")
    w2 = np.ascontiguousarray(w.T)
    want, = oracle.run_node("Gemm", [a, w2, bias], {"alpha": 0.5, "beta": 2.0})
    got = dispatch(ctx, "Gemm", [a, w2, bias], {"alpha": 0.5, "beta": 2.0})
    assert_close_tf32(got[0], want, "Gemm alpha beta")
    a3 = rng.standard_normal((2, 3, 17, 64)).astype(np.float32)
    b2 = rng.standard_normal((64, 40)).astype(np.float32)
    want, = oracle.run_node("MatMul", [a3, b2])
    got = dispatch(ctx, "MatMul", [a3, b2])
    assert_close_tf32(got[0], want, "MatMul stacked A")


def test_glue_ops_match_oracle(ctx_auto):
    ctx = ctx_auto
    rng = np.random.default_rng(37)
    x = rng.standard_normal((2, 24, 13, 11)).astype(np.float32)
    y = rng.standard_normal((2, 24, 13, 11)).astype(np.float32)
    for op in ("Add", "Sub", "Mul", "Div"):
        want, = oracle.run_node(op, [x, y])
        got = dispatch(ctx, op, [x, y])
        assert np.array_equal(got[0], want), op
    sc = rng.standard_normal((2, 24, 1, 1)).astype(np.float32)
    for op in ("Mul", "Add"):
        want, = oracle.run_node(op, [x, sc])
        got = dispatch(ctx, op, [x, sc])
        assert np.array_equal(got[0], want), op + " per-sample broadcast"
    want, = oracle.run_node("Relu", [x])
    assert np.array_equal(dispatch(ctx, "Relu", [x])[0], want)
    want, = oracle.run_node("Tanh", [x])
    assert np.allclose(dispatch(ctx, "Tanh", [x])[0], want, rtol=1e-5, atol=1e-6)
    slope = rng.uniform(0.05, 0.3, (24, 1, 1)).astype(np.float32)
    want, = oracle.run_node("PRelu", [x, slope])
    assert np.array_equal(dispatch(ctx, "PRelu", [x, slope])[0], want)
    attrs = {"kernel_shape": [3, 3], "strides": [2, 2], "pads": [1, 1, 1, 1]}
    want, = oracle.run_node("MaxPool", [x], attrs)
    assert np.array_equal(dispatch(ctx, "MaxPool", [x], attrs)[0], want)
    want, = oracle.run_node("GlobalAveragePool", [x])
    assert np.array_equal(dispatch(ctx, "GlobalAveragePool", [x])[0], want), "sequential f32 sum order"
    want, = oracle.run_node("OxiInstanceNorm", [x], {"epsilon": 1e-5})
    got = dispatch(ctx, "OxiInstanceNorm", [x], {"epsilon": 1e-5})[0]
    assert np.allclose(got, want, rtol=1e-4, atol=1e-5)
    # planes of 256 positions or more are staged in shared memory by the first pass (one read of the tensor)
    big = (rng.standard_normal((3, 40, 16, 20)) * 3 + 1.5).astype(np.float32)
    want, = oracle.run_node("OxiInstanceNorm", [big], {"epsilon": 1e-5})
    got = dispatch(ctx, "OxiInstanceNorm", [big], {"epsilon": 1e-5})[0]
    assert np.allclose(got, want, rtol=1e-4, atol=1e-5)
    for attrs in ({"mode": "nearest", "coordinate_transformation_mode": "asymmetric", "nearest_mode": "floor"},
                  {"mode": "linear", "coordinate_transformation_mode": "half_pixel"},
                  {"mode": "linear", "coordinate_transformation_mode": "pytorch_half_pixel"}):
        ins = [x, None, np.float32([1, 1, 2, 2])]
        want, = oracle.run_node("Resize", ins, attrs)
        got = dispatch(ctx, "Resize", ins, attrs)
        assert got is not None, ctx.last_error()
        assert np.allclose(got[0], want, rtol=1e-6, atol=1e-6), attrs
    for mode in ("reflect", "constant", "edge"):
        ins = [x, np.float32([0, 0, 1, 2, 0, 0, 1, 2])]
        want, = oracle.run_node("Pad", ins, {"mode": mode})
        assert np.array_equal(dispatch(ctx, "Pad", ins, {"mode": mode})[0], want), mode
    z = rng.standard_normal((2, 8, 13, 11)).astype(np.float32)
    want, = oracle.run_node("Concat", [x, z], {"axis": 1})
    assert np.array_equal(dispatch(ctx, "Concat", [x, z], {"axis": 1})[0], want)
    want, = oracle.run_node("Flatten", [x], {"axis": 1})
    assert np.array_equal(dispatch(ctx, "Flatten", [x], {"axis": 1})[0], want)
    for ins in ([x, np.float32([1, 2]), np.float32([3, 9.3e18]), np.float32([1, 3])], [x, np.float32([-3]), np.float32([-1]), np.float32([2])],
                [x[0, 0], np.float32([0, 4]), np.float32([5, 4])]):
        want, = oracle.run_node("Slice", ins)
        got = dispatch(ctx, "Slice", ins)
        assert got is not None, ctx.last_error()
        assert np.array_equal(got[0], want), ins[1:]
    assert dispatch(ctx, "Slice", [x, np.float32([0]), np.float32([4]), np.float32([3]), np.float32([2])]) is None  # strided: declined


def test_transformer_glue_ops_match_oracle(ctx_auto):
    """LayerNormalization, Softmax, Gelu (both forms), Erf, Gather and Transpose, each as one node through the ABI,
    at the absolute tolerances of the reference's own tests (oxionnx-ops src/nn/normalization.rs:912 layer_norm 1e-4,
    :1087 softmax 1e-5; the activations at 1e-5); the two movers are exact."""
    ctx = ctx_auto
    rng = np.random.default_rng(131)
    x = (rng.standard_normal((3, 37, 768)) * 2.5 + 0.7).astype(np.float32)
    gamma = rng.uniform(0.5, 1.5, 768).astype(np.float32)
    beta = rng.standard_normal(768).astype(np.float32)
    for ins, attrs in (([x, gamma, beta], {"axis": -1, "epsilon": 1e-5}), ([x, gamma], {"axis": -1, "epsilon": 1e-12}),
                       ([x[:, :, :96], gamma[:96], beta[:96]], {"axis": 2}), ([x[:, :, :256], gamma[:256], beta[:256]], {}),
                       ([x[:, :, :512], gamma[:512]], {}), ([np.concatenate([x, x[:, :, :256]], -1), np.tile(gamma, 2)[:1024], np.tile(beta, 2)[:1024]], {})):
        want, = oracle.run_node("LayerNormalization", ins, attrs)
        got = dispatch(ctx, "LayerNormalization", ins, attrs, initializers=(1, 2))
        assert got is not None, ctx.last_error()
        assert got[0].shape == want.shape and np.max(np.abs(got[0] - want)) <= 1e-4, (attrs, np.max(np.abs(got[0] - want)))
    # trailing-axes broadcasts (a bias row, a position table added to every sample): bit-exact elementwise results
    pos = rng.standard_normal((37, 768)).astype(np.float32)
    for op in ("Add", "Sub", "Mul", "Div"):
        for other in (beta, pos, pos[None], beta[:6].repeat(128)[None, None]):
            want, = oracle.run_node(op, [x, other])
            got = dispatch(ctx, op, [x, other])
            assert got is not None and np.array_equal(got[0], want), (op, other.shape)
    scores = (rng.standard_normal((2, 12, 37, 37)) * 4).astype(np.float32)
    scores[0, :, :, 30:] = -10000.0  # an attention mask already added
    wide = (rng.standard_normal((2, 3, 128, 128)) * 4).astype(np.float32)  # rows of 128 / 256 / 512 lanes stay in registers
    for ins, attrs in (([scores], {"axis": -1}), ([scores], {}), ([scores[0, 0]], {"axis": 1}), ([x[0]], {"axis": -1}), ([wide], {}),
                       ([wide.reshape(2, 3, 64, 256)], {}), ([wide.reshape(6, 32, 512)], {"axis": 2})):
        want, = oracle.run_node("Softmax", ins, attrs)
        got = dispatch(ctx, "Softmax", ins, attrs)
        assert got is not None, ctx.last_error()
        assert np.max(np.abs(got[0] - want)) <= 1e-5, attrs
        assert np.allclose(got[0].sum(-1), 1.0, atol=1e-5)
    h = (rng.standard_normal((2, 37, 3072)) * 3).astype(np.float32)
    h[0, 0, :8] = [0.0, -0.0, 1e-8, -1e-8, 12.0, -12.0, 40.0, -40.0]
    for op, attrs in (("Gelu", {}), ("Gelu", {"approximate": "none"}), ("Gelu", {"approximate": "tanh"}), ("Erf", {})):
        want, = oracle.run_node(op, [h], attrs)
        got = dispatch(ctx, op, [h], attrs)
        assert got is not None, ctx.last_error()
        assert np.all(np.abs(got[0] - want) <= 1e-5 + 1e-5 * np.abs(want)), (op, attrs, np.max(np.abs(got[0] - want)))
    table = rng.standard_normal((211, 96)).astype(np.float32)
    ids = rng.integers(-211, 211, size=(3, 37)).astype(np.float32)  # negative indices wrap (oxionnx-ops src/indexing/gather.rs:12-44)
    want, = oracle.run_node("Gather", [table, ids], {"axis": 0})
    got = dispatch(ctx, "Gather", [table, ids], {"axis": 0}, initializers=(0,))
    assert got is not None, ctx.last_error()
    assert np.array_equal(got[0], want)
    # an index outside the table is reported, not clamped (the reference raises its own error there)
    own = S.CudaContext(0)  # the failure is counted on the context that met it
    with pytest.raises(S.OnnxError, match="out of range"):
        dispatch(own, "Gather", [table, np.float32([[0, 211]])], {"axis": 0}, initializers=(0,))
    assert own.cache_counters()["failures"] == 1
    own.close()
    t4 = rng.standard_normal((2, 37, 12, 64)).astype(np.float32)
    t5 = rng.standard_normal((2, 128, 3, 64)).astype(np.float32)  # extents in multiples of four: the 16-byte tiled form
    for ins, attrs in (([t4], {"perm": [0, 2, 1, 3]}), ([t4], {"perm": [0, 2, 3, 1]}), ([t4[0, :, 0]], {}), ([t4], {"perm": [0, 1, 2, 3]}),
                       ([t5], {"perm": [0, 2, 3, 1]}), ([t5[:, :40]], {"perm": [0, 2, 3, 1]}), ([t5[0, :, 0, :36]], {})):
        want, = oracle.run_node("Transpose", ins, attrs)
        got = dispatch(ctx, "Transpose", ins, attrs)
        assert got is not None, (attrs, ctx.last_error())
        assert np.array_equal(got[0], want), attrs


def test_decline_and_failure_contract(ctx_auto):
    ctx = ctx_auto
    x = np.zeros((1, 4, 5, 5), np.float32)
    w = np.zeros((4, 4, 3, 3), np.float32)
    # not claimed: a clean decline
    assert dispatch(ctx, "Softplus", [x]) is None
    # unknown attribute: decline, never ignore
    assert dispatch(ctx, "Conv", [x, w], {"made_up_attribute": 3}) is None
    # fused activation outside what the optimizer emits
    assert dispatch(ctx, "Conv", [x, w], {"activation": "gelu"}) is None
    # malformed quantised operands decline (the CPU operator owns the typed error)
    bad = np.full((1, 4, 5, 5), np.nan, np.float32)
    assert dispatch(ctx, "ConvInteger", [bad, w]) is None
    assert dispatch(ctx, "QuantizeLinear", [x, np.float32([0.0])]) is None
    c = ctx.cache_counters()
    assert c["declines"] >= 5 and c["failures"] == 0


def test_device_resident_chain_and_counters():
    """Conv -> Relu -> Conv with the intermediate kept in HBM: two uploads of activations at
    most, one read-back, and the same lanes as the host-placed chain."""
    ctx = S.CudaContext(0)
    rng = np.random.default_rng(41)
    x = rng.standard_normal((2, 32, 10, 10)).astype(np.float32)
    w1 = (rng.standard_normal((64, 32, 3, 3)) * 0.06).astype(np.float32)
    w2 = (rng.standard_normal((32, 64, 1, 1)) * 0.1).astype(np.float32)
    weights = {"w1": w1, "w2": w2}
    ctx.register_weights(weights)
    n1 = Node("Conv", "c1", ["x", "w1"], ["h"], {"pads": [1, 1, 1, 1], "activation": "relu"})
    n2 = Node("Conv", "c2", ["h", "w2"], ["y"], {})
    h = S.try_cuda_dispatch_resident(n1, weights, {"x": x}, "device", ctx)
    assert isinstance(h, S.DeviceTensor) and h.shape == (2, 64, 10, 10)
    before = ctx.cache_counters()
    y = S.try_cuda_dispatch_resident(n2, weights, {"h": h}, "host", ctx)[0]
    after = ctx.cache_counters()
    assert after["uploads"] == before["uploads"], "a resident operand must not be re-uploaded"
    assert ctx.is_weight_resident("w1") and ctx.is_weight_resident("w2")
    h_host = S.try_cuda_dispatch(n1, weights, {"x": x}, ctx)[0]
    assert np.array_equal(h.read_back(), h_host)
    y_host = S.try_cuda_dispatch(n2, weights, {"h": h_host}, ctx)[0]
    assert np.array_equal(y, y_host)
    # second use of the same weights: no new weight upload
    wu = ctx.cache_counters()["weight_uploads"]
    S.try_cuda_dispatch(n2, weights, {"h": h_host}, ctx)
    assert ctx.cache_counters()["weight_uploads"] == wu
    h.release()
    ctx.close()


def test_device_tensor_alias_reserved_bytes_and_context_queries():
    """CudaDeviceTensor::alias / reserved_bytes and CudaContext::{streams_unified, cached_device_bytes,
    set_graph_capture} (oxionnx-cuda src/activation.rs:116-163, src/context.rs:384-447)."""
    ctx = S.CudaContext(0)
    rng = np.random.default_rng(5)
    a = rng.standard_normal((6, 32)).astype(np.float32)
    w = (rng.standard_normal((32, 48)) * 0.1).astype(np.float32)
    weights = {"w": w}
    ctx.register_weights(weights)
    assert ctx.streams_unified() and ctx.cached_device_bytes() == 0
    y = S.try_cuda_dispatch_resident(Node("MatMul", "mm", ["a", "w"], ["y"], {}), weights, {"a": a}, "device", ctx)
    assert isinstance(y, S.DeviceTensor) and y.shape == (6, 48) and y.reserved_bytes >= 6 * 48 * 4
    assert ctx.cached_device_bytes() >= 32 * 48 * 4  # the packed weight stays resident
    flat = y.alias((2, 144))
    assert flat is not None and flat.shape == (2, 144)
    assert y.alias((5, 5)) is None  # another element count: the reference's None
    want = y.read_back()
    y.release()  # the alias keeps the allocation alive
    assert np.array_equal(flat.read_back(), want.reshape(2, 144))
    # the alias is a usable operand
    r = S.try_cuda_dispatch_resident(Node("Relu", "r", ["t"], ["z"], {}), {}, {"t": flat}, "host", ctx)[0]
    assert np.array_equal(r, np.maximum(want, 0).reshape(2, 144))
    flat.release()
    # a channels-last rank-4 value does not alias into another order
    x = rng.standard_normal((1, 32, 4, 4)).astype(np.float32)
    wc = (rng.standard_normal((64, 32, 1, 1)) * 0.1).astype(np.float32)
    h = S.try_cuda_dispatch_resident(Node("Conv", "c", ["x", "wc"], ["h"], {}), {"wc": wc}, {"x": x}, "device", ctx)
    assert h.alias((1, 64 * 16)) is None and "channels-last" in ctx.last_error()
    h.release()
    assert not ctx.graph_capture_enabled()
    ctx.set_graph_capture(True)
    assert ctx.graph_capture_enabled()
    ctx.set_graph_capture(False)
    ctx.close()
    verify = S.CudaContext(0, verify=True, cuda_graph=True)
    assert not verify.graph_capture_enabled()  # never under shadow verification
    verify.close()


def test_shadow_verify_contract():
    """A 'wrong kernel' is simulated on the host by handing mismatching vectors to the
    comparator, as the reference's own shadow_verify tests do."""
    a = np.float32([1.0, 2.0, 3.0])
    for strict, exc in ((True, S.VerifyMismatch), (False, S.OnnxError)):
        ctx = S.CudaContext(0, verify=True, strict=strict)
        ctx.shadow_verify("Conv", a, a + np.float32(5e-5))
        with pytest.raises(exc) as ei:
            ctx.shadow_verify("Conv", a, a + np.float32(0.5))
        assert S.is_verify_mismatch(str(ei.value))
        ctx.close()
