"""Times one contraction layer through the planned session (the tensor-core kernel in isolation).

  python -m oxionnx_b200.layer_bench f32|i8 N C H W OC K STRIDE PAD [ITERS]
  python -m oxionnx_b200.layer_bench dql ROWS COLS [ITERS]      (DynamicQuantizeLinear of a [ROWS, COLS] activation)

The layer sits between two cheap glue nodes so that its input and output are device-resident
activations, exactly as inside a network.  Prints the kernel chosen by the planner, its best
CUDA-event time and the algorithmic rate.  Used for the ncu captures summarised under profiles/.
"""
import sys

import numpy as np

from .graph import Graph, Node
from .session import Session


def build(kind, n, c, h, w, oc, k, stride, pad):
    rng = np.random.default_rng(0)
    if kind == "f32":
        weights = {"w": (rng.standard_normal((oc, c, k, k)) * 0.05).astype(np.float32), "b": rng.standard_normal(oc).astype(np.float32)}
        nodes = [Node("Relu", "pre", ["x"], ["x1"], {}),
                 Node("Conv", "conv", ["x1", "w", "b"], ["y"], {"strides": [stride, stride], "pads": [pad] * 4, "activation": "relu"}),
                 Node("GlobalAveragePool", "gap", ["y"], ["z"], {})]
        x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    else:
        weights = {"w": rng.integers(-127, 128, (oc, c, k, k)).astype(np.float32), "ws": rng.uniform(0.001, 0.01, oc).astype(np.float32),
                   "wz": np.zeros(oc, np.float32), "b": rng.integers(-1000, 1000, oc).astype(np.float32), "xs": np.float32([0.02]),
                   "z0": np.float32([0]), "ys": np.float32([0.5]), "qs": np.float32([0.02])}
        nodes = [Node("QuantizeLinear", "q", ["x", "qs", "z0"], ["xq"], {}),
                 Node("QLinearConv", "conv", ["xq", "xs", "z0", "w", "ws", "wz", "ys", "z0", "b"], ["yq"],
                      {"strides": [stride, stride], "pads": [pad] * 4}),
                 Node("Relu", "r", ["yq"], ["yr"], {}),
                 Node("DequantizeLinear", "dq", ["yr", "ys", "z0"], ["yd"], {}),
                 Node("GlobalAveragePool", "gap", ["yd"], ["z"], {})]
        x = np.abs(rng.standard_normal((n, c, h, w))).astype(np.float32)
    return Graph(nodes=nodes, input_names=["x"], output_names=["z"]), weights, x


def main_dql(argv):
    rows, cols = int(argv[0]), int(argv[1])
    iters = int(argv[2]) if len(argv) > 2 else 5
    nodes = [Node("Relu", "pre", ["x"], ["x1"], {}), Node("DynamicQuantizeLinear", "dq", ["x1"], ["y", "s", "z"], {})]
    graph = Graph(nodes=nodes, input_names=["x"], output_names=["s", "z"])
    x = np.random.default_rng(0).standard_normal((rows, cols)).astype(np.float32)
    sess = Session.builder().with_profiling(True).build_from_graph(graph, {})
    sess.upload({"x": x})
    for _ in range(3):
        sess.run_resident(1)
    best = 1e9
    for _ in range(iters):
        sess.run_resident(1)
        best = min([best] + [s["ms"] for s in sess.steps() if s["node"] == "dq" and s["ms"] >= 0])
    n = rows * cols
    print(f"dynamic_quantize_linear [{rows}, {cols}]: best {best * 1000:.1f} us (two launches)  {9 * n / (best / 1e3) / 1e12:.2f} TB/s at 9 bytes per lane")
    sess.close()


def main(argv):
    kind = argv[0]
    if kind == "dql":
        return main_dql(argv[1:])
    n, c, h, w, oc, k, stride, pad = [int(a) for a in argv[1:9]]
    iters = int(argv[9]) if len(argv) > 9 else 5
    graph, weights, x = build(kind, n, c, h, w, oc, k, stride, pad)
    sess = Session.builder().with_profiling(True).build_from_graph(graph, weights)
    sess.upload({"x": x})
    for _ in range(3):
        sess.run_resident(1)
    best, desc, work = 1e9, "", 0.0
    for _ in range(iters):
        sess.run_resident(1)
        for s in sess.steps():
            if s["node"] == "conv" and not s["work_is_bytes"] and s["ms"] >= 0 and s["ms"] < best:
                best, desc, work = s["ms"], s["kernel"], s["work"]
    print(f"{desc}: best {best * 1000:.1f} us  {work / (best / 1e3) / 1e12:.1f} T/s")
    sess.close()


if __name__ == "__main__":
    main(sys.argv[1:])
