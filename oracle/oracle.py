"""ctypes front end of the CPU oracle (oracle/oxi_oracle.cpp).

TEST INFRASTRUCTURE ONLY.  Tensors are numpy float32 arrays (the reference's f32-lane
convention); a node is any object with .op, .inputs, .outputs and .attrs (a dict whose
values are int, float, str, list[int] or list[float]).
"""
import ctypes
import os

import numpy as np

from . import build as _build

MAX_RANK = 8


class OracleError(RuntimeError):
    """Raised with the reference's error class name (ShapeMismatch, InvalidModel, ...)."""

    def __init__(self, code, message):
        kinds = {-1: "ShapeMismatch", -2: "InvalidModel", -3: "Unsupported", -4: "Internal"}
        self.kind = kinds.get(code, "Internal")
        super().__init__(f"{self.kind}: {message}")


class _Tensor(ctypes.Structure):
    _fields_ = [("data", ctypes.POINTER(ctypes.c_float)), ("shape", ctypes.c_int64 * MAX_RANK), ("rank", ctypes.c_int32),
                ("present", ctypes.c_int32), ("len", ctypes.c_int64), ("dtype", ctypes.c_int32)]

DT_UNTYPED, DT_U8, DT_I8 = 0, 1, 2


class _Attr(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("kind", ctypes.c_int32), ("i", ctypes.c_int64), ("f", ctypes.c_float),
                ("s", ctypes.c_char_p), ("ints", ctypes.POINTER(ctypes.c_int64)), ("floats", ctypes.POINTER(ctypes.c_float)),
                ("len", ctypes.c_int64)]


_lib = None


def _load():
    global _lib
    if _lib is None:
        path = _build.LIB if os.path.exists(_build.LIB) else _build.build()
        try:
            path = _build.build()
        except Exception:  # no compiler on this host: use the prebuilt library
            if not os.path.exists(path):
                raise
        lib = ctypes.CDLL(path)
        lib.oxo_run_node.argtypes = [ctypes.c_char_p, ctypes.POINTER(_Tensor), ctypes.c_int32, ctypes.POINTER(_Attr), ctypes.c_int32,
                                     ctypes.POINTER(_Tensor), ctypes.c_int32]
        lib.oxo_run_node.restype = ctypes.c_int
        lib.oxo_free_tensor.argtypes = [ctypes.POINTER(_Tensor)]
        lib.oxo_last_error.restype = ctypes.c_char_p
        lib.oxo_set_threads.argtypes = [ctypes.c_int32]
        lib.oxo_get_threads.restype = ctypes.c_int32
        lib.oxo_set_float_accum.argtypes = [ctypes.c_int32]
        lib.oxo_round_ties_even_f64.argtypes = [ctypes.c_double]
        lib.oxo_round_ties_even_f64.restype = ctypes.c_double
        lib.oxo_round_ties_even_f32.argtypes = [ctypes.c_float]
        lib.oxo_round_ties_even_f32.restype = ctypes.c_float
        lib.oxo_requantize.argtypes = [ctypes.c_int64, ctypes.c_float, ctypes.c_int32, ctypes.c_int64, ctypes.c_int64]
        lib.oxo_requantize.restype = ctypes.c_float
        _lib = lib
    return _lib


def set_threads(n):
    _load().oxo_set_threads(int(n))


def get_threads():
    return int(_load().oxo_get_threads())


def set_float_accum(mode):
    """0: f64 accumulation rounded once; 1: sequential f32 accumulation."""
    _load().oxo_set_float_accum(int(mode))


def round_ties_even_f64(v):
    return float(_load().oxo_round_ties_even_f64(float(v)))


def round_ties_even_f32(v):
    return float(_load().oxo_round_ties_even_f32(float(v)))


def requantize(acc, combined, zero_point, lo, hi):
    return float(_load().oxo_requantize(int(acc), float(combined), int(zero_point), int(lo), int(hi)))


def _pack_attrs(attrs):
    keep = []
    items = list((attrs or {}).items())
    arr = (_Attr * max(len(items), 1))()
    for idx, (name, value) in enumerate(items):
        a = arr[idx]
        a.name = name.encode()
        if isinstance(value, bool):
            a.kind, a.i = 0, int(value)
        elif isinstance(value, (int, np.integer)):
            a.kind, a.i = 0, int(value)
        elif isinstance(value, (float, np.floating)):
            a.kind, a.f = 1, float(value)
        elif isinstance(value, str):
            a.kind, a.s = 2, value.encode()
        elif isinstance(value, (list, tuple, np.ndarray)):
            vals = list(value)
            if all(isinstance(v, (int, np.integer)) for v in vals):
                buf = (ctypes.c_int64 * max(len(vals), 1))(*[int(v) for v in vals])
                a.kind, a.ints, a.len = 3, buf, len(vals)
            else:
                buf = (ctypes.c_float * max(len(vals), 1))(*[float(v) for v in vals])
                a.kind, a.floats, a.len = 4, buf, len(vals)
            keep.append(buf)
        else:
            raise TypeError(f"attribute {name!r}: unsupported value type {type(value)}")
    return arr, len(items), keep


def run_node(op, inputs, attrs=None, n_outputs=1):
    """Execute one operator.  `inputs` is a list of arrays (None = omitted optional input); a uint8 or int8 array
    is a typed tensor (its lanes are widened to f32, its declared type travels with it, as on the reference's
    execute_typed path), anything else is plain f32 lanes.  Returns a list of n_outputs float32 arrays."""
    lib = _load()
    n_in = len(inputs)
    tin = (_Tensor * max(n_in, 1))()
    keep = []
    for i, x in enumerate(inputs):
        if x is None:
            tin[i].present = 0
            continue
        declared = getattr(x, "dtype", None)
        tin[i].dtype = DT_U8 if declared == np.uint8 else (DT_I8 if declared == np.int8 else DT_UNTYPED)
        arr = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
        keep.append(arr)
        if arr.ndim > MAX_RANK:
            raise ValueError("rank too large for the oracle")
        tin[i].data = arr.ctypes.data_as(ctypes.POINTER(ctypes.c_float))
        tin[i].rank = arr.ndim
        for d, s in enumerate(arr.shape):
            tin[i].shape[d] = s
        tin[i].present = 1
        tin[i].len = arr.size
    carr, n_attr, keep2 = _pack_attrs(attrs)
    tout = (_Tensor * max(n_outputs, 1))()
    rc = lib.oxo_run_node(op.encode(), tin, n_in, carr, n_attr, tout, n_outputs)
    if rc != 0:
        raise OracleError(rc, lib.oxo_last_error().decode())
    outs = []
    for i in range(n_outputs):
        t = tout[i]
        if not t.present:
            outs.append(None)
            continue
        shape = tuple(t.shape[d] for d in range(t.rank))
        n = int(t.len)
        a = np.ctypeslib.as_array(t.data, shape=(max(n, 1),))[:n].copy().reshape(shape)
        outs.append(a)
        lib.oxo_free_tensor(ctypes.byref(t))
    del keep, keep2
    return outs


def run_graph(graph, weights, feeds, keep_all=True):
    """Execute `graph.nodes` in order (they must be topologically sorted), the way
    Session::run does with OptLevel::None (src/session/run/sequential.rs:505).  Returns a
    dict holding every value (feeds, intermediates, outputs) when keep_all, else only the
    graph outputs.  uint8 / int8 weights and feeds stay typed tensors (run_typed: the declared type of a
    y_zero_point then fixes the saturation range); every other array is f32 lanes."""
    def lanes(v):
        v = np.asarray(v)
        return v if v.dtype in (np.uint8, np.int8) else v.astype(np.float32)
    state = {k: lanes(v) for k, v in weights.items()}
    state.update({k: lanes(v) for k, v in feeds.items()})
    for node in graph.nodes:
        ins = [state[name] if name else None for name in node.inputs]
        outs = run_node(node.op, ins, node.attrs, n_outputs=len(node.outputs))
        for name, val in zip(node.outputs, outs):
            if name:
                state[name] = val
    if keep_all:
        return state
    return {name: state[name] for name in graph.output_names}
