"""ONNX files in and out of the package.

`write_onnx(graph, weights, inputs, path)` serialises one of the package's graphs (or any hand-built
graph) as a standard ONNX ModelProto, with no dependency beyond numpy: the protobuf wire format is
written directly.  `Model` wraps the C-ABI loader (oxb200_model_*): it parses a model file, runs the
reference's fusion passes for this path (Conv+BatchNormalization, Conv+Relu/Clip, the
InstanceNorm-style chain, MatMul+Add, Conv+Add+Relu, Mul(x, Sigmoid(x))) and hands the result to a
session, which is what `Session::from_file` does in the reference (root crate
src/session/loading.rs:181, oxionnx-proto src/model.rs:45).
"""
import ctypes
import struct
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import _ffi
from .graph import Graph, Node

# TensorProto.DataType
ONNX_DTYPE = {np.dtype(np.float32): 1, np.dtype(np.uint8): 2, np.dtype(np.int8): 3, np.dtype(np.uint16): 4, np.dtype(np.int16): 5,
              np.dtype(np.int32): 6, np.dtype(np.int64): 7, np.dtype(np.bool_): 9, np.dtype(np.float16): 10, np.dtype(np.float64): 11}


# ---- protobuf wire format ---------------------------------------------------------------------
def _varint(v: int) -> bytes:
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _key(field: int, wire: int) -> bytes:
    return _varint((field << 3) | wire)


def _len(field: int, payload: bytes) -> bytes:
    return _key(field, 2) + _varint(len(payload)) + payload


def _int(field: int, v: int) -> bytes:
    return _key(field, 0) + _varint(int(v))


def _str(field: int, s: str) -> bytes:
    return _len(field, s.encode())


def _tensor(name: str, array: np.ndarray) -> bytes:
    a = np.asarray(array)
    if not a.flags.c_contiguous:
        a = np.ascontiguousarray(a)
    if a.dtype not in ONNX_DTYPE:
        raise TypeError(f"initializer {name!r}: element type {a.dtype} has no ONNX code here")
    body = b"".join(_int(1, d) for d in a.shape) + _int(2, ONNX_DTYPE[a.dtype]) + _str(8, name) + _len(9, a.tobytes())
    return body


def _attr(name: str, value) -> bytes:
    body = _str(1, name)
    if isinstance(value, (bool, int, np.integer)):
        body += _int(3, int(value)) + _int(20, 2)
    elif isinstance(value, (float, np.floating)):
        body += _key(2, 5) + struct.pack("<f", float(value)) + _int(20, 1)
    elif isinstance(value, str):
        body += _len(4, value.encode()) + _int(20, 3)
    elif isinstance(value, (list, tuple, np.ndarray)):
        vals = list(value)
        if all(isinstance(v, (int, np.integer)) and not isinstance(v, bool) for v in vals):
            body += _len(8, b"".join(_varint(int(v)) for v in vals)) + _int(20, 7)
        else:
            body += _len(7, b"".join(struct.pack("<f", float(v)) for v in vals)) + _int(20, 6)
    else:
        raise TypeError(f"attribute {name!r}: unsupported value type {type(value)}")
    return body


def _value_info(name: str, shape: Sequence, dtype) -> bytes:
    dims = b""
    for d in shape:
        if isinstance(d, str) or d is None or (isinstance(d, (int, np.integer)) and d < 0):
            dims += _len(1, _str(2, d if isinstance(d, str) else "N"))  # dim_param
        else:
            dims += _len(1, _int(1, int(d)))  # dim_value
    tensor_type = _int(1, ONNX_DTYPE[np.dtype(dtype)]) + _len(2, dims)
    return _str(1, name) + _len(2, _len(1, tensor_type))


def write_onnx(graph: Graph, weights: Dict[str, np.ndarray], inputs: Dict[str, Tuple[Sequence, object]], path: Optional[str] = None,
               outputs: Optional[Dict[str, Tuple[Sequence, object]]] = None, opset: int = 13, list_initializers_as_inputs: bool = False) -> bytes:
    """Serialises `graph` as an ONNX model.  `inputs` maps each graph input to (shape, numpy dtype); a dimension
    given as a string, None or a negative number becomes a symbolic dimension.  Initializers keep the element type
    of the arrays in `weights` (uint8 / int8 zero points stay typed).  Returns the bytes and, when `path` is given,
    writes them there."""
    g = b""
    for node in graph.nodes:
        body = b"".join(_str(1, s) for s in node.inputs) + b"".join(_str(2, s) for s in node.outputs)
        body += _str(3, node.name or "") + _str(4, node.op)
        body += b"".join(_len(5, _attr(k, v)) for k, v in (node.attrs or {}).items())
        g += _len(1, body)
    g += _str(2, "oxionnx_b200_graph")
    for name, arr in weights.items():
        g += _len(5, _tensor(name, np.asarray(arr)))
    for name in graph.input_names:
        shape, dtype = inputs[name]
        g += _len(11, _value_info(name, shape, dtype))
    if list_initializers_as_inputs:  # the pre-IR-4 convention some exporters still follow
        for name, arr in weights.items():
            g += _len(11, _value_info(name, np.asarray(arr).shape, np.asarray(arr).dtype))
    for name in graph.output_names:
        shape, dtype = (outputs or {}).get(name, ((), np.float32))
        g += _len(12, _value_info(name, shape, dtype))
    model = _int(1, 8) + _str(2, "oxionnx_b200") + _len(7, g) + _len(8, _str(1, "") + _int(2, opset))
    if path:
        with open(path, "wb") as fh:
            fh.write(model)
    return model


# ---- loader / optimizer over the C ABI -----------------------------------------------------------
class ModelError(RuntimeError):
    pass


class Model:
    """A parsed ONNX model (oxb200_model)."""

    def __init__(self, handle):
        self.handle = handle

    @classmethod
    def from_bytes(cls, data: bytes) -> "Model":
        lib = _ffi.lib()
        h = ctypes.c_void_p()
        buf = (ctypes.c_uint8 * max(len(data), 1)).from_buffer_copy(data if data else b"\0")
        st = lib.oxb200_model_load(buf, len(data), ctypes.byref(h))
        if st != _ffi.OK_HOST:
            raise ModelError(f"{_ffi.STATUS_NAMES.get(st, st)}: {lib.oxb200_last_error(None).decode()}")
        return cls(h)

    @classmethod
    def from_file(cls, path: str) -> "Model":
        lib = _ffi.lib()
        h = ctypes.c_void_p()
        st = lib.oxb200_model_load_file(path.encode(), ctypes.byref(h))
        if st != _ffi.OK_HOST:
            raise ModelError(f"{_ffi.STATUS_NAMES.get(st, st)}: {lib.oxb200_last_error(None).decode()}")
        return cls(h)

    def close(self):
        if self.handle:
            _ffi.lib().oxb200_model_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def optimize(self, level: int = 1) -> int:
        """The reference's fusion passes for this path, in its order; returns the number of nodes fused away."""
        removed = ctypes.c_uint32()
        st = _ffi.lib().oxb200_model_optimize(self.handle, level, ctypes.byref(removed))
        if st != _ffi.OK_HOST:
            raise ModelError(_ffi.lib().oxb200_last_error(None).decode())
        return int(removed.value)

    def run_pass(self, name: str) -> int:
        removed = ctypes.c_uint32()
        st = _ffi.lib().oxb200_model_run_pass(self.handle, name.encode(), ctypes.byref(removed))
        if st != _ffi.OK_HOST:
            raise ModelError(_ffi.lib().oxb200_last_error(None).decode())
        return int(removed.value)

    def nodes(self) -> List[Node]:
        lib = _ffi.lib()
        out = []
        for i in range(lib.oxb200_model_node_count(self.handle)):
            c = _ffi.CNode()
            lib.oxb200_model_node(self.handle, i, ctypes.byref(c))
            attrs = {}
            for k in range(c.n_attrs):
                a = c.attrs[k]
                name = a.name.decode()
                if a.kind == 0:
                    attrs[name] = int(a.i)
                elif a.kind == 1:
                    attrs[name] = float(a.f)
                elif a.kind == 2:
                    attrs[name] = a.s.decode()
                elif a.kind == 3:
                    attrs[name] = [int(a.ints[j]) for j in range(a.len)]
                else:
                    attrs[name] = [float(a.floats[j]) for j in range(a.len)]
            out.append(Node(op=c.op_type.decode(), name=c.name.decode(), inputs=[c.inputs[j].decode() for j in range(c.n_inputs)],
                            outputs=[c.outputs[j].decode() for j in range(c.n_outputs)], attrs=attrs))
        return out

    def inputs(self) -> List[Tuple[str, tuple, int]]:
        """(name, shape with None for symbolic dimensions, OXB200_DT_* code or -1)."""
        lib = _ffi.lib()
        out = []
        for i in range(lib.oxb200_model_input_count(self.handle)):
            v = _ffi.ValueInfo()
            lib.oxb200_model_input(self.handle, i, ctypes.byref(v))
            shape = tuple(None if v.shape[d] == 0xFFFFFFFFFFFFFFFF else int(v.shape[d]) for d in range(v.rank))
            out.append((v.name.decode(), shape, int(v.dtype)))
        return out

    def output_names(self) -> List[str]:
        lib = _ffi.lib()
        return [lib.oxb200_model_output_name(self.handle, i).decode() for i in range(lib.oxb200_model_output_count(self.handle))]

    def initializers(self) -> Dict[str, Tuple[np.ndarray, int]]:
        """name -> (f32 lanes in the tensor's shape, declared OXB200_DT_* code)."""
        lib = _ffi.lib()
        out = {}
        for i in range(lib.oxb200_model_initializer_count(self.handle)):
            o = _ffi.Operand()
            lib.oxb200_model_initializer(self.handle, i, ctypes.byref(o))
            shape = tuple(int(o.shape[d]) for d in range(o.rank))
            n = int(o.len)
            data = np.ctypeslib.as_array(o.lanes, shape=(max(n, 1),))[:n].copy().reshape(shape) if n else np.zeros(shape, np.float32)
            out[o.name.decode()] = (data, int(o.dtype))
        return out

    def to_graph(self) -> Tuple[Graph, Dict[str, np.ndarray]]:
        """The model as one of the package's graphs plus its weights (declared 8-bit types restored), e.g. to run it
        through the CPU oracle."""
        weights = {}
        for name, (data, code) in self.initializers().items():
            weights[name] = data.astype(np.uint8) if code == _ffi.DT_U8 else (data.astype(np.int8) if code == _ffi.DT_I8 else data)
        return Graph(nodes=self.nodes(), input_names=[n for n, _, _ in self.inputs()], output_names=self.output_names()), weights


def plan_model(ctx, model: Model, input_shapes: Optional[Dict[str, Sequence[int]]] = None):
    """oxb200_session_plan_model: the model's initializers become the context's weights, its graph is planned."""
    lib = _ffi.lib()
    keep = _ffi.Keep()
    items = list((input_shapes or {}).items())
    infos = keep.add((_ffi.ValueInfo * max(len(items), 1))())
    for i, (name, shape) in enumerate(items):
        infos[i].name = name.encode()
        infos[i].shape = keep.add((ctypes.c_uint64 * max(len(shape), 1))(*[int(d) for d in shape]))
        infos[i].rank = len(shape)
    st = lib.oxb200_session_plan_model(ctx.handle, model.handle, infos, len(items))
    return st, ctx.last_error() if st not in (_ffi.OK_HOST, _ffi.OK_DEVICE) else ""
