"""Host-side mirror of the reference's interface for the hot path, over the C ABI.

Names and argument meaning follow the reference so that tests read like the reference's own:

  Session.builder().build_from_graph(graph, weights)   root crate src/session/builder.rs:336
  Session.run(feeds) -> {name: tensor}                  root crate src/session/run/entry.rs:92
  CudaContext.try_new()                                 oxionnx-cuda src/context.rs:467
  try_cuda_dispatch_resident(node, weights, intermediates, placement, ctx)
                                                        oxionnx-cuda src/lib.rs:561
  is_supported_op / accepts_resident_slot               oxionnx-cuda src/lib.rs:217,419
  OpPlacement / decide_placement                        root crate src/execution_providers.rs:111,352

Errors keep the reference's three-way meaning: `Declined` (Ok(None): let the next provider
try), `OnnxError` (Err: log and fall back) and `VerifyMismatch` (proved wrong: fail the run).
"""
import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional

import numpy as np

from . import _ffi
from .graph import Graph, Node


class OnnxError(RuntimeError):
    """A failed dispatch or run (the Err arm)."""


class Declined(Exception):
    """The provider does not take this node (the Ok(None) arm); not an error."""


class VerifyMismatch(OnnxError):
    """The device result was proved wrong against the shadow check under strict mode."""


def is_supported_op(op: str) -> bool:
    return bool(_ffi.lib().oxb200_is_supported_op(op.encode()))


def accepts_resident_slot(op: str, slot: int) -> bool:
    return bool(_ffi.lib().oxb200_accepts_resident_slot(op.encode(), slot))


def is_verify_mismatch(message: str) -> bool:
    return bool(_ffi.lib().oxb200_is_verify_mismatch(message.encode()))


def env_truthy(value: Optional[str]) -> bool:
    return bool(_ffi.lib().oxb200_env_truthy(None if value is None else value.encode()))


def device_count() -> int:
    return int(_ffi.lib().oxb200_device_count())


@dataclass
class OpPlacement:
    """OpPlacement {CpuOnly, Auto{gpu_threshold_bytes}, Manual(map)}."""
    policy: str = "auto"
    gpu_threshold_bytes: int = 4096
    manual: Optional[Dict[str, str]] = None  # op name -> "cpu" | "cuda"

    def decide(self, op: str, output_bytes: int) -> bool:
        """True when the node goes to this provider (decide_placement)."""
        code = {"cpu_only": 0, "auto": 1, "manual": 2}[self.policy]
        pin = 0
        if self.manual is not None and op in self.manual:
            pin = 2 if self.manual[op] == "cuda" else 1
        return bool(_ffi.lib().oxb200_decide_placement(code, self.gpu_threshold_bytes, pin, op.encode(), output_bytes))


def _raise_for(status, message):
    if status in (_ffi.OK_HOST, _ffi.OK_DEVICE):
        return
    if status == _ffi.DECLINED:
        raise Declined(message)
    if status == _ffi.VERIFY_MISMATCH:
        raise VerifyMismatch(message)
    raise OnnxError(message)


class DeviceTensor:
    """CudaDeviceTensor: a value that stays in HBM between dispatches."""

    def __init__(self, ctx, handle):
        self._ctx = ctx
        self.handle = handle

    @property
    def shape(self):
        shape = (ctypes.c_uint64 * _ffi.MAX_RANK)()
        rank = ctypes.c_uint32()
        n = ctypes.c_uint64()
        _ffi.lib().oxb200_tensor_shape(self.handle, shape, ctypes.byref(rank), ctypes.byref(n))
        return tuple(int(shape[d]) for d in range(rank.value))

    def read_back(self) -> np.ndarray:
        shape = self.shape
        n = int(np.prod(shape)) if len(shape) else 1
        buf = np.empty(max(n, 1), np.float32)
        st = _ffi.lib().oxb200_tensor_read_back(self._ctx.handle, self.handle, buf.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), buf.size)
        _raise_for(st, self._ctx.last_error())
        return buf[:n].reshape(shape).copy()

    def alias(self, shape) -> Optional["DeviceTensor"]:
        """CudaDeviceTensor::alias: the same allocation under another shape of the same element count, or None."""
        arr = (ctypes.c_uint64 * max(len(shape), 1))(*[int(d) for d in shape])
        out = ctypes.c_void_p()
        st = _ffi.lib().oxb200_tensor_alias(self._ctx.handle, self.handle, arr, len(shape), ctypes.byref(out))
        if st == _ffi.DECLINED:
            return None
        _raise_for(st, self._ctx.last_error())
        return DeviceTensor(self._ctx, out)

    @property
    def reserved_bytes(self) -> int:
        return int(_ffi.lib().oxb200_tensor_reserved_bytes(self.handle))

    def release(self):
        if self.handle:
            _ffi.lib().oxb200_tensor_release(self._ctx.handle, self.handle)
            self.handle = None


class CudaContext:
    """One device, one stream, session-lifetime weight residency."""

    def __init__(self, device: int = 0, *, verify=False, strict=False, residency=True, kernel_path="auto", keep_intermediates=False,
                 profile=False, cuda_graph=False, requant_f64=False, split_k_max=0, cta_pairs="auto", float_precision="tf32"):
        cfg = _ffi.Config()
        cfg.struct_size = ctypes.sizeof(_ffi.Config)
        cfg.verify, cfg.strict, cfg.residency = int(verify), int(strict), int(residency)
        cfg.kernel_path = 1 if kernel_path == "direct" else 0
        cfg.keep_intermediates = int(keep_intermediates)
        cfg.profile = int(profile)
        cfg.cuda_graph = int(cuda_graph)
        cfg.requant_f64 = int(requant_f64)  # False/0 auto, True/1 two-pass f64, 2 one-FMA without the packed saturation
        cfg.split_k_max = int(split_k_max)
        cfg.cta_pairs = {"auto": 0, "never": 1, "always": 2}[cta_pairs]
        # operand type of the float contractions on the tensor cores (f32 accumulation and f32 results in every case)
        cfg.float_precision = {"tf32": 0, "f16": 1, "bf16": 2}[float_precision]
        h = ctypes.c_void_p()
        st = _ffi.lib().oxb200_ctx_create(device, ctypes.byref(cfg), ctypes.byref(h))
        if st != _ffi.OK_HOST:
            raise OnnxError(_ffi.lib().oxb200_last_error(None).decode())
        self.handle = h
        self.device = device
        self._weights = {}

    @classmethod
    def try_new(cls, device: int = 0, **kw):
        """None when no usable device exists (CudaContext::try_new returns Option)."""
        try:
            return cls(device, **kw)
        except OnnxError:
            return None

    def last_error(self) -> str:
        return _ffi.lib().oxb200_last_error(self.handle).decode()

    def close(self):
        if self.handle:
            _ffi.lib().oxb200_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def register_weights(self, weights: Dict[str, np.ndarray]):
        """Initializers as f32 lanes.  An array that arrives as uint8 / int8 keeps that declared type beside its
        lanes (an ONNX initializer's data_type), which makes a quantised operator saturate exactly to it; a float16
        array is declared FLOAT16, which makes the contraction it feeds run with f16 operands."""
        for name, w in weights.items():
            declared = _ffi.TYPED.get(np.asarray(w).dtype, _ffi.DT_F16 if np.asarray(w).dtype == np.float16 else _ffi.DT_F32)
            a = np.ascontiguousarray(np.asarray(w, dtype=np.float32))
            shape = (ctypes.c_uint64 * max(a.ndim, 1))(*a.shape)
            st = _ffi.lib().oxb200_weight_register_typed(self.handle, name.encode(), a.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), a.size, shape,
                                                         a.ndim, declared)
            _raise_for(st, self.last_error())
            self._weights[name] = a.shape

    def is_weight_resident(self, name: str) -> bool:
        return bool(_ffi.lib().oxb200_is_weight_resident(self.handle, name.encode()))

    def cache_counters(self) -> dict:
        c = _ffi.Counters()
        _ffi.lib().oxb200_get_counters(self.handle, ctypes.byref(c))
        return c.as_dict()

    def release_device_caches(self):
        _raise_for(_ffi.lib().oxb200_release_device_caches(self.handle), self.last_error())

    def streams_unified(self) -> bool:
        return bool(_ffi.lib().oxb200_streams_unified(self.handle))

    def cached_device_bytes(self) -> int:
        return int(_ffi.lib().oxb200_cached_device_bytes(self.handle))

    def set_graph_capture(self, on: bool):
        _ffi.lib().oxb200_set_graph_capture(self.handle, int(on))

    def graph_capture_enabled(self) -> bool:
        return bool(_ffi.lib().oxb200_graph_capture_enabled(self.handle))

    def probe_tensor_peak(self, kind: str) -> float:
        """Operations per second of the tensor pipe for "i8" | "tf32" | "f16" | "bf16", measured on this device."""
        rate = ctypes.c_double()
        code = {"i8": 0, "tf32": 1, "f16": 2, "bf16": 3}[kind]
        _raise_for(_ffi.lib().oxb200_probe_tensor_peak(self.handle, code, ctypes.byref(rate)), self.last_error())
        return float(rate.value)

    def set_profiling(self, on: bool):
        """Per-node CUDA-event timing of planned runs, on or off, for the runs that follow."""
        _raise_for(_ffi.lib().oxb200_set_profile(self.handle, int(bool(on))), self.last_error())

    def shadow_verify(self, op: str, device_result: np.ndarray, cpu_result: np.ndarray):
        a = np.ascontiguousarray(device_result, dtype=np.float32).ravel()
        b = np.ascontiguousarray(cpu_result, dtype=np.float32).ravel()
        st = _ffi.lib().oxb200_shadow_verify(self.handle, op.encode(), a.ctypes.data_as(ctypes.POINTER(ctypes.c_float)),
                                             b.ctypes.data_as(ctypes.POINTER(ctypes.c_float)), min(a.size, b.size))
        _raise_for(st, self.last_error())


def try_cuda_dispatch_resident(node: Node, weights: Dict[str, np.ndarray], intermediates: Dict[str, object], placement: str,
                               ctx: CudaContext):
    """One node through the provider.  `intermediates` maps names to numpy arrays (host) or
    DeviceTensor (resident).  Returns a list of numpy arrays (placement "host"), a DeviceTensor
    (placement "device"), or None when the provider declines."""
    lib = _ffi.lib()
    keep = _ffi.Keep()
    cnode = _ffi.CNode()
    _ffi.pack_node(node, cnode, keep)
    n_in = len(node.inputs)
    ops = keep.add((_ffi.Operand * max(n_in, 1))())
    for i, name in enumerate(node.inputs):
        if not name:
            ops[i].name = b""
            continue
        if name in intermediates:
            v = intermediates[name]
            if isinstance(v, DeviceTensor):
                _ffi.pack_operand(ops[i], name, None, keep, resident=v.handle)
            else:
                _ffi.pack_operand(ops[i], name, v, keep)
        elif name in weights:
            if name in ctx._weights:
                _ffi.pack_operand(ops[i], name, None, keep)
            else:
                _ffi.pack_operand(ops[i], name, weights[name], keep)
        else:
            raise OnnxError(f"TensorNotFound: {name}")
    n_out = len(node.outputs)
    res = keep.add((_ffi.Result * max(n_out, 1))())
    cap = int(intermediates.get("__cap__", 0)) if isinstance(intermediates, dict) else 0
    bufs = []
    # generous host buffers: the output extent is not known to the caller before the dispatch
    guess = max([int(np.asarray(v).size) for v in intermediates.values() if isinstance(v, np.ndarray)] + [1])
    guess = min(max(guess * 64, 1 << 16, cap), 1 << 26)
    for i in range(n_out):
        b = np.empty(guess, np.float32)
        bufs.append(b)
        res[i].lanes = b.ctypes.data_as(ctypes.POINTER(ctypes.c_float))
        res[i].cap = b.size
    want = _ffi.PLACE_DEVICE if placement == "device" else _ffi.PLACE_HOST
    st = lib.oxb200_dispatch(ctx.handle, ctypes.byref(cnode), ops, n_in, want, res, n_out)
    if st == _ffi.DECLINED:
        return None
    _raise_for(st, ctx.last_error())
    if st == _ffi.OK_DEVICE:
        return DeviceTensor(ctx, ctypes.c_void_p(res[0].resident))
    return [_ffi.result_array(res[i], bufs[i]) if node.outputs[i] else None for i in range(n_out)]


def try_cuda_dispatch(node, weights, intermediates, ctx):
    """Host tensors in, host tensors out (oxionnx-cuda src/lib.rs:354)."""
    return try_cuda_dispatch_resident(node, weights, intermediates, "host", ctx)


class SessionBuilder:
    def __init__(self):
        self._device = 0
        self._ctx_kw = {}
        self._input_shapes = {}
        self._input_types = {}

    def with_device(self, device: int):
        self._device = device
        return self

    def with_optimization_level(self, level):
        """SessionBuilder::with_optimization_level (root crate src/session/builder/options.rs): 0 runs the nodes as
        given; from 1 on the reference's fusion passes for this path run first (Conv+BatchNormalization,
        Conv+Relu/Clip, Conv+Add+Relu, the InstanceNorm chain, MatMul+Add, x*Sigmoid(x)).  Without this call a
        graph passed to build_from_graph is run as given (it is taken to be optimised already); a model file is
        optimised at level 1."""
        self._opt_level = int(level)
        return self

    def with_kernel_path(self, path: str):
        self._ctx_kw["kernel_path"] = path
        return self

    def with_keep_intermediates(self, on=True):
        self._ctx_kw["keep_intermediates"] = on
        return self

    def with_profiling(self, on=True):
        self._ctx_kw["profile"] = on
        return self

    def with_cuda_graph(self, on=True):
        """Replay the planned step list as one CUDA graph (OXIONNX_CUDA_GRAPH; oxionnx-cuda src/graph_cache.rs)."""
        self._ctx_kw["cuda_graph"] = on
        return self

    def with_tuning(self, **kw):
        """Kernel choices of the context: requant_f64, split_k_max, cta_pairs ("auto" | "never" | "always"),
        float_precision ("tf32" | "f16" | "bf16": the operand type of float contractions)."""
        self._ctx_kw.update(kw)
        return self

    def with_verify(self, on=True):
        self._ctx_kw["verify"] = on
        return self

    def with_input_shapes(self, shapes: Dict[str, tuple]):
        self._input_shapes = dict(shapes)
        return self

    def with_input_types(self, types: Dict[str, object]):
        """Declared element types of graph inputs (TensorInfo.dtype): np.uint8 / np.int8 inputs are stored, fed and
        bound as 8-bit lanes instead of f32 lanes."""
        self._input_types = dict(types)
        return self

    def build_from_graph(self, graph: Graph, weights: Dict[str, np.ndarray]):
        level = getattr(self, "_opt_level", None)
        if level:
            # the passes live behind the model ABI: hand the graph over as ONNX bytes
            from .onnx_io import write_onnx
            missing = [n for n in graph.input_names if n not in self._input_shapes]
            if missing:
                raise OnnxError(f"optimising a graph needs the shapes of its inputs; missing: {missing}")
            types = getattr(self, "_input_types", {})
            data = write_onnx(graph, weights, {n: (self._input_shapes[n], types.get(n, np.float32)) for n in graph.input_names})
            return self.load_from_bytes(data)
        return Session(graph, weights, self._device, self._input_shapes, self._ctx_kw, getattr(self, "_input_types", None))

    def load_from_bytes(self, data: bytes):
        """SessionBuilder::load_from_bytes (src/session/loading.rs): an ONNX ModelProto held in memory."""
        from .onnx_io import Model
        level = getattr(self, "_opt_level", None)
        return Session.from_model(Model.from_bytes(data), self._device, 1 if level is None else level, self._input_shapes, **self._ctx_kw)

    def load(self, path: str):
        """SessionBuilder::load: an ONNX file."""
        from .onnx_io import Model
        level = getattr(self, "_opt_level", None)
        return Session.from_model(Model.from_file(path), self._device, 1 if level is None else level, self._input_shapes, **self._ctx_kw)


class Session:
    """A graph planned once and run device-resident: every intermediate stays in HBM."""

    @staticmethod
    def builder() -> SessionBuilder:
        return SessionBuilder()

    def __init__(self, graph, weights, device, input_shapes, ctx_kw, input_types=None):
        self.graph = graph
        self.ctx = CudaContext(device, **ctx_kw)
        self.ctx.register_weights(weights)
        self._input_shapes = dict(input_shapes)
        self._input_types = dict(input_types or {})  # name -> np.uint8 / np.int8 for inputs declared 8-bit
        self._planned_for = None
        self._out_bufs = None

    @classmethod
    def from_file(cls, path: str, device: int = 0, optimization_level: int = 1, input_shapes: Optional[Dict[str, tuple]] = None, **ctx_kw):
        """Session::from_file (root crate src/session/loading.rs:181): parses the ONNX file, runs the reference's
        fusion passes for this path, registers the initializers (with their declared element types) as the context's
        weights and plans the graph at the first run.  `input_shapes` gives the concrete shape of every input that
        has a symbolic dimension."""
        from .onnx_io import Model
        model = Model.from_file(path)
        return cls.from_model(model, device, optimization_level, input_shapes, **ctx_kw)

    @classmethod
    def from_model(cls, model, device: int = 0, optimization_level: int = 1, input_shapes: Optional[Dict[str, tuple]] = None, **ctx_kw):
        if optimization_level > 0:
            model.optimize(optimization_level)
        graph = Graph(nodes=model.nodes(), input_names=[n for n, _, _ in model.inputs()], output_names=model.output_names())
        self = cls.__new__(cls)
        self.graph = graph
        self.ctx = CudaContext(device, **ctx_kw)
        self._model = model
        self._input_shapes = dict(input_shapes or {})
        for name, shape, _ in model.inputs():
            if name not in self._input_shapes and all(d is not None for d in shape):
                self._input_shapes[name] = tuple(shape)
        self._input_types = {name: (np.uint8 if code == _ffi.DT_U8 else np.int8) for name, _, code in model.inputs() if code in (_ffi.DT_U8, _ffi.DT_I8)}
        self._planned_for = None
        self._out_bufs = None
        return self

    def _plan(self, shapes):
        if getattr(self, "_model", None) is not None:
            from .onnx_io import plan_model
            st, msg = plan_model(self.ctx, self._model, shapes)
            _raise_for(st, msg)
            self._planned_for = {k: tuple(v) for k, v in shapes.items()}
            self._out_bufs = None
            return
        lib = _ffi.lib()
        keep = _ffi.Keep()
        nodes = keep.add((_ffi.CNode * max(len(self.graph.nodes), 1))())
        for i, n in enumerate(self.graph.nodes):
            _ffi.pack_node(n, nodes[i], keep)
        ins = keep.add((_ffi.ValueInfo * max(len(self.graph.input_names), 1))())
        for i, name in enumerate(self.graph.input_names):
            ins[i].name = name.encode()
            sh = shapes[name]
            ins[i].shape = keep.add((ctypes.c_uint64 * max(len(sh), 1))(*sh))
            ins[i].rank = len(sh)
            ins[i].dtype = _ffi.TYPED.get(np.dtype(self._input_types[name]), _ffi.DT_F32) if name in self._input_types else _ffi.DT_F32
        outs = keep.add((ctypes.c_char_p * max(len(self.graph.output_names), 1))(*[s.encode() for s in self.graph.output_names]))
        st = lib.oxb200_session_plan(self.ctx.handle, nodes, len(self.graph.nodes), ins, len(self.graph.input_names), outs,
                                     len(self.graph.output_names))
        _raise_for(st, self.ctx.last_error())
        self._planned_for = {k: tuple(v) for k, v in shapes.items()}
        self._out_bufs = None

    def ensure_planned(self, feeds=None):
        shapes = dict(self._input_shapes)
        if feeds is not None:
            shapes.update({k: tuple(np.asarray(v).shape) for k, v in feeds.items()})
            if self._planned_for is None:  # a feed that arrives as 8-bit lanes declares its input 8-bit
                for k, v in feeds.items():
                    if isinstance(v, np.ndarray) and v.dtype in _ffi.TYPED:
                        self._input_types.setdefault(k, v.dtype)
        if self._planned_for != {k: tuple(shapes[k]) for k in self.graph.input_names}:
            self._plan({k: tuple(shapes[k]) for k in self.graph.input_names})

    def _operands(self, feeds, keep):
        ops = keep.add((_ffi.Operand * max(len(self.graph.input_names), 1))())
        for i, name in enumerate(self.graph.input_names):
            if name not in feeds:
                raise OnnxError(f"TensorNotFound: missing feed '{name}'")
            _ffi.pack_operand(ops[i], name, feeds[name], keep)
        return ops

    def _results(self, keep, probe=True):
        lib = _ffi.lib()
        n_out = len(self.graph.output_names)
        res = keep.add((_ffi.Result * max(n_out, 1))())
        if self._out_bufs is None:
            # learn the output extents from the plan
            self._out_bufs = []
            for name in self.graph.output_names:
                r = _ffi.Result()
                st = lib.oxb200_fetch_value(self.ctx.handle, name.encode(), ctypes.byref(r))
                _raise_for(st, self.ctx.last_error())
                self._out_bufs.append(np.empty(max(int(r.len), 1), np.float32))
        for i, b in enumerate(self._out_bufs):
            res[i].lanes = b.ctypes.data_as(ctypes.POINTER(ctypes.c_float))
            res[i].cap = b.size
        return res

    def run(self, feeds: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
        self.ensure_planned(feeds)
        lib = _ffi.lib()
        keep = _ffi.Keep()
        ops = self._operands(feeds, keep)
        res = self._results(keep)
        st = lib.oxb200_run(self.ctx.handle, ops, len(self.graph.input_names), res, len(self.graph.output_names))
        _raise_for(st, self.ctx.last_error())
        return {name: _ffi.result_array(res[i], self._out_bufs[i]) for i, name in enumerate(self.graph.output_names)}

    # ---- pipelined runs: the upload of the next batch overlaps the run of the current one ----
    def submit(self, feeds: Dict[str, np.ndarray]):
        """Enqueues one run (upload, steps, download) and returns at once; at most two may be in flight.
        The feed arrays must stay unchanged until the matching collect()."""
        self.ensure_planned(feeds)
        keep = _ffi.Keep()
        ops = self._operands(feeds, keep)
        _raise_for(_ffi.lib().oxb200_run_submit(self.ctx.handle, ops, len(self.graph.input_names)), self.ctx.last_error())
        if not hasattr(self, "_in_flight"):
            self._in_flight = []
        self._in_flight.append(keep)

    def collect(self) -> Dict[str, np.ndarray]:
        """Waits for the oldest submitted run and returns its outputs."""
        keep = _ffi.Keep()
        res = self._results(keep)
        st = _ffi.lib().oxb200_run_collect(self.ctx.handle, res, len(self.graph.output_names))
        if getattr(self, "_in_flight", None):
            self._in_flight.pop(0)
        _raise_for(st, self.ctx.last_error())
        return {name: _ffi.result_array(res[i], self._out_bufs[i]) for i, name in enumerate(self.graph.output_names)}

    def run_pipelined(self, batches):
        """Runs a sequence of feed dictionaries with one batch in flight behind the one being awaited."""
        out, pending = [], 0
        for feeds in batches:
            self.submit(feeds)
            pending += 1
            if pending == 2:
                out.append(self.collect())
                pending -= 1
        while pending:
            out.append(self.collect())
            pending -= 1
        return out

    # ---- device I/O binding (IoBinding / run_with_binding, extended to device memory) ----
    def bind_input_device(self, name: str, device_ptr: int, dtype, count: int):
        """Graph input `name` is read from the caller's device buffer by the following runs."""
        code = _ffi.TYPED.get(np.dtype(dtype), _ffi.DT_F32)
        _raise_for(_ffi.lib().oxb200_bind_input_device(self.ctx.handle, name.encode(), ctypes.c_void_p(device_ptr), code, count), self.ctx.last_error())

    def bind_output_device(self, name: str, device_ptr: int, capacity: int):
        """Graph output `name` (f32 lanes, logical order) is also written to the caller's device buffer."""
        _raise_for(_ffi.lib().oxb200_bind_output_device(self.ctx.handle, name.encode(), ctypes.c_void_p(device_ptr), capacity), self.ctx.last_error())

    def output_device_ptr(self, name: str):
        """(device address, element count) of the library-owned buffer holding an output's f32 lanes after a run."""
        p, n = ctypes.c_void_p(), ctypes.c_uint64()
        _raise_for(_ffi.lib().oxb200_output_device_ptr(self.ctx.handle, name.encode(), ctypes.byref(p), ctypes.byref(n)), self.ctx.last_error())
        return int(p.value or 0), int(n.value)

    def run_with_binding(self, feeds: Optional[Dict[str, np.ndarray]] = None, fetch: bool = True) -> Optional[Dict[str, np.ndarray]]:
        """One run with the current bindings: bound inputs are read on the device, unbound ones come from `feeds`;
        with fetch=False nothing is read back (the outputs stay in their device buffers)."""
        feeds = feeds or {}
        keep = _ffi.Keep()
        names = [n for n in self.graph.input_names if n in feeds]
        ops = keep.add((_ffi.Operand * max(len(names), 1))())
        for i, name in enumerate(names):
            _ffi.pack_operand(ops[i], name, feeds[name], keep)
        if not fetch:
            st = _ffi.lib().oxb200_run_bound(self.ctx.handle, ops, len(names), None, 0)
            _raise_for(st, self.ctx.last_error())
            return None
        res = self._results(keep)
        st = _ffi.lib().oxb200_run_bound(self.ctx.handle, ops, len(names), res, len(self.graph.output_names))
        _raise_for(st, self.ctx.last_error())
        return {name: _ffi.result_array(res[i], self._out_bufs[i]) for i, name in enumerate(self.graph.output_names)}

    def clear_bindings(self):
        _raise_for(_ffi.lib().oxb200_clear_bindings(self.ctx.handle), self.ctx.last_error())

    # ---- measurement helpers: the same run split into stage / resident launches / read ----
    def upload(self, feeds):
        self.ensure_planned(feeds)
        keep = _ffi.Keep()
        ops = self._operands(feeds, keep)
        _raise_for(_ffi.lib().oxb200_upload_feeds(self.ctx.handle, ops, len(self.graph.input_names)), self.ctx.last_error())

    def run_resident(self, iters=1) -> float:
        ms = ctypes.c_float()
        _raise_for(_ffi.lib().oxb200_run_resident(self.ctx.handle, iters, ctypes.byref(ms)), self.ctx.last_error())
        return float(ms.value)

    def download(self) -> Dict[str, np.ndarray]:
        keep = _ffi.Keep()
        res = self._results(keep)
        _raise_for(_ffi.lib().oxb200_download_fetches(self.ctx.handle, res, len(self.graph.output_names)), self.ctx.last_error())
        return {name: _ffi.result_array(res[i], self._out_bufs[i]) for i, name in enumerate(self.graph.output_names)}

    def fetch_value(self, name: str) -> np.ndarray:
        """Any value of the planned graph after a run (keep_intermediates for intermediates)."""
        lib = _ffi.lib()
        r = _ffi.Result()
        _raise_for(lib.oxb200_fetch_value(self.ctx.handle, name.encode(), ctypes.byref(r)), self.ctx.last_error())
        buf = np.empty(max(int(r.len), 1), np.float32)
        r.lanes = buf.ctypes.data_as(ctypes.POINTER(ctypes.c_float))
        r.cap = buf.size
        _raise_for(lib.oxb200_fetch_value(self.ctx.handle, name.encode(), ctypes.byref(r)), self.ctx.last_error())
        return _ffi.result_array(r, buf)

    def has_value(self, name: str) -> bool:
        r = _ffi.Result()
        return _ffi.lib().oxb200_fetch_value(self.ctx.handle, name.encode(), ctypes.byref(r)) == _ffi.OK_HOST

    def steps(self) -> List[dict]:
        """NodeProfile-like records of the planned steps (profiling_results)."""
        lib = _ffi.lib()
        out = []
        for i in range(lib.oxb200_plan_step_count(self.ctx.handle)):
            s = _ffi.StepInfo()
            lib.oxb200_plan_step_info(self.ctx.handle, i, ctypes.byref(s))
            out.append(dict(node=s.node_name.decode(), op=s.op_type.decode(), kernel=s.kernel.decode(), work=float(s.work),
                            work_is_bytes=bool(s.work_is_bytes), ms=float(s.last_ms), launches=int(s.launches), bytes=float(s.bytes)))
        return out

    def cuda_cache_counters(self) -> dict:
        return self.ctx.cache_counters()

    def close(self):
        self.ctx.close()
