"""ctypes bindings of include/oxb200.h.  Loading fails loudly when the CUDA library has not
been built: there is no CPU path behind this package."""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("OXB200_LIBRARY") or os.path.join(HERE, "_lib", "liboxb200.so")

MAX_RANK = 8
DT_F32, DT_U8, DT_I8, DT_I32, DT_F16, DT_BF16 = 0, 1, 2, 3, 5, 6
# numpy element types that cross the boundary as typed lanes
TYPED = {np.dtype(np.uint8): DT_U8, np.dtype(np.int8): DT_I8}
OK_HOST, OK_DEVICE, DECLINED, FAILED, VERIFY_MISMATCH = 0, 1, 2, 3, 4
PLACE_HOST, PLACE_DEVICE = 0, 1
STATUS_NAMES = {0: "OK_HOST", 1: "OK_DEVICE", 2: "DECLINED", 3: "FAILED", 4: "VERIFY_MISMATCH"}


class Attr(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("kind", ctypes.c_int32), ("i", ctypes.c_int64), ("f", ctypes.c_float),
                ("s", ctypes.c_char_p), ("ints", ctypes.POINTER(ctypes.c_int64)), ("floats", ctypes.POINTER(ctypes.c_float)),
                ("len", ctypes.c_uint64)]


class CNode(ctypes.Structure):
    _fields_ = [("op_type", ctypes.c_char_p), ("name", ctypes.c_char_p), ("inputs", ctypes.POINTER(ctypes.c_char_p)),
                ("n_inputs", ctypes.c_uint32), ("outputs", ctypes.POINTER(ctypes.c_char_p)), ("n_outputs", ctypes.c_uint32),
                ("attrs", ctypes.POINTER(Attr)), ("n_attrs", ctypes.c_uint32)]


class Operand(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("lanes", ctypes.POINTER(ctypes.c_float)), ("len", ctypes.c_uint64),
                ("shape", ctypes.POINTER(ctypes.c_uint64)), ("rank", ctypes.c_uint32), ("resident", ctypes.c_void_p),
                ("dtype", ctypes.c_int32), ("typed", ctypes.c_void_p)]


class Result(ctypes.Structure):
    _fields_ = [("lanes", ctypes.POINTER(ctypes.c_float)), ("cap", ctypes.c_uint64), ("len", ctypes.c_uint64),
                ("shape", ctypes.c_uint64 * MAX_RANK), ("rank", ctypes.c_uint32), ("resident", ctypes.c_void_p)]


class ValueInfo(ctypes.Structure):
    _fields_ = [("name", ctypes.c_char_p), ("shape", ctypes.POINTER(ctypes.c_uint64)), ("rank", ctypes.c_uint32), ("dtype", ctypes.c_int32)]


class Config(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_uint32), ("verify", ctypes.c_int32), ("strict", ctypes.c_int32), ("residency", ctypes.c_int32),
                ("cuda_graph", ctypes.c_int32), ("kernel_path", ctypes.c_int32), ("keep_intermediates", ctypes.c_int32),
                ("profile", ctypes.c_int32), ("requant_f64", ctypes.c_int32), ("split_k_max", ctypes.c_int32), ("cta_pairs", ctypes.c_int32),
                ("float_precision", ctypes.c_int32), ("reserved", ctypes.c_int32 * 4)]


class Counters(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint64) for n in (
        "uploads", "upload_bytes", "downloads", "download_bytes", "fences", "weight_uploads", "weight_bytes_resident", "arena_bytes",
        "arena_peak_bytes", "arena_slots", "kernel_launches", "umma_launches", "simt_launches", "glue_launches", "dispatches", "declines",
        "failures", "graph_captures", "graph_replays", "graph_poisoned")]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


class StepInfo(ctypes.Structure):
    _fields_ = [("node_name", ctypes.c_char_p), ("op_type", ctypes.c_char_p), ("kernel", ctypes.c_char_p), ("work", ctypes.c_double),
                ("work_is_bytes", ctypes.c_int32), ("last_ms", ctypes.c_float), ("launches", ctypes.c_uint64), ("bytes", ctypes.c_double)]


# every symbol include/oxb200.h declares: (restype, argtypes)
_P = ctypes.POINTER
SYMBOLS = {
    "oxb200_is_supported_op": (ctypes.c_int, [ctypes.c_char_p]),
    "oxb200_accepts_resident_slot": (ctypes.c_int, [ctypes.c_char_p, ctypes.c_uint32]),
    "oxb200_decide_placement": (ctypes.c_int, [ctypes.c_int, ctypes.c_uint64, ctypes.c_int, ctypes.c_char_p, ctypes.c_uint64]),
    "oxb200_is_verify_mismatch": (ctypes.c_int, [ctypes.c_char_p]),
    "oxb200_env_truthy": (ctypes.c_int, [ctypes.c_char_p]),
    "oxb200_config_from_env": (None, [_P(Config)]),
    "oxb200_device_count": (ctypes.c_int, []),
    "oxb200_tensor_alias": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, _P(ctypes.c_uint64), ctypes.c_uint32, _P(ctypes.c_void_p)]),
    "oxb200_tensor_reserved_bytes": (ctypes.c_uint64, [ctypes.c_void_p]),
    "oxb200_streams_unified": (ctypes.c_int, [ctypes.c_void_p]),
    "oxb200_cached_device_bytes": (ctypes.c_uint64, [ctypes.c_void_p]),
    "oxb200_set_graph_capture": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int]),
    "oxb200_graph_capture_enabled": (ctypes.c_int, [ctypes.c_void_p]),
    "oxb200_ctx_create": (ctypes.c_int, [ctypes.c_int, _P(Config), _P(ctypes.c_void_p)]),
    "oxb200_ctx_destroy": (None, [ctypes.c_void_p]),
    "oxb200_last_error": (ctypes.c_char_p, [ctypes.c_void_p]),
    "oxb200_get_counters": (None, [ctypes.c_void_p, _P(Counters)]),
    "oxb200_release_device_caches": (ctypes.c_int, [ctypes.c_void_p]),
    "oxb200_set_profile": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int]),
    "oxb200_probe_tensor_peak": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, _P(ctypes.c_double)]),
    "oxb200_host_alloc": (ctypes.c_void_p, [ctypes.c_size_t]),
    "oxb200_host_free": (None, [ctypes.c_void_p]),
    "oxb200_weight_register": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p, _P(ctypes.c_float), ctypes.c_uint64, _P(ctypes.c_uint64),
                                              ctypes.c_uint32]),
    "oxb200_weight_register_typed": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p, _P(ctypes.c_float), ctypes.c_uint64, _P(ctypes.c_uint64),
                                                    ctypes.c_uint32, ctypes.c_int32]),
    "oxb200_is_weight_resident": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p]),
    "oxb200_dispatch": (ctypes.c_int, [ctypes.c_void_p, _P(CNode), _P(Operand), ctypes.c_uint32, ctypes.c_int, _P(Result), ctypes.c_uint32]),
    "oxb200_shadow_verify": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p, _P(ctypes.c_float), _P(ctypes.c_float), ctypes.c_uint64]),
    "oxb200_tensor_shape": (ctypes.c_int, [ctypes.c_void_p, _P(ctypes.c_uint64), _P(ctypes.c_uint32), _P(ctypes.c_uint64)]),
    "oxb200_tensor_read_back": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, _P(ctypes.c_float), ctypes.c_uint64]),
    "oxb200_tensor_release": (None, [ctypes.c_void_p, ctypes.c_void_p]),
    "oxb200_session_plan": (ctypes.c_int, [ctypes.c_void_p, _P(CNode), ctypes.c_uint32, _P(ValueInfo), ctypes.c_uint32, _P(ctypes.c_char_p),
                                           ctypes.c_uint32]),
    "oxb200_run": (ctypes.c_int, [ctypes.c_void_p, _P(Operand), ctypes.c_uint32, _P(Result), ctypes.c_uint32]),
    "oxb200_run_submit": (ctypes.c_int, [ctypes.c_void_p, _P(Operand), ctypes.c_uint32]),
    "oxb200_run_collect": (ctypes.c_int, [ctypes.c_void_p, _P(Result), ctypes.c_uint32]),
    "oxb200_last_run_ms": (ctypes.c_float, [ctypes.c_void_p]),
    "oxb200_bind_input_device": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_uint64]),
    "oxb200_bind_output_device": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_uint64]),
    "oxb200_output_device_ptr": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p, _P(ctypes.c_void_p), _P(ctypes.c_uint64)]),
    "oxb200_run_bound": (ctypes.c_int, [ctypes.c_void_p, _P(Operand), ctypes.c_uint32, _P(Result), ctypes.c_uint32]),
    "oxb200_clear_bindings": (ctypes.c_int, [ctypes.c_void_p]),
    "oxb200_upload_feeds": (ctypes.c_int, [ctypes.c_void_p, _P(Operand), ctypes.c_uint32]),
    "oxb200_run_resident": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint32, _P(ctypes.c_float)]),
    "oxb200_download_fetches": (ctypes.c_int, [ctypes.c_void_p, _P(Result), ctypes.c_uint32]),
    "oxb200_fetch_value": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p, _P(Result)]),
    "oxb200_plan_step_count": (ctypes.c_uint32, [ctypes.c_void_p]),
    "oxb200_plan_step_info": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint32, _P(StepInfo)]),
    "oxb200_model_load": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint64, _P(ctypes.c_void_p)]),
    "oxb200_model_load_file": (ctypes.c_int, [ctypes.c_char_p, _P(ctypes.c_void_p)]),
    "oxb200_model_free": (None, [ctypes.c_void_p]),
    "oxb200_model_optimize": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_int32, _P(ctypes.c_uint32)]),
    "oxb200_model_run_pass": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_char_p, _P(ctypes.c_uint32)]),
    "oxb200_model_node_count": (ctypes.c_uint32, [ctypes.c_void_p]),
    "oxb200_model_node": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint32, _P(CNode)]),
    "oxb200_model_input_count": (ctypes.c_uint32, [ctypes.c_void_p]),
    "oxb200_model_input": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint32, _P(ValueInfo)]),
    "oxb200_model_output_count": (ctypes.c_uint32, [ctypes.c_void_p]),
    "oxb200_model_output_name": (ctypes.c_char_p, [ctypes.c_void_p, ctypes.c_uint32]),
    "oxb200_model_initializer_count": (ctypes.c_uint32, [ctypes.c_void_p]),
    "oxb200_model_initializer": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_uint32, _P(Operand)]),
    "oxb200_session_plan_model": (ctypes.c_int, [ctypes.c_void_p, ctypes.c_void_p, _P(ValueInfo), ctypes.c_uint32]),
    "oxb200_dynamic_quantize_linear_noalloc": (ctypes.c_int, [ctypes.c_int, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p,
                                                              ctypes.c_void_p]),
}

_lib = None


def lib():
    """The loaded C-ABI library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python oxionnx_b200/build.py`. "
                "This package has no CPU implementation to fall back to.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


# ---- marshalling helpers --------------------------------------------------------------------
class Keep:
    """Owns the ctypes buffers of a marshalled call."""

    def __init__(self):
        self.items = []

    def add(self, x):
        self.items.append(x)
        return x


def pack_attr_list(attrs, keep):
    items = list((attrs or {}).items())
    arr = keep.add((Attr * max(len(items), 1))())
    for idx, (name, value) in enumerate(items):
        a = arr[idx]
        a.name = name.encode()
        if isinstance(value, (bool, int, np.integer)):
            a.kind, a.i = 0, int(value)
        elif isinstance(value, (float, np.floating)):
            a.kind, a.f = 1, float(value)
        elif isinstance(value, str):
            a.kind, a.s = 2, value.encode()
        elif isinstance(value, (list, tuple, np.ndarray)):
            vals = list(value)
            if all(isinstance(v, (int, np.integer)) and not isinstance(v, bool) for v in vals):
                buf = keep.add((ctypes.c_int64 * max(len(vals), 1))(*[int(v) for v in vals]))
                a.kind, a.ints, a.len = 3, buf, len(vals)
            else:
                buf = keep.add((ctypes.c_float * max(len(vals), 1))(*[float(v) for v in vals]))
                a.kind, a.floats, a.len = 4, buf, len(vals)
        else:
            raise TypeError(f"attribute {name!r}: unsupported value type {type(value)}")
    return arr, len(items)


def pack_node(node, cnode, keep):
    cnode.op_type = node.op.encode()
    cnode.name = (node.name or "").encode()
    ins = keep.add((ctypes.c_char_p * max(len(node.inputs), 1))(*[s.encode() for s in node.inputs]))
    outs = keep.add((ctypes.c_char_p * max(len(node.outputs), 1))(*[s.encode() for s in node.outputs]))
    cnode.inputs, cnode.n_inputs = ins, len(node.inputs)
    cnode.outputs, cnode.n_outputs = outs, len(node.outputs)
    arr, n = pack_attr_list(node.attrs, keep)
    cnode.attrs, cnode.n_attrs = arr, n


def pack_operand(op, name, array, keep, resident=None):
    op.name = name.encode()
    if resident is not None:
        op.resident = resident
        return
    if array is None:
        return
    if isinstance(array, np.ndarray) and array.dtype in TYPED:
        # 8-bit lanes of a graph input that was declared with that type
        a = keep.add(np.ascontiguousarray(array))
        op.typed = a.ctypes.data_as(ctypes.c_void_p)
        op.dtype = TYPED[a.dtype]
        op.len = a.size
        op.shape = keep.add((ctypes.c_uint64 * max(a.ndim, 1))(*a.shape))
        op.rank = a.ndim
        return
    a = keep.add(np.ascontiguousarray(np.asarray(array, dtype=np.float32)))
    op.lanes = a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))
    op.len = a.size
    op.shape = keep.add((ctypes.c_uint64 * max(a.ndim, 1))(*a.shape))
    op.rank = a.ndim


def result_array(res, buf):
    shape = tuple(int(res.shape[d]) for d in range(res.rank))
    n = int(res.len)
    return buf[:n].reshape(shape).copy()
