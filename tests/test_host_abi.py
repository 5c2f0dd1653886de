"""CPU-side checks: the C-ABI library loads and exports every symbol include/oxb200.h
declares, the pure boundary predicates follow the reference's rules, and creating a context
fails loudly when no GPU exists (there is no CPU path behind the library)."""
import os
import re

import pytest

from oxionnx_b200 import _ffi
from oxionnx_b200 import build as build_lib
from oxionnx_b200 import session as S

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module", autouse=True)
def built():
    if not os.path.exists(_ffi.LIB_PATH):
        build_lib.build()


def declared_symbols():
    with open(os.path.join(ROOT, "include", "oxb200.h")) as fh:
        text = re.sub(r"/\*.*?\*/", "", fh.read(), flags=re.S)
    return sorted(set(re.findall(r"\b(oxb200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    names = declared_symbols()
    assert len(names) >= 28
    lib = _ffi.lib()
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/oxb200.h but not exported"
        assert n in _ffi.SYMBOLS, f"{n} has no ctypes signature"
    assert sorted(_ffi.SYMBOLS) == names


def test_is_supported_op_adds_the_int8_family():
    for op in ("Conv", "Gemm", "MatMul", "QLinearConv", "QLinearMatMul", "MatMulInteger", "ConvInteger", "QuantizeLinear",
               "DequantizeLinear", "DynamicQuantizeLinear", "GlobalAveragePool", "OxiInstanceNorm", "Resize", "Concat", "Add"):
        assert S.is_supported_op(op), op
    for op in ("LSTM", "Softplus", "NonMaxSuppression", "If", "Loop", ""):
        assert not S.is_supported_op(op), op


def test_accepts_resident_slot_only_for_data_operands():
    assert S.accepts_resident_slot("QLinearConv", 0)
    for slot in range(1, 9):
        assert not S.accepts_resident_slot("QLinearConv", slot)
    assert S.accepts_resident_slot("MatMulInteger", 0) and S.accepts_resident_slot("MatMulInteger", 2)
    assert not S.accepts_resident_slot("MatMulInteger", 1)
    assert S.accepts_resident_slot("Add", 0) and S.accepts_resident_slot("Add", 1)
    assert not S.accepts_resident_slot("LSTM", 0)


def test_decide_placement_follows_the_reference_policy():
    """root crate src/execution_providers.rs:352-387: CpuOnly never; Auto by the byte
    threshold and the provider's own claim; Manual by the pin and the 4096-byte floor."""
    P = S.OpPlacement
    assert not P("cpu_only").decide("Conv", 1 << 30)
    auto = P("auto", gpu_threshold_bytes=65536)
    assert not auto.decide("Conv", 65535)
    assert auto.decide("Conv", 65536)
    assert not auto.decide("LSTM", 1 << 30)
    manual = P("manual", manual={"Conv": "cuda", "Relu": "cpu"})
    assert manual.decide("Conv", 4096)
    assert not manual.decide("Conv", 4095)        # MIN_GPU_DISPATCH_BYTES floor
    assert not manual.decide("Relu", 1 << 20)     # pinned to the CPU
    assert not manual.decide("MatMul", 1 << 20)   # unmapped


def test_env_truthiness_rule():
    """oxionnx-cuda src/context.rs:179-192: anything unrecognised is enabled."""
    for v in (None, "", "  ", "0", "false", "FALSE", "off", "No"):
        assert not S.env_truthy(v), repr(v)
    for v in ("1", "true", "on", "yes", "banana", "2"):
        assert S.env_truthy(v), repr(v)


def test_verify_mismatch_marker():
    assert S.is_verify_mismatch("CUDA VERIFY MISMATCH: Conv: element 3")
    assert not S.is_verify_mismatch("Conv: CUDA VERIFY MISMATCH")
    assert not S.is_verify_mismatch("")


def test_context_creation_fails_loudly_without_a_gpu():
    if S.device_count() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(S.OnnxError) as ei:
        S.CudaContext(0)
    assert "no CUDA device" in str(ei.value) and "no CPU path" in str(ei.value)
    assert S.CudaContext.try_new(0) is None


def test_config_from_env(monkeypatch):
    import ctypes
    monkeypatch.setenv("OXIONNX_CUDA_VERIFY", "1")
    monkeypatch.setenv("OXIONNX_CUDA_STRICT", "off")
    monkeypatch.delenv("OXIONNX_CUDA_RESIDENCY", raising=False)
    cfg = _ffi.Config()
    _ffi.lib().oxb200_config_from_env(ctypes.byref(cfg))
    assert cfg.verify == 1 and cfg.strict == 0 and cfg.residency == 1
    monkeypatch.setenv("OXIONNX_CUDA_RESIDENCY", "0")
    _ffi.lib().oxb200_config_from_env(ctypes.byref(cfg))
    assert cfg.residency == 0
