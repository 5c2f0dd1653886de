"""The allocation-free DynamicQuantizeLinear entry point against the ordinary one.

Hosts that may not allocate device memory at run time (fixed-memory frame loops, plug-ins living
inside another runtime's arena) call oxb200_dynamic_quantize_linear_noalloc with buffers they
already own; its reduction scratch is a static array inside the library.  The test calls it
twice in a row through the C ABI -- the second call with different data, which would expose
stale contents of the shared scratch -- and requires the quantised lanes, the scale and the zero
point to equal, bit for bit, what the DynamicQuantizeLinear node of oxb200_dispatch produces and
what the CPU oracle (the restatement of the reference's operator) produces.
This file is named so that pytest collects it last.
"""
import ctypes

import numpy as np
import pytest

import oracle
from oxionnx_b200 import _ffi
from oxionnx_b200.graph import Node
from oxionnx_b200 import session as S

pytestmark = pytest.mark.gpu


def _reference(ctx, x):
    node = Node("DynamicQuantizeLinear", "dq", ["x"], ["y", "scale", "zp"], {})
    y, scale, zp = S.try_cuda_dispatch(node, {}, {"x": x}, ctx)
    return y, scale, zp


def test_no_alloc_entry_point_matches_the_ordinary_one_twice_in_a_row():
    import torch

    lib = _ffi.lib()
    ctx = S.CudaContext(0)
    rng = np.random.default_rng(20261125)
    inputs = [
        (rng.standard_normal((777, 129)) * 3.0).astype(np.float32),          # odd length: exercises the scalar tail
        (rng.uniform(-0.25, 9.0, (64, 1024))).astype(np.float32),            # different range: stale min/max would show
    ]
    stream = torch.cuda.current_stream().cuda_stream
    for x in inputs:
        want_y, want_scale, want_zp = _reference(ctx, x)
        xd = torch.from_numpy(x).cuda()
        yd = torch.empty(x.size, dtype=torch.uint8, device="cuda")
        pd = torch.empty(2, dtype=torch.float32, device="cuda")
        st = lib.oxb200_dynamic_quantize_linear_noalloc(0, ctypes.c_void_p(xd.data_ptr()), x.size, ctypes.c_void_p(yd.data_ptr()),
                                                        ctypes.c_void_p(pd.data_ptr()), ctypes.c_void_p(stream))
        assert st == _ffi.OK_DEVICE, lib.oxb200_last_error(None).decode()
        torch.cuda.synchronize()
        got_y = yd.cpu().numpy().astype(np.float32).reshape(x.shape)
        got_p = pd.cpu().numpy()
        assert np.array_equal(got_y, want_y)
        assert got_p[0] == np.float32(want_scale) and got_p[1] == np.float32(want_zp)
        # and against the CPU oracle (quant_ops/dynamic_quantize.rs:51-93 restated)
        o_y, o_scale, o_zp = oracle.run_node("DynamicQuantizeLinear", [x], {}, n_outputs=3)
        assert np.array_equal(got_y, o_y)
        assert got_p[0] == np.float32(o_scale) and got_p[1] == np.float32(o_zp)
    ctx.close()


def test_no_alloc_entry_point_rejects_oversized_and_null_arguments():
    lib = _ffi.lib()
    st = lib.oxb200_dynamic_quantize_linear_noalloc(0, ctypes.c_void_p(256), (1 << 28) + 1, ctypes.c_void_p(256), ctypes.c_void_p(256), None)
    assert st == _ffi.FAILED
    assert "exceed the maximum" in lib.oxb200_last_error(None).decode()
    st = lib.oxb200_dynamic_quantize_linear_noalloc(0, None, 16, ctypes.c_void_p(256), ctypes.c_void_p(256), None)
    assert st == _ffi.FAILED


def test_no_alloc_entry_point_rejects_misaligned_buffers_before_any_launch():
    """x is read in 16-byte pieces and y written in 4-byte words: a sub-buffer at an odd offset is refused on the
    host (nothing is launched, so the dummy addresses are never touched)."""
    lib = _ffi.lib()
    for x, y, p, word in ((256 + 4, 256, 256, "x_device"), (256, 256 + 1, 256, "y_device"), (256, 256, 256 + 2, "scale_zp_device")):
        st = lib.oxb200_dynamic_quantize_linear_noalloc(0, ctypes.c_void_p(x), 64, ctypes.c_void_p(y), ctypes.c_void_p(p), None)
        assert st == _ffi.FAILED
        msg = lib.oxb200_last_error(None).decode()
        assert word in msg and "aligned" in msg
