"""CPU tests of the C-ABI boundary: the library loads, exports exactly what include/magnetron_b200.h
declares, validates arguments on the host, and refuses to compute without a device (no fallback)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import magnetron_b200 as mb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "magnetron_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(magb200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    names = declared_functions()
    assert len(names) >= 25
    assert sorted(mb.SIGNATURES) == names


def test_library_exports_every_declared_symbol():
    handle = C.CDLL(mb.lib_path())
    for name in declared_functions():
        assert hasattr(handle, name), name


def test_view_struct_layout():
    assert C.sizeof(mb.View) == 8 + 8 + 4 + 4 + 16 * 8 * 2


def test_result_shape_rules_without_device():
    L = mb.lib()
    dummy = 0x1000  # never dereferenced by shape inference
    def shape(xs, ys):
        rank = C.c_int32()
        out = (C.c_int64 * 18)()
        rc = L.magb200_matmul_result_shape(C.byref(mb.make_view(dummy, mb.BFLOAT16, xs)),
                                           C.byref(mb.make_view(dummy, mb.BFLOAT16, ys)), C.byref(rank), out)
        return rc, tuple(out[i] for i in range(rank.value))
    assert shape((4,), (4,)) == (0, ())
    assert shape((4,), (4, 5)) == (0, (5,))
    assert shape((3, 4), (4,)) == (0, (3,))
    assert shape((2, 1, 3, 4), (1, 6, 4, 5)) == (0, (2, 6, 3, 5))
    rc, _ = shape((3, 4), (5, 6))
    assert rc == mb.ERR_SHAPE and b"does not match" in L.magb200_last_error()
    rc, _ = shape((2, 3, 4), (3, 4, 5))
    assert rc == mb.ERR_SHAPE and b"batch dimensions" in L.magb200_last_error()


def test_argument_validation_on_host():
    L = mb.lib()
    bad = mb.make_view(0x1000, 7, (4, 4))  # dtype outside {f32,f16,bf16}
    rank = C.c_int32()
    out = (C.c_int64 * 18)()
    assert L.magb200_matmul_result_shape(C.byref(bad), C.byref(bad), C.byref(rank), out) == mb.ERR_INVALID_ARG
    assert L.magb200_force_kernel(99) == mb.ERR_INVALID_ARG
    assert L.magb200_force_kernel(0) == 0


def test_no_silent_cpu_fallback():
    if mb.device_count() > 0:
        pytest.skip("a device is present")
    L = mb.lib()
    v = mb.make_view(0x1000, mb.BFLOAT16, (4, 4))
    assert L.magb200_matmul(0, C.byref(v), C.byref(v), C.byref(v)) == mb.ERR_NO_DEVICE
    assert L.magb200_cast(0, C.byref(v), C.byref(v)) == mb.ERR_NO_DEVICE
    assert b"no CPU fallback" in L.magb200_last_error()
    with pytest.raises(mb.MagB200Error):
        mb.Tensor.from_bits(0, mb.BFLOAT16, np.zeros((2, 2), np.uint16))


def test_view_solver():
    f = mb.solve_view_strides
    assert f((2, 3, 4), (12, 4, 1), (6, 4)) == (4, 1)
    assert f((2, 3, 4), (12, 4, 1), (2, 12)) == (12, 1)
    assert f((4, 6), (1, 4), (24,)) is None                       # transposed: not viewable flat
    assert f((1, 2, 8, 16), (256, 128, 1, 8), (1, 2, 1, 8, 16)) == (0, 128, 0, 1, 8)   # K^T with a broadcast slot
    assert f((2, 3), (3, 1), (3, 2)) == (2, 1)
