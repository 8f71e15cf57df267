"""ctypes driver for the UNMODIFIED magnetron C API (include/magnetron/magnetron.h of the reference).

TEST INFRASTRUCTURE ONLY: this module is the checker, never the product. It loads a directory that
holds `libmagnetron_core.so` plus backend modules (`libmagnetron_cpu.so`, optionally a
`libmagnetron_cuda.so`) and exposes the handful of C API calls that the matmul / cast path uses:

    mag_ctx_create / mag_ctx_destroy            include/magnetron/magnetron.h:103,118
    mag_empty, mag_as_strided                   include/magnetron/magnetron.h:210-211
    mag_copy_raw_                               include/magnetron/magnetron.h:231
    mag_cast                                    include/magnetron/magnetron.h:239
    mag_view / mag_reshape / mag_transpose / mag_permute / mag_contiguous   :240-246
    mag_matmul                                  include/magnetron/magnetron.h:372
    mag_tensor_* accessors                      include/magnetron/magnetron.h:398-446

The default directory is `oracle/_ref/`, the output of `make -C oracle REF=<magnetron source tree>` (the reference's own sources
compiled where they lie). The same class drives a directory where the B200 plug-in was dropped next
to the reference core, which is how the drop-in boundary is tested: same calls, device "cuda:0".
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")

# mag_dtype_t, include/magnetron/magnetron.h:171-186
FLOAT32, FLOAT16, BFLOAT16 = 0, 1, 2
DTYPE_SIZE = {FLOAT32: 4, FLOAT16: 2, BFLOAT16: 2}
DTYPE_NP = {FLOAT32: np.uint32, FLOAT16: np.uint16, BFLOAT16: np.uint16}  # raw bit containers
MAG_STATUS_OK = 0


class MagError(C.Structure):  # include/magnetron/magnetron.h:87-93
    _fields_ = [("code", C.c_int), ("message", C.c_char * 256), ("file", C.c_char_p),
                ("line", C.c_int), ("func", C.c_char_p)]


class MagStatusError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"magnetron status {code}: {message}")
        self.code = code


def available(lib_dir: str = REF_DIR) -> bool:
    return os.path.exists(os.path.join(lib_dir, "libmagnetron_core.so")) and \
        os.path.exists(os.path.join(lib_dir, "libmagnetron_cpu.so"))


class Tensor:
    """Owning handle of one mag_tensor_t* (decref on release)."""

    def __init__(self, api: "MagApi", ptr: int):
        self.api, self.ptr = api, ptr

    def release(self):
        if self.ptr:
            self.api.lib.mag_tensor_decref(self.ptr)
            self.ptr = None

    @property
    def rank(self) -> int:
        return self.api.lib.mag_tensor_rank(self.ptr)

    @property
    def shape(self) -> tuple:
        p = self.api.lib.mag_tensor_shape_ptr(self.ptr)
        return tuple(p[i] for i in range(self.rank))

    @property
    def strides(self) -> tuple:
        p = self.api.lib.mag_tensor_strides_ptr(self.ptr)
        return tuple(p[i] for i in range(self.rank))

    @property
    def dtype(self) -> int:
        return self.api.lib.mag_tensor_type(self.ptr)

    @property
    def numel(self) -> int:
        return self.api.lib.mag_tensor_numel(self.ptr)

    @property
    def data_ptr(self) -> int:
        return self.api.lib.mag_tensor_data_ptr(self.ptr)

    # view recipes (same method names as magnetron_b200.Tensor so one case list drives both)
    def transpose(self, d0, d1):
        return self.api.transpose(self, d0, d1)

    def permute(self, dims):
        return self.api.permute(self, dims)

    def view(self, shape):
        return self.api.view(self, shape)

    def slice(self, dim, start, length, step=1):
        return self.api.view_slice(self, dim, start, length, step)


class MagApi:
    """One magnetron context on one device string ("cpu", "cuda:0", ...)."""

    def __init__(self, device: str = "cpu", lib_dir: str = REF_DIR, log_level: int | None = None):
        path = os.path.join(lib_dir, "libmagnetron_core.so")
        if not os.path.exists(path):
            raise FileNotFoundError(f"{path} missing: run `make -C oracle REF=<magnetron source tree>` where the reference sources are present")
        self.lib = lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
        P, I64, VP = C.c_void_p, C.c_int64, C.c_void_p
        I64P = C.POINTER(C.c_int64)
        sig = {
            "mag_ctx_create": (P, [C.c_char_p]),
            "mag_ctx_destroy": (None, [P, C.c_bool]),
            "mag_ctx_get_compute_device_name": (C.c_char_p, [P]),
            "mag_ctx_get_cpu_name": (C.c_char_p, [P]),
            "mag_ctx_get_cpu_virtual_cores": (C.c_uint32, [P]),
            "mag_ctx_grad_recorder_stop": (None, [P]),
            "mag_set_log_level": (None, [C.c_int]),
            "mag_empty": (C.c_int, [VP, C.POINTER(P), P, C.c_int, I64, I64P]),
            "mag_as_strided": (C.c_int, [VP, C.POINTER(P), P, P, I64, I64P, I64P, I64]),
            "mag_copy_raw_": (C.c_int, [VP, P, VP, C.c_size_t]),
            "mag_cast": (C.c_int, [VP, C.POINTER(P), P, C.c_int]),
            "mag_clone": (C.c_int, [VP, C.POINTER(P), P]),
            "mag_contiguous": (C.c_int, [VP, C.POINTER(P), P]),
            "mag_view": (C.c_int, [VP, C.POINTER(P), P, I64P, I64]),
            "mag_reshape": (C.c_int, [VP, C.POINTER(P), P, I64P, I64]),
            "mag_transpose": (C.c_int, [VP, C.POINTER(P), P, I64, I64]),
            "mag_permute": (C.c_int, [VP, C.POINTER(P), P, I64P, I64]),
            "mag_view_slice": (C.c_int, [VP, C.POINTER(P), P, I64, I64, I64, I64]),
            "mag_matmul": (C.c_int, [VP, C.POINTER(P), P, P]),
            "mag_silu": (C.c_int, [VP, C.POINTER(P), P]),
            "mag_mul": (C.c_int, [VP, C.POINTER(P), P, P]),
            "mag_tensor_rank": (I64, [P]),
            "mag_tensor_shape_ptr": (I64P, [P]),
            "mag_tensor_strides_ptr": (I64P, [P]),
            "mag_tensor_type": (C.c_int, [P]),
            "mag_tensor_numel": (I64, [P]),
            "mag_tensor_data_ptr": (C.c_size_t, [P]),
            "mag_tensor_is_contiguous": (C.c_bool, [P]),
            "mag_tensor_decref": (C.c_bool, [P]),
        }
        for name, (res, args) in sig.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        if log_level is not None:
            lib.mag_set_log_level(log_level)
        self.ctx = lib.mag_ctx_create(device.encode())
        if not self.ctx:
            raise RuntimeError("mag_ctx_create failed")
        lib.mag_ctx_grad_recorder_stop(self.ctx)  # inference path: no autograd retention
        self.device_name = lib.mag_ctx_get_compute_device_name(self.ctx).decode()
        self.cpu_name = lib.mag_ctx_get_cpu_name(self.ctx).decode()
        self.cores = int(lib.mag_ctx_get_cpu_virtual_cores(self.ctx))

    def close(self, suppress_leak_detection: bool = False):
        if self.ctx:
            self.lib.mag_ctx_destroy(self.ctx, suppress_leak_detection)
            self.ctx = None

    # ---- helpers -------------------------------------------------------------------------------
    def _call(self, fn, *args) -> Tensor:
        err = MagError()
        out = C.c_void_p()
        st = fn(C.byref(err), C.byref(out), *args)
        if st != MAG_STATUS_OK:
            raise MagStatusError(st, err.message.decode(errors="replace"))
        return Tensor(self, out.value)

    @staticmethod
    def _dims(d: Sequence[int]):
        return (C.c_int64 * len(d))(*d)

    def empty(self, dtype: int, shape: Sequence[int]) -> Tensor:
        return self._call(self.lib.mag_empty, self.ctx, dtype, len(shape), self._dims(shape))

    def from_bits(self, dtype: int, bits: np.ndarray) -> Tensor:
        """New contiguous tensor holding exactly these bit patterns (uint16 / uint32 array)."""
        bits = np.ascontiguousarray(bits, dtype=DTYPE_NP[dtype])
        t = self.empty(dtype, bits.shape if bits.ndim else (1,))
        err = MagError()
        st = self.lib.mag_copy_raw_(C.byref(err), t.ptr, bits.ctypes.data, bits.nbytes)
        if st != MAG_STATUS_OK:
            raise MagStatusError(st, err.message.decode(errors="replace"))
        return t

    def to_bits(self, t: Tensor) -> np.ndarray:
        """Bit patterns of a contiguous CPU tensor."""
        assert self.lib.mag_tensor_is_contiguous(t.ptr)
        n = t.numel
        buf = (C.c_uint8 * (n * DTYPE_SIZE[t.dtype])).from_address(t.data_ptr)
        return np.frombuffer(buf, dtype=DTYPE_NP[t.dtype]).reshape(t.shape).copy()

    def as_strided(self, base: Tensor, shape, strides, offset=0) -> Tensor:
        return self._call(self.lib.mag_as_strided, self.ctx, base.ptr, len(shape), self._dims(shape),
                          self._dims(strides), offset)

    def view(self, x: Tensor, shape) -> Tensor:
        return self._call(self.lib.mag_view, x.ptr, self._dims(shape), len(shape))

    def reshape(self, x: Tensor, shape) -> Tensor:
        return self._call(self.lib.mag_reshape, x.ptr, self._dims(shape), len(shape))

    def transpose(self, x: Tensor, d0: int, d1: int) -> Tensor:
        return self._call(self.lib.mag_transpose, x.ptr, d0, d1)

    def permute(self, x: Tensor, dims) -> Tensor:
        return self._call(self.lib.mag_permute, x.ptr, self._dims(dims), len(dims))

    def view_slice(self, x: Tensor, dim: int, start: int, length: int, step: int = 1) -> Tensor:
        return self._call(self.lib.mag_view_slice, x.ptr, dim, start, length, step)

    def contiguous(self, x: Tensor) -> Tensor:
        return self._call(self.lib.mag_contiguous, x.ptr)

    def cast(self, x: Tensor, dtype: int) -> Tensor:
        return self._call(self.lib.mag_cast, x.ptr, dtype)

    def matmul(self, x: Tensor, y: Tensor) -> Tensor:
        return self._call(self.lib.mag_matmul, x.ptr, y.ptr)

    def silu(self, x: Tensor) -> Tensor:          # include/magnetron/magnetron.h:342
        return self._call(self.lib.mag_silu, x.ptr)

    def mul(self, x: Tensor, y: Tensor) -> Tensor:  # include/magnetron/magnetron.h:362
        return self._call(self.lib.mag_mul, x.ptr, y.ptr)
