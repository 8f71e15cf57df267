"""magnetron_b200 -- B200 (sm_100a) implementation of magnetron's MATMUL and fp32<->bf16/fp16 CAST.

The product is the C ABI of `include/magnetron_b200.h` (built into `lib/libmagnetron_b200.so`) and the
magnetron backend module `lib/libmagnetron_cuda.so`. This Python package is a thin ctypes binding of
that C ABI plus a small `Tensor` handle whose methods carry the names of the magnetron C API they
stand for (`mag_transpose`, `mag_view`, `mag_matmul`, `mag_cast`, ...), so tests and the benchmark
can state problems the way a magnetron user would. There is no CPU fallback anywhere: every
operator call goes to the CUDA library and raises if it is missing or no sm_100 device exists.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Sequence

import numpy as np

__all__ = ["FLOAT32", "FLOAT16", "BFLOAT16", "View", "MagB200Error", "lib", "lib_path", "Tensor",
           "device_count", "synchronize", "KERNEL_NAMES"]

FLOAT32, FLOAT16, BFLOAT16 = 0, 1, 2          # mag_dtype_t values (include/magnetron/magnetron.h:171-174)
DTYPE_SIZE = {FLOAT32: 4, FLOAT16: 2, BFLOAT16: 2}
BITS_DTYPE = {FLOAT32: np.uint32, FLOAT16: np.uint16, BFLOAT16: np.uint16}
MAX_DIMS = 16
KERNEL_NAMES = {0: "none", 1: "tcgen05", 2: "skinny", 3: "simt", 4: "skinny_splitk", 5: "tcgen05_2sm", 6: "tcgen05_f32x3"}
KERNEL_IDS = {v: k for k, v in KERNEL_NAMES.items()}

_PKG = os.path.dirname(os.path.abspath(__file__))


class View(C.Structure):
    """magb200_view_t"""
    _fields_ = [("base", C.c_void_p), ("offset", C.c_int64), ("dtype", C.c_int32), ("rank", C.c_int32),
                ("shape", C.c_int64 * MAX_DIMS), ("strides", C.c_int64 * MAX_DIMS)]


class TpPlan(C.Structure):
    """magb200_tp_plan_t"""
    _fields_ = [("mode", C.c_int32), ("exchange", C.c_int32), ("chunks", C.c_int32), ("pays", C.c_int32),
                ("single_us", C.c_double), ("sharded_us", C.c_double), ("speedup", C.c_double)]


TP_REPLICATE, TP_COLUMN, TP_ROW = 0, 1, 2
TP_EXCHANGE = {0: "none", 1: "nccl", 2: "scatter", 3: "switch"}


class MagB200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"magb200 error {code}: {message}")
        self.code = code


ERR_NO_DEVICE, ERR_INVALID_ARG, ERR_SHAPE, ERR_CUDA, ERR_OOM, ERR_TIMEOUT, ERR_TOO_LARGE = -1, -2, -3, -4, -5, -6, -7


def lib_path() -> str:
    return os.path.join(_PKG, "lib", "libmagnetron_b200.so")


_lib = None

# name -> (restype, argtypes); one entry per declaration in include/magnetron_b200.h
_VP = C.POINTER(View)

SIGNATURES = {
    "magb200_last_error": (C.c_char_p, []),
    "magb200_device_count": (C.c_int, []),
    "magb200_device_name": (C.c_int, [C.c_int, C.c_char_p, C.c_size_t]),
    "magb200_device_init": (C.c_int, [C.c_int]),
    "magb200_device_shutdown": (C.c_int, [C.c_int]),
    "magb200_synchronize": (C.c_int, [C.c_int]),
    "magb200_set_stream": (C.c_int, [C.c_int, C.c_void_p]),
    "magb200_get_stream": (C.c_void_p, [C.c_int]),
    "magb200_set_cta_limit": (C.c_int, [C.c_int, C.c_int]),
    "magb200_malloc": (C.c_int, [C.c_int, C.POINTER(C.c_void_p), C.c_size_t]),
    "magb200_free": (C.c_int, [C.c_int, C.c_void_p]),
    "magb200_upload": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t]),
    "magb200_download": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t]),
    "magb200_upload_async": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t]),
    "magb200_download_async": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t]),
    "magb200_upload_overlapped": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t]),
    "magb200_download_overlapped": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_size_t]),
    "magb200_host_alloc_pinned": (C.c_int, [C.POINTER(C.c_void_p), C.c_size_t]),
    "magb200_host_free_pinned": (C.c_int, [C.c_void_p]),
    "magb200_cast": (C.c_int, [C.c_int, _VP, _VP]),
    "magb200_clone": (C.c_int, [C.c_int, _VP, _VP]),
    "magb200_fill": (C.c_int, [C.c_int, _VP, C.c_double]),
    "magb200_cat": (C.c_int, [C.c_int, C.POINTER(_VP), C.c_int, C.c_int, _VP]),
    "magb200_matmul": (C.c_int, [C.c_int, _VP, _VP, _VP]),
    "magb200_upload_2d": (C.c_int, [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t]),
    "magb200_matmul_route": (C.c_int, [_VP, _VP, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "magb200_decode_plan": (C.c_int, [_VP, _VP] + [C.POINTER(C.c_int)] * 5 + [C.POINTER(C.c_int64)]),
    "magb200_set_decode_cluster": (C.c_int, [C.c_int]),
    "magb200_set_gemm_overlap": (C.c_int, [C.c_int]),
    "magb200_overlapped_launch_count": (C.c_uint64, []),
    "magb200_set_decode_row_streaming": (C.c_int, [C.c_int]),
    "magb200_set_small_output_split": (C.c_int, [C.c_int]),
    "magb200_matmul_swiglu": (C.c_int, [C.c_int, _VP, _VP, _VP, _VP]),
    "magb200_matmul_grouped": (C.c_int, [C.c_int, _VP, C.c_int, C.POINTER(_VP), C.POINTER(_VP)]),
    "magb200_matmul_result_shape": (C.c_int, [_VP, _VP, C.POINTER(C.c_int32), C.POINTER(C.c_int64)]),
    "magb200_last_kernel": (C.c_int, []),
    "magb200_launch_count": (C.c_uint64, []),
    "magb200_launch_count_reset": (None, []),
    "magb200_force_kernel": (C.c_int, [C.c_int]),
    "magb200_set_wait_limit_ns": (C.c_int, [C.c_uint64]),
    "magb200_get_wait_limit_ns": (C.c_uint64, []),
    "magb200_test_leave_stage_unarmed": (C.c_int, [C.c_int]),
    "magb200_test_inject_fault": (C.c_int, [C.c_int, C.c_int]),
    "magb200_pool_stats": (C.c_int, [C.c_int] + [C.POINTER(C.c_uint64)] * 4),
    "magb200_pool_trim": (C.c_int, [C.c_int]),
    "magb200_mem_info": (C.c_int, [C.c_int, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "magb200_set_balanced_last_wave": (C.c_int, [C.c_int]),
    "magb200_matmul_scatter": (C.c_int, [C.c_int, _VP, _VP, C.POINTER(C.c_void_p), C.c_int, C.c_int]),
    "magb200_reduce_broadcast": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int]),
    "magb200_tp_plan": (C.c_int, [C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(TpPlan)]),
    "magb200_multimem_reduce_broadcast": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int64, C.c_int, C.c_int]),
    "magb200_matmul_skinny_noalloc": (C.c_int, [C.c_int, C.c_void_p, _VP, _VP, _VP]),
    "magb200_matmul_host": (C.c_int, [C.c_int, _VP, C.c_size_t, _VP, C.c_size_t, _VP]),
    "magb200_cast_host": (C.c_int, [C.c_int, _VP, C.c_size_t, _VP]),
    "magb200_graph_begin_capture": (C.c_int, [C.c_int]),
    "magb200_graph_end_capture": (C.c_int, [C.c_int, C.POINTER(C.c_void_p)]),
    "magb200_graph_launch": (C.c_int, [C.c_int, C.c_void_p]),
    "magb200_graph_destroy": (C.c_int, [C.c_void_p]),
    "magb200_event_create": (C.c_int, [C.POINTER(C.c_void_p)]),
    "magb200_event_destroy": (C.c_int, [C.c_void_p]),
    "magb200_event_record": (C.c_int, [C.c_int, C.c_void_p]),
    "magb200_event_elapsed_ms": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_float)]),
}


def lib():
    """The loaded C-ABI library. Raises when it has not been built: there is no other code path."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise ImportError(f"{path} is missing: build it with `python -m magnetron_b200.build` (needs nvcc); "
                              "magnetron_b200 has no CPU fallback")
        handle = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(code: int) -> None:
    if code != 0:
        raise MagB200Error(code, lib().magb200_last_error().decode(errors="replace"))


def device_count() -> int:
    return lib().magb200_device_count()


def synchronize(device: int = 0) -> None:
    check(lib().magb200_synchronize(device))


def force_kernel(name: str | None) -> None:
    """Pin matmul routing to one kernel ("tcgen05", "tcgen05_2sm", "tcgen05_f32x3", "skinny", "simt") or restore automatic routing."""
    check(lib().magb200_force_kernel(KERNEL_IDS[name] if name else 0))


def last_kernel() -> str:
    return KERNEL_NAMES[lib().magb200_last_kernel()]


def contiguous_strides(shape: Sequence[int]) -> tuple:
    out, acc = [], 1
    for n in reversed(shape):
        out.append(acc)
        acc *= n
    return tuple(reversed(out))


def make_view(base: int, dtype: int, shape: Sequence[int], strides: Sequence[int] | None = None, offset: int = 0) -> View:
    if strides is None:
        strides = contiguous_strides(shape)
    v = View()
    v.base, v.offset, v.dtype, v.rank = base, offset, dtype, len(shape)
    for i, (n, s) in enumerate(zip(shape, strides)):
        v.shape[i], v.strides[i] = n, s
    return v


def solve_view_strides(old_shape, old_strides, new_shape):
    """Strides that let `new_shape` alias the same elements, or None when a copy is needed.
    Chunk matching as in the reference's view solver (magnetron/core/mag_coords.c:119-178): walk the
    old dims from the innermost outwards, close a chunk wherever the next-outer old dim does not
    continue it contiguously, and tile each chunk exactly with new dims; size-1 dims of the new shape
    get stride 0 as there (:133-136)."""
    old_shape, old_strides, new_shape = list(old_shape), list(old_strides), list(new_shape)
    numel = int(np.prod(old_shape)) if old_shape else 1
    if numel != (int(np.prod(new_shape)) if new_shape else 1):
        return None
    new_strides = [0] * len(new_shape)
    vd = len(new_shape) - 1
    base = old_strides[-1] if old_strides else 1
    t_numel = v_numel = 1
    for td in range(len(old_shape) - 1, -1, -1):
        t_numel *= old_shape[td]
        closes = td == 0 or (old_shape[td - 1] != 1 and old_strides[td - 1] != t_numel * base)
        if not closes:
            continue
        while vd >= 0 and (v_numel < t_numel or new_shape[vd] == 1):
            new_strides[vd] = v_numel * base
            v_numel *= new_shape[vd]
            vd -= 1
        if v_numel != t_numel:
            return None
        if td > 0:
            base = old_strides[td - 1]
            t_numel = v_numel = 1
    if vd != -1:
        return None
    return tuple(0 if n == 1 else s for n, s in zip(new_shape, new_strides))


class Tensor:
    """A device tensor header: storage pointer + dtype, shape, strides (elements), storage offset --
    the fields of `mag_tensor_t` that a backend reads (magnetron/core/mag_tensor.h:52-68). Views share
    the storage of their base; the storage is freed when the owning tensor is released."""

    def __init__(self, device: int, dtype: int, shape, strides=None, *, base_ptr: int | None = None,
                 offset: int = 0, owner: "Tensor | None" = None, storage_elems: int | None = None):
        self.device, self.dtype = device, dtype
        self.shape = tuple(int(s) for s in shape)
        self.strides = tuple(int(s) for s in (strides if strides is not None else contiguous_strides(self.shape)))
        self.offset = offset
        self._owner = owner
        if base_ptr is None:  # mag_empty (include/magnetron/magnetron.h:210)
            n = int(np.prod(self.shape)) if self.shape else 1
            p = C.c_void_p()
            check(lib().magb200_malloc(device, C.byref(p), max(n, 1) * DTYPE_SIZE[dtype]))
            self.ptr = p.value
            self.storage_elems = n
            self._owns = True
        else:
            self.ptr = base_ptr
            self.storage_elems = storage_elems
            self._owns = False

    # ---- lifetime ----
    def release(self):
        if self._owns and self.ptr:
            check(lib().magb200_free(self.device, self.ptr))
            self.ptr = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass

    # ---- data in / out (mag_copy_raw_, mag_tensor_copy_data) ----
    @classmethod
    def from_bits(cls, device: int, dtype: int, bits: np.ndarray) -> "Tensor":
        bits = np.ascontiguousarray(bits, dtype=BITS_DTYPE[dtype])
        t = cls(device, dtype, bits.shape if bits.ndim else (1,))
        check(lib().magb200_upload(device, t.ptr, bits.ctypes.data, bits.nbytes))
        return t

    def to_bits(self) -> np.ndarray:
        src = self if self.is_contiguous() else self.contiguous()
        out = np.empty(src.shape, dtype=BITS_DTYPE[self.dtype])
        check(lib().magb200_download(self.device, out.ctypes.data, src.ptr + src.offset * DTYPE_SIZE[self.dtype], out.nbytes))
        return out

    # ---- header-only views ----
    @property
    def numel(self) -> int:
        return int(np.prod(self.shape)) if self.shape else 1

    @property
    def rank(self) -> int:
        return len(self.shape)

    def view_struct(self) -> View:
        return make_view(self.ptr, self.dtype, self.shape, self.strides, self.offset)

    def is_contiguous(self) -> bool:
        expect = 1
        for n, s in zip(reversed(self.shape), reversed(self.strides)):
            if n != 1 and s != expect:
                return False
            expect *= n
        return True

    def _alias(self, shape, strides, offset=None) -> "Tensor":
        return Tensor(self.device, self.dtype, shape, strides, base_ptr=self.ptr,
                      offset=self.offset if offset is None else offset, owner=self._owner or self,
                      storage_elems=self.storage_elems)

    def as_strided(self, shape, strides, offset=0) -> "Tensor":       # mag_as_strided
        return self._alias(shape, strides, offset)

    def transpose(self, d0: int, d1: int) -> "Tensor":                 # mag_transpose
        sh, st = list(self.shape), list(self.strides)
        sh[d0], sh[d1] = sh[d1], sh[d0]
        st[d0], st[d1] = st[d1], st[d0]
        return self._alias(sh, st)

    @property
    def T(self) -> "Tensor":                                           # mag_T
        return self.transpose(self.rank - 2, self.rank - 1) if self.rank >= 2 else self

    def permute(self, dims) -> "Tensor":                               # mag_permute
        return self._alias([self.shape[d] for d in dims], [self.strides[d] for d in dims])

    def view(self, shape) -> "Tensor":                                 # mag_view
        st = solve_view_strides(self.shape, self.strides, tuple(shape))
        if st is None:
            raise MagB200Error(ERR_SHAPE, "view: the shape is not expressible as a view of these strides")
        return self._alias(shape, st)

    def reshape(self, shape) -> "Tensor":                              # mag_reshape: view when possible, else copy
        st = solve_view_strides(self.shape, self.strides, tuple(shape))
        return self._alias(shape, st) if st is not None else self.contiguous().view(shape)

    def slice(self, dim: int, start: int, length: int, step: int = 1) -> "Tensor":   # mag_view_slice
        sh, st = list(self.shape), list(self.strides)
        sh[dim] = length
        st[dim] = self.strides[dim] * step
        return self._alias(sh, st, self.offset + start * self.strides[dim])

    # ---- operators ----
    def contiguous(self) -> "Tensor":                                  # mag_contiguous -> MAG_OP_CLONE
        out = Tensor(self.device, self.dtype, self.shape)
        check(lib().magb200_clone(self.device, C.byref(self.view_struct()), C.byref(out.view_struct())))
        return out

    def cast(self, dtype: int) -> "Tensor":                            # mag_cast -> MAG_OP_CAST
        out = Tensor(self.device, dtype, self.shape)
        check(lib().magb200_cast(self.device, C.byref(self.view_struct()), C.byref(out.view_struct())))
        return out

    @staticmethod
    def cat(tensors: Sequence["Tensor"], dim: int) -> "Tensor":        # mag_cat -> MAG_OP_CAT
        t0 = tensors[0]
        shape = list(t0.shape)
        shape[dim] = sum(t.shape[dim] for t in tensors)
        out = Tensor(t0.device, t0.dtype, shape)
        views = [t.view_struct() for t in tensors]
        arr = (_VP * len(views))(*[C.pointer(v) for v in views])
        check(lib().magb200_cat(t0.device, arr, len(views), dim, C.byref(out.view_struct())))
        return out

    def matmul(self, other: "Tensor") -> "Tensor":                     # mag_matmul -> MAG_OP_MATMUL
        rank = C.c_int32()
        shape = (C.c_int64 * (MAX_DIMS + 2))()
        xv, yv = self.view_struct(), other.view_struct()
        check(lib().magb200_matmul_result_shape(C.byref(xv), C.byref(yv), C.byref(rank), shape))
        out = Tensor(self.device, self.dtype, [shape[i] for i in range(rank.value)])
        check(lib().magb200_matmul(self.device, C.byref(xv), C.byref(yv), C.byref(out.view_struct())))
        return out

    __matmul__ = matmul

    def matmul_swiglu(self, w_gate: "Tensor", w_up: "Tensor") -> "Tensor":   # silu(self @ w_gate) * (self @ w_up)
        rank = C.c_int32()
        shape = (C.c_int64 * (MAX_DIMS + 2))()
        xv, gv, uv = self.view_struct(), w_gate.view_struct(), w_up.view_struct()
        check(lib().magb200_matmul_result_shape(C.byref(xv), C.byref(gv), C.byref(rank), shape))
        out = Tensor(self.device, self.dtype, [shape[i] for i in range(rank.value)])
        check(lib().magb200_matmul_swiglu(self.device, C.byref(xv), C.byref(gv), C.byref(uv), C.byref(out.view_struct())))
        return out
