"""What a magnetron user calls when the B200 backend module is installed: a ctypes binding of the few entry points of
magnetron's public C API that the matmul / cast path needs, plus the module's additive transfer exports.

    mag_ctx_create("cuda:0") / mag_ctx_destroy          include/magnetron/magnetron.h:103,118
    mag_empty, mag_transpose, mag_view, mag_matmul, mag_cast, mag_cat    :210, :240-246, :372, :239
    mag_tensor_decref                                   include/magnetron/magnetron.h:398-446
    mag_b200_upload[_async] / mag_b200_download[_async] / mag_b200_synchronize / mag_b200_host_alloc   (this package's module)

`install(dir)` lays out a directory the way an installed magnetron looks -- `libmagnetron_core.so` with the backend
modules beside it (the loader looks for `libmagnetron_<id>.so` next to the core, magnetron/core/mag_backend.c:209-220) --
from a built magnetron core and this package's `lib/libmagnetron_cuda.so`. Nothing here computes anything: every operator
call goes through the unchanged core to the backend module, and a context that did not come up on the B200 is refused.
"""
from __future__ import annotations

import ctypes as C
import os
import shutil
from typing import Sequence

FLOAT32, FLOAT16, BFLOAT16 = 0, 1, 2
_PKG = os.path.dirname(os.path.abspath(__file__))


class MagError(C.Structure):  # mag_error_t, include/magnetron/magnetron.h:87-93
    _fields_ = [("code", C.c_int), ("message", C.c_char * 256), ("file", C.c_char_p), ("line", C.c_int), ("func", C.c_char_p)]


def install(target_dir: str, core_dir: str) -> str:
    """Copy a built magnetron core (+ its CPU module) and this package's backend module side by side into `target_dir`.
    Real copies: the core resolves its own real path to find its modules."""
    os.makedirs(target_dir, exist_ok=True)
    for name in ("libmagnetron_core.so", "libmagnetron_cpu.so"):
        shutil.copy2(os.path.join(core_dir, name), os.path.join(target_dir, name))
    plugin = os.path.join(_PKG, "lib", "libmagnetron_cuda.so")
    if not os.path.exists(plugin):
        raise FileNotFoundError(f"{plugin} is missing: build it with `python -m magnetron_b200.build` where the magnetron headers are")
    shutil.copy2(plugin, os.path.join(target_dir, "libmagnetron_cuda.so"))
    return target_dir


class Context:
    """One magnetron context on "cuda:<ordinal>" of an installation directory."""

    def __init__(self, install_dir: str, ordinal: int = 0):
        self.core = core = C.CDLL(os.path.join(install_dir, "libmagnetron_core.so"), mode=C.RTLD_GLOBAL)
        self.mod = mod = C.CDLL(os.path.join(install_dir, "libmagnetron_cuda.so"), mode=C.RTLD_GLOBAL)
        P, I64 = C.c_void_p, C.c_int64
        PP, I64P = C.POINTER(C.c_void_p), C.POINTER(C.c_int64)
        for name, res, args in (
                ("mag_ctx_create", P, [C.c_char_p]), ("mag_ctx_destroy", None, [P, C.c_bool]),
                ("mag_ctx_get_compute_device_name", C.c_char_p, [P]), ("mag_ctx_grad_recorder_stop", None, [P]),
                ("mag_set_log_level", None, [C.c_int]),
                ("mag_empty", C.c_int, [P, PP, P, C.c_int, I64, I64P]), ("mag_transpose", C.c_int, [P, PP, P, I64, I64]),
                ("mag_view", C.c_int, [P, PP, P, I64P, I64]), ("mag_matmul", C.c_int, [P, PP, P, P]),
                ("mag_cast", C.c_int, [P, PP, P, C.c_int]), ("mag_cat", C.c_int, [P, PP, PP, C.c_size_t, I64]),
                ("mag_tensor_decref", C.c_bool, [P])):
            fn = getattr(core, name)
            fn.restype, fn.argtypes = res, args
        for name, args in (("mag_b200_upload", [P, P, C.c_size_t]), ("mag_b200_download", [P, P, C.c_size_t]),
                           ("mag_b200_upload_async", [P, P, C.c_size_t]), ("mag_b200_download_async", [P, P, C.c_size_t]),
                           ("mag_b200_synchronize", [P]), ("mag_b200_host_alloc", [PP, C.c_size_t]), ("mag_b200_host_free", [P])):
            fn = getattr(mod, name)
            fn.restype, fn.argtypes = C.c_int, args
        core.mag_set_log_level(1)
        self.ctx = core.mag_ctx_create(f"cuda:{ordinal}".encode())
        if not self.ctx:
            raise RuntimeError("mag_ctx_create failed")
        core.mag_ctx_grad_recorder_stop(self.ctx)       # inference path: no autograd retention of inputs
        self.device_name = core.mag_ctx_get_compute_device_name(self.ctx).decode()
        if "B200" not in self.device_name:              # the core falls back to the CPU backend silently when a module declines
            name = self.device_name
            self.close(True)
            raise RuntimeError(f'mag_ctx_create("cuda:{ordinal}") came up on "{name}": the B200 backend module is not active')

    def close(self, suppress_leak_detection: bool = False):
        if self.ctx:
            self.core.mag_ctx_destroy(self.ctx, suppress_leak_detection)
            self.ctx = None

    def _call(self, fn, *args) -> int:
        err, out = MagError(), C.c_void_p()
        st = fn(C.byref(err), C.byref(out), *args)
        if st != 0:
            raise RuntimeError(f"magnetron status {st}: {err.message.decode(errors='replace')}")
        return out.value

    def empty(self, dtype: int, shape: Sequence[int]) -> int:
        return self._call(self.core.mag_empty, self.ctx, dtype, len(shape), (C.c_int64 * len(shape))(*shape))

    def transpose(self, t: int, d0: int, d1: int) -> int:
        return self._call(self.core.mag_transpose, t, d0, d1)

    def view(self, t: int, shape: Sequence[int]) -> int:
        return self._call(self.core.mag_view, t, (C.c_int64 * len(shape))(*shape), len(shape))

    def matmul(self, x: int, y: int) -> int:
        return self._call(self.core.mag_matmul, x, y)

    def cast(self, x: int, dtype: int) -> int:
        return self._call(self.core.mag_cast, x, dtype)

    def cat(self, tensors: Sequence[int], dim: int) -> int:
        arr = (C.c_void_p * len(tensors))(*tensors)
        return self._call(self.core.mag_cat, arr, len(tensors), dim)

    def decref(self, t: int) -> None:
        self.core.mag_tensor_decref(t)

    def check(self, status: int, what: str) -> None:
        if status != 0:
            raise RuntimeError(f"{what} failed with magnetron status {status}")

    def upload(self, t: int, host_ptr: int, nbytes: int, wait: bool = True) -> None:
        self.check((self.mod.mag_b200_upload if wait else self.mod.mag_b200_upload_async)(t, host_ptr, nbytes), "upload")

    def download(self, t: int, host_ptr: int, nbytes: int, wait: bool = True) -> None:
        self.check((self.mod.mag_b200_download if wait else self.mod.mag_b200_download_async)(t, host_ptr, nbytes), "download")

    def synchronize(self) -> None:
        self.check(self.mod.mag_b200_synchronize(self.ctx), "synchronize")

    def host_alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        self.check(self.mod.mag_b200_host_alloc(C.byref(p), nbytes), "page-locked allocation")
        return p.value

    def host_free(self, ptr: int) -> None:
        self.mod.mag_b200_host_free(ptr)
