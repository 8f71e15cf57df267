"""The drop-in boundary: libmagnetron_cuda.so next to the UNMODIFIED reference core, driven through the
reference's own C API (mag_ctx_create("cuda:0"), mag_transpose, mag_view, mag_matmul, mag_cast ...)."""
import ctypes as C
import os
import shutil
import tempfile

import numpy as np
import pytest

import magnetron_b200 as mb
from oracle import mag_oracle as O
from oracle import ref_driver as R
from tests import cases
from tests.common import unit_roundoff

PLUGIN = os.path.join(os.path.dirname(mb.lib_path()), "libmagnetron_cuda.so")
needs_ref = pytest.mark.skipif(not (R.available() and os.path.exists(PLUGIN)),
                               reason="needs oracle/_ref (reference core) and the built backend module")


@pytest.fixture(scope="module")
def deploy_dir():
    """A directory laid out like an installed magnetron: core + cpu module + our cuda module side by side
    (the loader looks for libmagnetron_<id>.so next to libmagnetron_core.so, magnetron/core/mag_backend.c:209-220)."""
    d = tempfile.mkdtemp(prefix="magdeploy_")
    # real copies, not symlinks: the core resolves its own real path to find its modules (magnetron/core/mag_os.c:32-54)
    for name in ("libmagnetron_core.so", "libmagnetron_cpu.so"):
        shutil.copy2(os.path.join(R.REF_DIR, name), os.path.join(d, name))
    shutil.copy2(PLUGIN, os.path.join(d, "libmagnetron_cuda.so"))
    yield d
    shutil.rmtree(d, ignore_errors=True)


def plugin_handle(deploy_dir):
    C.CDLL(os.path.join(deploy_dir, "libmagnetron_core.so"), mode=C.RTLD_GLOBAL)
    return C.CDLL(os.path.join(deploy_dir, "libmagnetron_cuda.so"), mode=C.RTLD_GLOBAL)


@needs_ref
def test_module_hooks_and_cookie(deploy_dir):
    h = plugin_handle(deploy_dir)
    for sym in ("mag_backend_module_hook_abi_cookie", "mag_backend_module_hook_init", "mag_backend_module_hook_shutdown",
                "mag_b200_upload", "mag_b200_download", "mag_b200_synchronize"):
        assert hasattr(h, sym), sym
    h.mag_backend_module_hook_abi_cookie.restype = C.c_uint32
    assert h.mag_backend_module_hook_abi_cookie() == (ord("M") | ord("A") << 8 | ord("G") << 16 | 1 << 24)


@needs_ref
def test_context_without_gpu_falls_back_to_cpu_cleanly(deploy_dir):
    """Without a device the module declines (init returns false) and the core falls back to cpu:0
    (magnetron/core/mag_context.c:158-174); nothing crashes and matmul still answers from the CPU backend."""
    if mb.device_count() > 0:
        pytest.skip("a device is present")
    api = R.MagApi("cuda:0", lib_dir=deploy_dir, log_level=1)
    try:
        assert api.device_name == api.cpu_name
        a = api.from_bits(R.FLOAT32, np.ones((2, 2), np.float32).view(np.uint32))
        r = api.matmul(a, a)
        assert np.array_equal(api.to_bits(r).view(np.float32), np.full((2, 2), 2.0, np.float32))
        r.release(); a.release()
    finally:
        api.close()


class CudaApi(R.MagApi):
    """The same driver on "cuda:0", with data movement through the module's additive exports."""

    def __init__(self, deploy_dir):
        super().__init__("cuda:0", lib_dir=deploy_dir, log_level=int(os.environ.get("MAG_TEST_LOG_LEVEL", "1")))
        self.mod = plugin_handle(deploy_dir)
        self.mod.mag_b200_upload.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        self.mod.mag_b200_download.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        self.mod.mag_b200_synchronize.argtypes = [C.c_void_p]

    def from_bits(self, dtype, bits):
        bits = np.ascontiguousarray(bits, dtype=R.DTYPE_NP[dtype])
        t = self.empty(dtype, bits.shape if bits.ndim else (1,))
        assert self.mod.mag_b200_upload(t.ptr, bits.ctypes.data, bits.nbytes) == 0
        return t

    def to_bits(self, t):
        c = t if self.lib.mag_tensor_is_contiguous(t.ptr) else self.contiguous(t)
        out = np.empty(c.shape, dtype=R.DTYPE_NP[c.dtype])
        assert self.mod.mag_b200_download(c.ptr, out.ctypes.data, out.nbytes) == 0
        if c is not t:
            c.release()
        return out


@pytest.mark.gpu
@needs_ref
def test_matmul_and_cast_through_the_reference_api(deploy_dir, gpu):
    api = CudaApi(deploy_dir)
    try:
        assert "B200" in api.device_name
        dt = R.BFLOAT16
        rng = np.random.default_rng(0)
        xb = O.f32_to_bits(dt, cases.gen_storage(rng, (512, 2048), 1.0))
        wb = O.f32_to_bits(dt, cases.gen_storage(rng, (2048, 2048), 0.02))
        x, w = api.from_bits(dt, xb), api.from_bits(dt, wb)
        wt = api.transpose(w, 0, 1)                       # W.T: shape (K,N), strides (1,K)
        assert wt.strides == (1, 2048)
        r = api.matmul(x, wt)
        got = api.to_bits(r)
        xf, wf = O.bits_to_f64(dt, xb), O.bits_to_f64(dt, wb)
        m = O.error_metrics(dt, got, xf @ wf.T, np.abs(xf) @ np.abs(wf).T)
        assert m["e"] <= unit_roundoff(dt) + 2048 * 2.0 ** -24, m
        # cast both ways, bit exact with the oracle
        f = api.cast(r, R.FLOAT32)
        assert np.array_equal(api.to_bits(f), O.cast_bits(dt, R.FLOAT32, got))
        x32 = api.from_bits(R.FLOAT32, cases.cast_inputs_f32(1, 1 << 16))
        h = api.cast(x32, R.FLOAT16)
        assert np.array_equal(api.to_bits(h), O.cast_bits(R.FLOAT32, R.FLOAT16, cases.cast_inputs_f32(1, 1 << 16)))
        # strided view -> contiguous (MAG_OP_CLONE), then a decode-shaped product
        wc = api.contiguous(wt)
        assert np.array_equal(api.to_bits(wc), np.ascontiguousarray(wb.T))
        x1 = api.from_bits(dt, xb[:1])
        r1 = api.matmul(x1, wt)
        m1 = O.error_metrics(dt, api.to_bits(r1), xf[:1] @ wf.T, np.abs(xf[:1]) @ np.abs(wf).T)
        assert m1["e"] <= unit_roundoff(dt) + 2048 * 2.0 ** -24, m1
        for t in (r1, x1, wc, h, x32, f, r, wt, w, x):
            t.release()
    finally:
        api.close()   # leak detection on: every storage must have been returned


@pytest.mark.gpu
@needs_ref
def test_gqa_broadcast_views_through_the_reference_api(deploy_dir, gpu):
    """Q.reshape(B,KV,G,T,D) @ K.transpose(2,3).view(B,KV,1,D,T): the view solver's stride-0 broadcast dim
    arrives at the backend untouched."""
    api = CudaApi(deploy_dir)
    try:
        dt = R.FLOAT16
        B, KV, G, T, D = 1, 2, 4, 128, 64
        rng = np.random.default_rng(4)
        q = O.f32_to_bits(dt, cases.gen_storage(rng, (B, KV, G, T, D), 1.0))
        k = O.f32_to_bits(dt, cases.gen_storage(rng, (B, KV, T, D), 1.0))
        tq, tk = api.from_bits(dt, q), api.from_bits(dt, k)
        kt = api.transpose(tk, 2, 3)
        kv = api.view(kt, (B, KV, 1, D, T))
        assert kv.strides[2] == 0
        s = api.matmul(tq, kv)
        assert s.shape == (B, KV, G, T, T)
        qf, kf = O.bits_to_f64(dt, q), O.bits_to_f64(dt, k)
        truth = np.einsum("bhgtd,bhsd->bhgts", qf, kf)
        m = O.error_metrics(dt, api.to_bits(s), truth, np.einsum("bhgtd,bhsd->bhgts", np.abs(qf), np.abs(kf)))
        assert m["e"] <= unit_roundoff(dt) + D * 2.0 ** -24, m
        for t in (s, kv, kt, tk, tq):
            t.release()
    finally:
        api.close()


@pytest.mark.gpu
@needs_ref
def test_unsupported_opcode_returns_a_status(deploy_dir, gpu):
    """Opcodes outside the path come back as a status code, not as an abort."""
    api = CudaApi(deploy_dir)
    try:
        api.lib.mag_softmax.restype = C.c_int
        api.lib.mag_softmax.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p]
        x = api.from_bits(R.FLOAT32, np.zeros((4, 4), np.uint32))
        err, out = R.MagError(), C.c_void_p()
        st = api.lib.mag_softmax(C.byref(err), C.byref(out), x.ptr)
        assert st != 0
        if out.value:
            api.lib.mag_tensor_decref(out.value)
        x.release()
    finally:
        api.close(True)
