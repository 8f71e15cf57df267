"""The drop-in boundary: libmagnetron_cuda.so next to the UNMODIFIED reference core, driven through the
reference's own C API (mag_ctx_create("cuda:0"), mag_transpose, mag_view, mag_matmul, mag_cast ...)."""
import ctypes as C
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np
import pytest

import magnetron_b200 as mb
from oracle import mag_oracle as O
from oracle import ref_driver as R
from tests import cases
from tests.common import unit_roundoff

ROOT_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
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
                "mag_b200_upload", "mag_b200_download", "mag_b200_synchronize", "mag_b200_upload_async", "mag_b200_download_async",
                "mag_b200_matmul_swiglu", "mag_b200_tensor_to_device", "mag_b200_status_of"):
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


def run_in_fresh_process(case: str, deploy_dir: str):
    res = subprocess.run([sys.executable, "-m", "tests.plugin_driver", case, deploy_dir], cwd=ROOT_DIR,
                         capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and f"OK {case}" in res.stdout, res.stdout[-3000:] + res.stderr[-3000:]


@pytest.mark.gpu
@needs_ref
def test_matmul_and_cast_through_the_reference_api(deploy_dir, gpu):
    """x @ W.T, casts, contiguous() of a strided view and a decode-shaped product through mag_* calls on "cuda:0";
    the context is destroyed with leak detection on."""
    run_in_fresh_process("matmul_cast", deploy_dir)


@pytest.mark.gpu
@needs_ref
def test_gqa_broadcast_views_through_the_reference_api(deploy_dir, gpu):
    """Q.reshape(B,KV,G,T,D) @ K.transpose(2,3).view(B,KV,1,D,T): the view solver's stride-0 dim reaches the backend."""
    run_in_fresh_process("gqa_views", deploy_dir)


@pytest.mark.gpu
@needs_ref
def test_unsupported_opcode_returns_a_status(deploy_dir, gpu):
    """Opcodes outside the path come back as a status code, not as an abort."""
    run_in_fresh_process("unsupported_op", deploy_dir)


@pytest.mark.gpu
@needs_ref
def test_kv_append_through_the_reference_api(deploy_dir, gpu):
    """mag_cat (KV-cache append) and the scores against the grown cache on "cuda:0", bit-compared with the reference CPU
    backend running the same calls in the same process."""
    run_in_fresh_process("kv_append", deploy_dir)


@pytest.mark.gpu
@needs_ref
def test_gated_mlp_through_the_module_export(deploy_dir, gpu):
    """mag_b200_matmul_swiglu (additive export) against MATMUL, MATMUL, SILU, MUL on the reference CPU backend."""
    run_in_fresh_process("gated_mlp", deploy_dir)


@pytest.mark.gpu
@needs_ref
def test_snapshot_tensors_to_the_device(deploy_dir, gpu):
    """.mag snapshot (written and mapped by the reference on its CPU context) -> "cuda:0": whole tensors and the shards of a
    tensor-parallel weight, bit-compared; column shards reproduce the unsharded product."""
    run_in_fresh_process("snapshot", deploy_dir)
