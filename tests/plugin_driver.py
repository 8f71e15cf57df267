"""Bodies of the backend-module GPU tests, run in a process of their own (`python -m tests.plugin_driver <case> <dir>`).

A fresh process matters: the reference core resolves its module directory and its own exported symbols process-wide,
so a second copy of libmagnetron_core.so loaded next to one that is already there (the CPU checker of other tests) would
look for backends in the first copy's directory. It also keeps the reference's abort-on-leak away from the test runner."""
import ctypes as C
import sys

import numpy as np

from oracle import mag_oracle as O
from oracle import ref_driver as R
from tests import cases
from tests.common import unit_roundoff


def plugin_handle(deploy_dir):
    import os
    C.CDLL(os.path.join(deploy_dir, "libmagnetron_core.so"), mode=C.RTLD_GLOBAL)
    return C.CDLL(os.path.join(deploy_dir, "libmagnetron_cuda.so"), mode=C.RTLD_GLOBAL)


def finish(api, ok: bool):
    """Destroy the context; with leak detection on only when the test body got through (a failed body leaves tensors
    alive on purpose-less paths, and the reference aborts the process on leaks, magnetron/core/mag_context.c:187-197)."""
    api.close(suppress_leak_detection=not ok)


class CudaApi(R.MagApi):
    """The same driver on "cuda:0", with data movement through the module's additive exports."""

    def __init__(self, deploy_dir):
        super().__init__("cuda:0", lib_dir=deploy_dir, log_level=1)
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


def test_matmul_and_cast_through_the_reference_api(deploy_dir):
    api = CudaApi(deploy_dir)
    ok = False
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
        ok = True
    finally:
        finish(api, ok)   # leak detection on: every storage must have been returned


def test_gqa_broadcast_views_through_the_reference_api(deploy_dir):
    """Q.reshape(B,KV,G,T,D) @ K.transpose(2,3).view(B,KV,1,D,T): the view solver's stride-0 broadcast dim
    arrives at the backend untouched."""
    api = CudaApi(deploy_dir)
    ok = False
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
        ok = True
    finally:
        finish(api, ok)


def test_unsupported_opcode_returns_a_status(deploy_dir):
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


def _cat(api, tensors, dim):
    api.lib.mag_cat.restype = C.c_int
    api.lib.mag_cat.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_size_t, C.c_int64]
    arr = (C.c_void_p * len(tensors))(*[t.ptr for t in tensors])
    return api._call(api.lib.mag_cat, arr, len(tensors), dim)


def test_kv_append_through_the_reference_api(deploy_dir):
    """mag_cat of a KV cache [B,H,T,D] with one new position, then scores against the grown cache: MAG_OP_CAT on the device
    must give the bits that the reference CPU backend gives for the same call (both contexts live in this process, same core)."""
    gpu_api = CudaApi(deploy_dir)
    cpu_api = R.MagApi("cpu", lib_dir=deploy_dir, log_level=1)
    ok = False
    try:
        dt = R.BFLOAT16
        B, H, T, D = 2, 8, 37, 128
        rng = np.random.default_rng(11)
        cache = O.f32_to_bits(dt, cases.gen_storage(rng, (B, H, T, D), 1.0))
        new = O.f32_to_bits(dt, cases.gen_storage(rng, (B, H, 1, D), 1.0))
        q = O.f32_to_bits(dt, cases.gen_storage(rng, (B, H, 1, D), 1.0))
        results = []
        for api in (gpu_api, cpu_api):
            tc, tn, tq = api.from_bits(dt, cache), api.from_bits(dt, new), api.from_bits(dt, q)
            grown = _cat(api, [tc, tn], 2)
            assert grown.shape == (B, H, T + 1, D)
            kt = api.transpose(grown, 2, 3)
            s = api.matmul(tq, kt)
            results.append((api.to_bits(grown), api.to_bits(s)))
            for t in (s, kt, grown, tq, tn, tc):
                t.release()
        assert np.array_equal(results[0][0], results[1][0])                     # the concat is a copy: bit exact
        assert np.array_equal(results[0][0], np.concatenate([cache, new], axis=2))
        qf, kf = O.bits_to_f64(dt, q), O.bits_to_f64(dt, results[0][0])
        truth = np.einsum("bhqd,bhtd->bhqt", qf, kf)
        m = O.error_metrics(dt, results[0][1], truth, np.einsum("bhqd,bhtd->bhqt", np.abs(qf), np.abs(kf)))
        assert m["e"] <= unit_roundoff(dt) + D * 2.0 ** -24, m
        ok = True
    finally:
        cpu_api.close(not ok)
        finish(gpu_api, ok)


def test_gated_mlp_through_the_module_export(deploy_dir):
    """mag_b200_matmul_swiglu on "cuda:0" against mag_matmul, mag_matmul, mag_silu, mag_mul on the reference CPU backend of the
    same process, in the reference operator tests' 16-bit tolerance."""
    gpu_api = CudaApi(deploy_dir)
    cpu_api = R.MagApi("cpu", lib_dir=deploy_dir, log_level=1)
    ok = False
    try:
        dt = R.BFLOAT16
        M, N, K = 512, 768, 256
        rng = np.random.default_rng(23)
        xb = O.f32_to_bits(dt, cases.gen_storage(rng, (M, K), 1.0))
        gb = O.f32_to_bits(dt, cases.gen_storage(rng, (N, K), 0.05))
        ub = O.f32_to_bits(dt, cases.gen_storage(rng, (N, K), 0.05))
        # device: one call
        tx, tg, tu = gpu_api.from_bits(dt, xb), gpu_api.from_bits(dt, gb), gpu_api.from_bits(dt, ub)
        gt, ut = gpu_api.transpose(tg, 0, 1), gpu_api.transpose(tu, 0, 1)
        out = gpu_api.empty(dt, (M, N))
        fn = gpu_api.mod.mag_b200_matmul_swiglu
        fn.restype, fn.argtypes = C.c_int, [C.c_void_p] * 4
        assert fn(tx.ptr, gt.ptr, ut.ptr, out.ptr) == 0
        got = O.bits_to_f64(dt, gpu_api.to_bits(out))
        for t in (out, ut, gt, tu, tg, tx):
            t.release()
        # reference: the four operators
        rx, rg, ru = cpu_api.from_bits(dt, xb), cpu_api.from_bits(dt, gb), cpu_api.from_bits(dt, ub)
        rgt, rut = cpu_api.transpose(rg, 0, 1), cpu_api.transpose(ru, 0, 1)
        mg, mu = cpu_api.matmul(rx, rgt), cpu_api.matmul(rx, rut)
        sg = cpu_api.silu(mg)
        rr = cpu_api.mul(sg, mu)
        ref = O.bits_to_f64(dt, cpu_api.to_bits(rr))
        for t in (rr, sg, mu, mg, rut, rgt, ru, rg, rx):
            t.release()
        assert np.all(np.abs(got - ref) <= 1e-2 * max(1.0, np.abs(ref).max()) + 1e-2 * np.abs(ref))
        ok = True
    finally:
        cpu_api.close(not ok)
        finish(gpu_api, ok)


def test_snapshot_tensors_to_the_device(deploy_dir):
    """A .mag snapshot written and read back by the reference itself (CPU context; its tensors borrow the mapped file) goes to
    "cuda:0" through mag_b200_tensor_to_device: whole, as the row block of a column-sharded weight and as the K slice of a
    row-sharded one; every copy is bit-compared with the numpy slice, and the shards reproduce the unsharded product."""
    import os
    import tempfile
    gpu_api = CudaApi(deploy_dir)
    cpu_api = R.MagApi("cpu", lib_dir=deploy_dir, log_level=1)
    lib = cpu_api.lib
    P = C.c_void_p
    for name, res, args in (("mag_snapshot_new", P, [P]), ("mag_snapshot_deserialize", P, [P, C.c_char_p]),
                            ("mag_snapshot_serialize", C.c_bool, [P, C.c_char_p]), ("mag_snapshot_get_tensor", P, [P, C.c_char_p]),
                            ("mag_snapshot_put_tensor", C.c_bool, [P, C.c_char_p, P]), ("mag_snapshot_free", None, [P])):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    to_device = gpu_api.mod.mag_b200_tensor_to_device
    to_device.restype, to_device.argtypes = C.c_int, [P, P, C.c_int64, C.c_int64, C.c_int64, C.POINTER(P)]
    ok = False
    tmp = tempfile.mkdtemp(prefix="magsnap_")
    path = os.path.join(tmp, "weights.mag").encode()
    try:
        dt = R.BFLOAT16
        N, K, M, ranks = 512, 384, 256, 2
        rng = np.random.default_rng(31)
        wb = O.f32_to_bits(dt, cases.gen_storage(rng, (N, K), 0.05))
        f32b = rng.standard_normal((3, 5, 7), dtype=np.float32).view(np.uint32)
        snap = lib.mag_snapshot_new(cpu_api.ctx)
        tw, tf = cpu_api.from_bits(dt, wb), cpu_api.from_bits(R.FLOAT32, f32b)
        assert lib.mag_snapshot_put_tensor(snap, b"layer.weight", tw.ptr) and lib.mag_snapshot_put_tensor(snap, b"misc.f32", tf.ptr)
        assert lib.mag_snapshot_serialize(snap, path)
        lib.mag_snapshot_free(snap)
        tw.release(); tf.release()
        snap = lib.mag_snapshot_deserialize(cpu_api.ctx, path)
        assert snap
        src_w, src_f = lib.mag_snapshot_get_tensor(snap, b"layer.weight"), lib.mag_snapshot_get_tensor(snap, b"misc.f32")
        assert src_w and src_f

        def upload(src, dim, r, n):
            out = P()
            assert to_device(gpu_api.ctx, src, dim, r, n, C.byref(out)) == 0
            return R.Tensor(gpu_api, out.value)

        whole = upload(src_w, -1, 0, 1)
        assert np.array_equal(gpu_api.to_bits(whole), wb)
        f = upload(src_f, -1, 0, 1)
        assert np.array_equal(gpu_api.to_bits(f), f32b)
        mid = upload(src_f, 1, 3, 5)                       # one of five slices of the middle dim of a rank-3 tensor
        assert np.array_equal(gpu_api.to_bits(mid), f32b[:, 3:4, :])
        rows = [upload(src_w, 0, r, ranks) for r in range(ranks)]       # column-sharded nn.Linear: rows of W
        cols = [upload(src_w, 1, r, ranks) for r in range(ranks)]       # row-sharded: K slices of W
        for r in range(ranks):
            assert np.array_equal(gpu_api.to_bits(rows[r]), wb[r * (N // ranks):(r + 1) * (N // ranks)])
            assert np.array_equal(gpu_api.to_bits(cols[r]), wb[:, r * (K // ranks):(r + 1) * (K // ranks)])
        bad = P()
        assert to_device(gpu_api.ctx, src_f, 2, 0, 2, C.byref(bad)) != 0            # 7 is not divisible by 2
        # the column shards give the columns of the unsharded product
        xb = O.f32_to_bits(dt, cases.gen_storage(rng, (M, K), 1.0))
        x = gpu_api.from_bits(dt, xb)
        wt = gpu_api.transpose(whole, 0, 1)
        full = gpu_api.matmul(x, wt)
        full_bits = gpu_api.to_bits(full)
        for r in range(ranks):
            rt = gpu_api.transpose(rows[r], 0, 1)
            part = gpu_api.matmul(x, rt)
            assert np.array_equal(gpu_api.to_bits(part), full_bits[:, r * (N // ranks):(r + 1) * (N // ranks)])
            part.release(); rt.release()
        for t in [full, wt, x, mid, f, whole] + rows + cols:
            t.release()
        lib.mag_tensor_decref(src_w); lib.mag_tensor_decref(src_f)
        lib.mag_snapshot_free(snap)
        ok = True
    finally:
        import shutil
        shutil.rmtree(tmp, ignore_errors=True)
        cpu_api.close(not ok)
        finish(gpu_api, ok)


CASES = {"matmul_cast": test_matmul_and_cast_through_the_reference_api,
         "kv_append": test_kv_append_through_the_reference_api,
         "gated_mlp": test_gated_mlp_through_the_module_export,
         "snapshot": test_snapshot_tensors_to_the_device,
         "gqa_views": test_gqa_broadcast_views_through_the_reference_api,
         "unsupported_op": test_unsupported_opcode_returns_a_status}

if __name__ == "__main__":
    CASES[sys.argv[1]](sys.argv[2])
    print("OK", sys.argv[1])
