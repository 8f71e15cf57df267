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


def test_injected_faults_take_the_error_paths_without_a_device():
    """A fault armed with magb200_test_inject_fault makes the next call at that site fail as if the CUDA runtime had
    returned the error, before any device is touched: cudaErrorMemoryAllocation (2) must come back as MAGB200_ERR_OOM,
    any other error as MAGB200_ERR_CUDA, and the fault is consumed by one call."""
    L = mb.lib()
    out = C.c_void_p(0x1234)
    mb.check(L.magb200_test_inject_fault(1, 2))                    # site MALLOC, cudaErrorMemoryAllocation
    assert L.magb200_malloc(0, C.byref(out), 1024) == mb.ERR_OOM
    assert out.value is None and b"injected" in L.magb200_last_error()
    mb.check(L.magb200_test_inject_fault(1, 999))                  # cudaErrorUnknown
    assert L.magb200_malloc(0, C.byref(out), 1024) == mb.ERR_CUDA
    v = mb.make_view(0x1000, mb.BFLOAT16, (4, 4))
    mb.check(L.magb200_test_inject_fault(2, 719))                  # site LAUNCH, cudaErrorLaunchFailure
    assert L.magb200_matmul(0, C.byref(v), C.byref(v), C.byref(v)) == mb.ERR_CUDA
    if mb.device_count() == 0:                                     # consumed: the next call fails for the real reason
        assert L.magb200_matmul(0, C.byref(v), C.byref(v), C.byref(v)) == mb.ERR_NO_DEVICE
    assert L.magb200_test_inject_fault(7, 1) == mb.ERR_INVALID_ARG


def test_knob_ranges():
    L = mb.lib()
    assert L.magb200_set_wait_limit_ns(10) == mb.ERR_INVALID_ARG          # below 1 ms
    assert L.magb200_set_wait_limit_ns(10 ** 12) == mb.ERR_INVALID_ARG    # above 60 s
    old = L.magb200_get_wait_limit_ns()
    assert old == 10 ** 9
    mb.check(L.magb200_set_wait_limit_ns(5 * 10 ** 6))
    assert L.magb200_get_wait_limit_ns() == 5 * 10 ** 6
    mb.check(L.magb200_set_wait_limit_ns(old))
    assert L.magb200_set_balanced_last_wave(3) == mb.ERR_INVALID_ARG
    mb.check(L.magb200_set_balanced_last_wave(1))
    mb.check(L.magb200_test_leave_stage_unarmed(-1))


STATUS_PROBE = r"""
import ctypes as C, os, sys
d = sys.argv[1]
C.CDLL(os.path.join(d, "libmagnetron_core.so"), mode=C.RTLD_GLOBAL)
h = C.CDLL(os.path.join(d, "libmagnetron_cuda.so"))
h.mag_b200_status_of.restype, h.mag_b200_status_of.argtypes = C.c_int, [C.c_int]
print(" ".join(str(h.mag_b200_status_of(int(a))) for a in sys.argv[2:]))
"""


def test_status_mapping_of_the_backend_module(tmp_path):
    """Every C-ABI code maps to a magnetron status of its own (mag_b200_status_of, exported by the backend module). Run in
    a process of its own: the module must sit next to a copy of the reference core, and a second copy of the core in
    this process would disturb the tests that drive the checker."""
    import shutil
    import subprocess
    import sys
    plugin = os.path.join(os.path.dirname(mb.lib_path()), "libmagnetron_cuda.so")
    core = os.path.join(ROOT, "oracle", "_ref", "libmagnetron_core.so")
    if not (os.path.exists(plugin) and os.path.exists(core)):
        pytest.skip("needs the backend module and the reference core it links against")
    shutil.copy2(core, tmp_path / "libmagnetron_core.so")
    shutil.copy2(plugin, tmp_path / "libmagnetron_cuda.so")
    # mag_status_t values in declaration order (include/magnetron/magnetron.h:59-75)
    names = ["OK", "PENDING", "THREAD_MISMATCH", "INVALID_RANK", "INVALID_DIM", "DIM_OVERFLOW", "INVALID_INDEX", "OUT_OF_BOUNDS",
             "INVALID_PARAM", "STRIDE_SOLVER_FAILED", "BROADCAST_IMPOSSIBLE", "OPERATOR_IMPOSSIBLE", "INVALID_STATE", "IMAGE_ERROR",
             "MEMORY_ALLOCATION_FAILED", "MEMORY_DEALLOCATION_FAILED", "UNKNOWN"]
    code = {n: i for i, n in enumerate(names)}
    want = {0: "OK", mb.ERR_OOM: "MEMORY_ALLOCATION_FAILED", mb.ERR_SHAPE: "OPERATOR_IMPOSSIBLE", mb.ERR_INVALID_ARG: "INVALID_PARAM",
            mb.ERR_TOO_LARGE: "DIM_OVERFLOW", mb.ERR_TIMEOUT: "INVALID_STATE", mb.ERR_NO_DEVICE: "INVALID_INDEX", mb.ERR_CUDA: "UNKNOWN"}
    rcs = list(want)
    res = subprocess.run([sys.executable, "-c", STATUS_PROBE, str(tmp_path)] + [str(rc) for rc in rcs], capture_output=True, text=True,
                         timeout=120)
    assert res.returncode == 0, res.stderr[-2000:]
    got = dict(zip(rcs, (int(v) for v in res.stdout.split())))
    assert got == {rc: code[n] for rc, n in want.items()}
    assert len(set(got.values())) == len(got)          # no two causes share a status


def _fake_view(dtype, shape, strides, base=0x7F0000000000):
    v = mb.View()
    v.base, v.offset, v.dtype, v.rank = base, 0, dtype, len(shape)
    for i, (n, st) in enumerate(zip(shape, strides)):
        v.shape[i], v.strides[i] = n, st
    return v


def _decode_plan(dtype, M, N, K, layout="W.T", batch=()):
    """magb200_decode_plan for x[batch..., M, K] @ y, y = W.T view of a [N, K] weight or a contiguous [K, N] weight."""
    L = mb.lib()
    xs = batch + (M, K)
    x = _fake_view(dtype, xs, mb.contiguous_strides(xs))
    y = _fake_view(dtype, (K, N), (1, K) if layout == "W.T" else (N, 1), base=0x7F1000000000)
    out = [C.c_int() for _ in range(5)]
    kch = C.c_int64()
    mb.check(L.magb200_decode_plan(C.byref(x), C.byref(y), *[C.byref(o) for o in out], C.byref(kch)))
    kind, splits, ctas, kw, cl = (o.value for o in out)
    return {"kind": kind, "splits": splits, "ctas": ctas, "kw": kw, "cluster": cl, "kch": kch.value}


def test_decode_planner_decisions():
    """The host-side planner of the decode kernels, without a device (148 SMs assumed): which kernel a shape gets, how K is cut."""
    BF, F32 = mb.BFLOAT16, mb.FLOAT32
    SMALL, RING, ROWS, NMAJOR, FFMA = 1, 2, 3, 4, 5
    # Qwen3-0.6B projections: register-load kernel, 8 warps along K; the 1024-row o / down add clusters of 2 / 4 CTAs
    q = _decode_plan(BF, 1, 2048, 1024)
    assert (q["kind"], q["kw"], q["cluster"], q["splits"]) == (SMALL, 8, 1, 1)
    o = _decode_plan(BF, 1, 1024, 2048)
    assert (o["kind"], o["kw"], o["cluster"], o["ctas"]) == (SMALL, 8, 2, 128)
    down = _decode_plan(BF, 8, 1024, 3072)
    assert (down["kind"], down["kw"], down["cluster"], down["ctas"]) == (SMALL, 8, 4, 256)
    # 384 row tiles (gate + up of the 0.6B model as one group has this count): 4 warps along K keep the launch within one wave
    g = _decode_plan(BF, 1, 6144, 1024)
    assert (g["kind"], g["kw"]) == (SMALL, 4) and g["ctas"] * (8 // g["kw"]) >= 384
    # lm_head and the wide projections of larger models: row-contiguous streaming, one CTA per SM, no K split
    lm = _decode_plan(BF, 1, 151936, 1024)
    assert (lm["kind"], lm["splits"], lm["ctas"]) == (ROWS, 1, 148)
    assert _decode_plan(BF, 8, 25600, 5120)["kind"] in (ROWS, RING)
    assert _decode_plan(BF, 1, 25600, 5120)["kind"] == ROWS
    # few row tiles and a long K: K split across CTAs on the per-lane-ring kernel (twice the warps balance better)
    sq = _decode_plan(BF, 1, 5120, 5120)
    assert sq["kind"] == RING and sq["splits"] > 1 and sq["kch"] % 256 == 0
    # contiguous [K, N] weights: mma.sync with transposing fragment loads; float32 stays on the FFMA kernels
    kn = _decode_plan(BF, 8, 151936, 1024, layout="KN")
    assert (kn["kind"], kn["splits"]) == (NMAJOR, 1)
    kn2 = _decode_plan(BF, 4, 12288, 4096, layout="KN")
    assert kn2["kind"] == NMAJOR and kn2["splits"] > 1 and 96 * kn2["splits"] <= 148 * 16
    assert _decode_plan(F32, 2, 4096, 4096)["kind"] == FFMA
    assert _decode_plan(F32, 2, 4096, 4096, layout="KN")["kind"] == FFMA
    # not decode-shaped (M > 8 after folding) or a layout the kernels do not take (weights with neither stride 1)
    assert _decode_plan(BF, 16, 4096, 4096)["kind"] == 0
    x = _fake_view(BF, (1, 64), (64, 1))
    y = _fake_view(BF, (64, 32), (2, 128), base=0x7F1000000000)
    out = [C.c_int() for _ in range(5)]
    kch = C.c_int64()
    mb.check(mb.lib().magb200_decode_plan(C.byref(x), C.byref(y), *[C.byref(o) for o in out], C.byref(kch)))
    assert out[0].value == 0
    # a batch of decode products folds into M only while it stays at or below 8 rows
    assert _decode_plan(BF, 2, 2048, 1024, batch=(4,))["kind"] == SMALL
    assert _decode_plan(BF, 4, 2048, 1024, batch=(4,))["kind"] == 0


def _route(dtype, xshape, xstrides, yshape, ystrides, xbase=0x7F0000000000, ybase=0x7F1000000000):
    x, y = _fake_view(dtype, xshape, xstrides, xbase), _fake_view(dtype, yshape, ystrides, ybase)
    k, rp = C.c_int(), C.c_int()
    mb.check(mb.lib().magb200_matmul_route(C.byref(x), C.byref(y), C.byref(k), C.byref(rp)))
    return mb.KERNEL_NAMES[k.value], rp.value


def test_matmul_routing_without_a_device():
    """Which kernel the configurations of the workload go to, decided on the host."""
    BF, F16, F32 = mb.BFLOAT16, mb.FLOAT16, mb.FLOAT32
    lin = lambda dt, M, N, K: _route(dt, (M, K), (K, 1), (K, N), (1, K))          # x @ W.T
    # prefill layer of the 8B model: q / o / gate / up / down on CTA pairs, k / v (64 tiles of 256 x 256) on the one-CTA kernel
    assert lin(BF, 4096, 4096, 4096) == ("tcgen05_2sm", 0)
    assert lin(BF, 4096, 12288, 4096) == ("tcgen05_2sm", 0)
    assert lin(BF, 4096, 1024, 4096) == ("tcgen05", 0)
    # the single-op workload: bf16 on the one-CTA kernel, fp32 on the split-operand tensor-core kernel, small fp32 on the FFMA kernel
    assert lin(BF, 512, 2048, 2048) == ("tcgen05", 0)
    assert lin(F32, 512, 2048, 2048) == ("tcgen05_f32x3", 0)
    assert lin(F32, 96, 80, 200) == ("simt", 0)
    assert lin(F32, 4096, 4096, 32) == ("simt", 0)                              # K below one 64-wide block
    # decode shapes
    assert lin(BF, 1, 151936, 1024) == ("skinny", 0)
    assert lin(F32, 8, 4096, 4096) == ("skinny", 0)
    assert lin(BF, 9, 4096, 4096)[0] == "tcgen05"
    # attention: scores [B,KV,G,T,D] @ [B,KV,1,D,T] with a broadcast dim, fp16
    B, KV, G, T, D = 8, 8, 4, 2048, 128
    q = (B, KV, G, T, D)
    kt = (B, KV, 1, D, T)
    assert _route(F16, q, mb.contiguous_strides(q), kt, (KV * T * D, T * D, 0, 1, D)) == ("tcgen05_2sm", 0)
    # operands TMA cannot describe: odd K (row pitch not a multiple of 16 bytes) is repacked on the device, then tensor cores
    assert lin(BF, 4096, 4096, 4095) == ("tcgen05_2sm", 1)
    assert _route(BF, (512, 1024), (2048, 2), (1024, 512), (1, 1024)) == ("tcgen05", 1)      # inner stride 2
    assert _route(BF, (512, 1024), (1024, 1), (1024, 512), (1, 1024), xbase=0x7F0000000002) == ("tcgen05", 1)   # misaligned slice
    assert lin(BF, 16, 24, 40) == ("tcgen05", 0)
    assert _route(BF, (16, 40), (80, 2), (40, 24), (1, 40)) == ("simt", 0)        # too small to be worth a repack
