"""Runs one kernel of the library a few times on a chosen size, for profilers and quick timing.

    python -m magnetron_b200.profile_cases gemm   --m 2048 --n 4096 --k 4096 [--dtype bf16|f16|f32] [--kn] [--iters 3]
    python -m magnetron_b200.profile_cases skinny --m 4 --n 32768 --k 4096
    python -m magnetron_b200.profile_cases cast   --n 67108864 [--src f32 --dst bf16]

Operands are seeded random values in device memory (weights in the `W.T` layout unless --kn); each
iteration uses the same buffers, so pick sizes beyond the 126 MB L2 when DRAM figures matter. Prints one
JSON line with the CUDA-event time per launch.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import numpy as np

import magnetron_b200 as mb

DT = {"f32": mb.FLOAT32, "f16": mb.FLOAT16, "bf16": mb.BFLOAT16}


def device_random(dev, dtype, shape, scale, rng):
    """Random tensor built on the device: one 16 Mi-element fp32 block is uploaded and cast repeatedly."""
    L = mb.lib()
    n = int(np.prod(shape))
    out = mb.Tensor(dev, dtype, shape)
    block = min(n, 1 << 24)
    host = (rng.standard_normal(block, dtype=np.float32) * np.float32(scale)).view(np.uint32)
    stage = mb.Tensor.from_bits(dev, mb.FLOAT32, host)
    for lo in range(0, n, block):
        m = min(block, n - lo)
        mb.check(L.magb200_cast(dev, C.byref(mb.make_view(stage.ptr, mb.FLOAT32, (m,))),
                                C.byref(mb.make_view(out.ptr, dtype, (m,), offset=lo))))
    mb.synchronize(dev)
    stage.release()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "skinny", "cast"])
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--dtype", default="bf16", choices=list(DT))
    ap.add_argument("--src", default="f32", choices=list(DT))
    ap.add_argument("--dst", default="bf16", choices=list(DT))
    ap.add_argument("--kn", action="store_true", help="weights stored [K,N] (N-major) instead of the W.T view of [N,K]")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    dev, L = 0, mb.lib()
    mb.check(L.magb200_device_init(dev))
    rng = np.random.default_rng(0)
    if a.case == "cast":
        src = device_random(dev, DT[a.src], (a.n,), 1.0, rng)
        dst = mb.Tensor(dev, DT[a.dst], (a.n,))
        sv, dv = src.view_struct(), dst.view_struct()
        call = lambda: mb.check(L.magb200_cast(dev, C.byref(sv), C.byref(dv)))
        work = {"bytes": a.n * (mb.DTYPE_SIZE[DT[a.src]] + mb.DTYPE_SIZE[DT[a.dst]])}
    else:
        dt = DT[a.dtype]
        x = device_random(dev, dt, (a.m, a.k), 1.0, rng)
        w = device_random(dev, dt, (a.k, a.n) if a.kn else (a.n, a.k), 0.02, rng)
        out = mb.Tensor(dev, dt, (a.m, a.n))
        xv, wv, ov = x.view_struct(), (w if a.kn else w.T).view_struct(), out.view_struct()
        call = lambda: mb.check(L.magb200_matmul(dev, C.byref(xv), C.byref(wv), C.byref(ov)))
        es = mb.DTYPE_SIZE[dt]
        work = {"flops": 2.0 * a.m * a.n * a.k, "bytes": (a.m * a.k + a.n * a.k + a.m * a.n) * es}
    call()
    mb.synchronize(dev)
    e0, e1 = C.c_void_p(), C.c_void_p()
    mb.check(L.magb200_event_create(C.byref(e0))); mb.check(L.magb200_event_create(C.byref(e1)))
    mb.check(L.magb200_event_record(dev, e0))
    for _ in range(a.iters):
        call()
    mb.check(L.magb200_event_record(dev, e1))
    ms = C.c_float()
    mb.check(L.magb200_event_elapsed_ms(e0, e1, C.byref(ms)))
    mb.synchronize(dev)
    per = ms.value / a.iters
    res = {"case": a.case, "ms": per, "kernel": mb.last_kernel() if a.case != "cast" else "cast", **vars(a)}
    if "flops" in work:
        res["tflops"] = work["flops"] / per / 1e9
    res["gbs"] = work["bytes"] / per / 1e6
    print(json.dumps(res))


if __name__ == "__main__":
    main()
