#!/usr/bin/env python
"""Benchmark of the matmul / cast hot path on B200 through the C ABI (include/magnetron_b200.h).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench.py --case gemm|skinny|cast --m .. --n .. --k ..        one kernel on one size (what the profiles capture)

One JSON line on stdout. A "step" is one pass of the hot path over one batch of synthetic input:

  N = 1  workload "qwen3-8b-prefill": the seven projection GEMMs of one Qwen3-8B layer at M = 4096 tokens
         (q, k, v, o, gate, up, down; bf16, fp32 accumulation, weights ~ N(0, 0.02^2) through the `W.T`
         view, activations ~ N(0,1), seed 3). `value` = TFLOP/s with everything resident in HBM;
         `e2e` = the same step driven the way a magnetron user would: `mag_matmul` on "cuda:0" through the unchanged
         core and the backend module, activations coming from page-locked host memory and every result copied back
         to it, both copies inside the timed region (`e2e_cabi`: the same through the C ABI directly).
         The same line carries every other single-GPU configuration with its own roofline fraction and the
         reference CPU backend timed beside it in the same run: `single_op` (512 x 2048 x 2048 through `W.T`,
         bf16 and fp32), `casts` (16 Mi elements both ways), `decode` (Qwen3-0.6B token pass, M in {1,2,4,8}),
         `attention` (scores and P.V over broadcast strided views, bf16 and fp16, full size), `tp_layer_1gpu`
         (the Qwen3-32B layer unsharded: the denominator of the multi-GPU scaling) and `gated_mlp` (the step's
         silu(gate) * up as one fused GEMM against the operator sequence).
  N > 1  workload "qwen3-32b-tp" (bench_tp.py): the four sharded GEMM groups of one Qwen3-32B layer at M = 8192, one rank
         per GPU. Total work is fixed, so scaling is "strong".

`--impl reference` times the reference CPU backend (oracle/_ref, all host threads) on the full prefill step.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BF16 = 2
HIDDEN, KV_DIM, INTER, TOKENS = 4096, 1024, 12288, 4096
# name, N (out features), K (in features), which activation feeds it
PREFILL_GEMMS = [("q", HIDDEN, HIDDEN, "x"), ("k", KV_DIM, HIDDEN, "x"), ("v", KV_DIM, HIDDEN, "x"),
                 ("o", HIDDEN, HIDDEN, "attn"), ("gate", INTER, HIDDEN, "x"), ("up", INTER, HIDDEN, "x"),
                 ("down", HIDDEN, INTER, "h")]
DECODE_LAYER = [("q", 2048, 1024), ("k", 1024, 1024), ("v", 1024, 1024), ("o", 1024, 2048),
                ("gate", 3072, 1024), ("up", 3072, 1024), ("down", 1024, 3072)]
DECODE_LAYERS, VOCAB = 28, 151936
# dram__bytes_read of one gemm_tcgen05_2sm_kernel launch on 4096^3 divided by its A + B bytes (one ncu capture of one launch)
DRAM_READ_FACTOR = 1.31


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm": p["hbm_gbs"], "tensor_burst": p["bf16_tflops"], "tensor_sustained": p["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm": 6650.0, "tensor_burst": 1590.0, "tensor_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for nm, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------------------
# device helpers on top of the C ABI
# ------------------------------------------------------------------------------------------------
class Dev:
    def __init__(self, device: int):
        import magnetron_b200 as mb
        self.mb, self.L, self.d = mb, mb.lib(), device
        mb.check(self.L.magb200_device_init(device))

    def event(self):
        p = C.c_void_p()
        self.mb.check(self.L.magb200_event_create(C.byref(p)))
        return p

    def record(self, ev):
        self.mb.check(self.L.magb200_event_record(self.d, ev))

    def elapsed_ms(self, a, b) -> float:
        ms = C.c_float()
        self.mb.check(self.L.magb200_event_elapsed_ms(a, b, C.byref(ms)))
        return ms.value

    def sync(self):
        self.mb.synchronize(self.d)

    def random_bf16(self, shape, scale: float, rng) -> "object":
        """Device bf16 tensor ~ N(0, scale^2): fp32 values drawn on the host in chunks, rounded on the GPU by
        the cast kernel of this library (bit-identical to the reference's conversion)."""
        mb = self.mb
        n = int(np.prod(shape))
        out = mb.Tensor(self.d, BF16, shape)
        chunk = 1 << 24
        stage = mb.Tensor(self.d, mb.FLOAT32, (min(chunk, n),))
        for lo in range(0, n, chunk):
            m = min(chunk, n - lo)
            host = (rng.standard_normal(m, dtype=np.float32) * np.float32(scale)).view(np.uint32)
            mb.check(self.L.magb200_upload(self.d, stage.ptr, host.ctypes.data, host.nbytes))
            src = mb.make_view(stage.ptr, mb.FLOAT32, (m,))
            dst = mb.make_view(out.ptr, BF16, (m,), offset=lo)
            mb.check(self.L.magb200_cast(self.d, C.byref(src), C.byref(dst)))
        self.sync()
        stage.release()
        return out

    def matmul(self, xv, wv, rv):
        self.mb.check(self.L.magb200_matmul(self.d, C.byref(xv), C.byref(wv), C.byref(rv)))


def timed_graph(dev: Dev, fn, launches: int, replays: int = 3):
    """Device time per call of `fn` with the host taken out: `launches` calls are recorded into one CUDA graph, the graph
    is replayed `replays` times after a warm-up replay, CUDA events bracket the replays. For kernels of a few microseconds,
    whose back-to-back issue rate from Python is slower than they run."""
    mb = dev.mb
    fn()
    dev.sync()
    graph = C.c_void_p()
    mb.check(dev.L.magb200_graph_begin_capture(dev.d))
    for _ in range(launches):
        fn()
    mb.check(dev.L.magb200_graph_end_capture(dev.d, C.byref(graph)))
    mb.check(dev.L.magb200_graph_launch(dev.d, graph))
    dev.sync()
    a, b = dev.event(), dev.event()
    dev.record(a)
    for _ in range(replays):
        mb.check(dev.L.magb200_graph_launch(dev.d, graph))
    dev.record(b)
    ms = dev.elapsed_ms(a, b)
    dev.sync()
    mb.check(dev.L.magb200_graph_destroy(graph))
    return ms / (launches * replays)


def timed(dev: Dev, fn, steps: int, warmup: int, barrier=None):
    """W untimed + K timed calls of fn, CUDA events on the launch stream, synchronised on both sides."""
    for _ in range(warmup):
        fn()
    dev.sync()
    if barrier:
        barrier()
    a, b = dev.event(), dev.event()
    dev.L.magb200_launch_count_reset()
    dev.record(a)
    for _ in range(steps):
        fn()
    dev.record(b)
    ms = dev.elapsed_ms(a, b)
    dev.sync()
    if barrier:
        barrier()
    return ms, int(dev.L.magb200_launch_count())


# ------------------------------------------------------------------------------------------------
# the reference CPU backend (oracle/_ref) beside every figure
# ------------------------------------------------------------------------------------------------
def host_bits(dtype: int, rng, shape, scale: float) -> np.ndarray:
    """fp32 values ~ N(0, scale^2) rounded on the host to the storage dtype with the reference's own conversion."""
    from oracle import mag_oracle as O
    return O.f32_to_bits(dtype, (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)))


class CpuRef:
    """The unmodified reference CPU backend, all host threads, timed in this same run. `None`-safe: when oracle/_ref is not
    built on this machine every figure comes back as None with the reason."""

    def __init__(self):
        from oracle import ref_driver as R
        self.R = R
        self.api = R.MagApi("cpu", log_level=1) if R.available() else None
        self.why = None if self.api else "oracle/_ref is not built on this machine"

    def close(self):
        if self.api:
            self.api.close(True)
            self.api = None

    def seconds(self, fn, reps: int, warm: int = 1) -> float:
        for _ in range(warm):
            fn()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        return (time.perf_counter() - t0) / reps

    def note(self, extra: str = "") -> dict:
        if not self.api:
            return {"value": None, "note": self.why}
        return {"cores": self.api.cores, "cpu": self.api.cpu_name, "kind": "reference", **({"sample": extra} if extra else {})}

    def linear(self, dtype: int, M: int, N: int, K: int, rng, reps: int) -> float | None:
        """Seconds per x[M,K] @ W[N,K].T through the transposed view (what nn.Linear dispatches)."""
        if not self.api:
            return None
        api = self.api
        x = api.from_bits(dtype, host_bits(dtype, rng, (M, K), 1.0))
        w = api.from_bits(dtype, host_bits(dtype, rng, (N, K), 0.02))
        wt = api.transpose(w, 0, 1)
        s = self.seconds(lambda: api.matmul(x, wt).release(), reps)
        for t in (wt, w, x):
            t.release()
        return s


def cpu_prefill_step(cpu: CpuRef, passes: int, warm: int = 1):
    """The full seven-GEMM prefill step on the reference CPU backend (1.58 TFLOP per pass, about two seconds)."""
    if not cpu.api:
        return {"value": None, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "reference", "sample": cpu.why}
    api = cpu.api
    rng = np.random.default_rng(3)
    acts = {"x": api.from_bits(BF16, host_bits(BF16, rng, (TOKENS, HIDDEN), 1.0)),
            "attn": api.from_bits(BF16, host_bits(BF16, rng, (TOKENS, HIDDEN), 1.0)),
            "h": api.from_bits(BF16, host_bits(BF16, rng, (TOKENS, INTER), 1.0))}
    ws = []
    for n, N, K, a in PREFILL_GEMMS:
        w = api.from_bits(BF16, host_bits(BF16, rng, (N, K), 0.02))
        ws.append((acts[a], w, api.transpose(w, 0, 1)))
    flops = sum(2.0 * TOKENS * N * K for _, N, K, _ in PREFILL_GEMMS)

    def step():
        for x, _, wt in ws:
            api.matmul(x, wt).release()

    s = cpu.seconds(step, passes, warm)
    for x, w, wt in ws:
        wt.release(); w.release()
    for t in acts.values():
        t.release()
    return {"value": flops / s / 1e12, "unit": "TFLOP/s", "cores": api.cores, "kind": "reference", "ms_per_pass": s * 1e3,
            "sample": "the full step: q,k,v,o,gate,up,down at 4096 tokens (%.0f GFLOP per pass), bf16 through the W.T view, %d passes; CPU %s"
                      % (flops / 1e9, passes, api.cpu_name)}


# ------------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------------
E2E_ORDER = ["gate", "up", "q", "k", "v", "o", "down"]   # largest results first: the download stream never idles


def prefill_workload(dev: Dev, steps: int, warmup: int):
    mb = dev.mb
    rng = np.random.default_rng(3)
    acts = {"x": dev.random_bf16((TOKENS, HIDDEN), 1.0, rng), "attn": dev.random_bf16((TOKENS, HIDDEN), 1.0, rng),
            "h": dev.random_bf16((TOKENS, INTER), 1.0, rng)}
    weights = {n: dev.random_bf16((N, K), 0.02, rng) for n, N, K, _ in PREFILL_GEMMS}
    outs = {n: mb.Tensor(dev.d, BF16, (TOKENS, N)) for n, N, K, _ in PREFILL_GEMMS}
    calls = [(acts[a].view_struct(), weights[n].T.view_struct(), outs[n].view_struct()) for n, N, K, a in PREFILL_GEMMS]
    flops = sum(2.0 * TOKENS * N * K for _, N, K, _ in PREFILL_GEMMS)
    abytes = sum(2.0 * (TOKENS * K + N * K + TOKENS * N) for _, N, K, _ in PREFILL_GEMMS)

    def step():
        for xv, wv, rv in calls:
            dev.matmul(xv, wv, rv)

    ms, launches = timed(dev, step, steps, warmup)
    kernel = mb.last_kernel()

    # end to end through the C ABI: activations from pinned host memory, every result back to pinned host memory. Each
    # activation is uploaded right before its first consumer and each result downloaded right after its producer, on the
    # library's copy streams: uploads, kernels and downloads of different operators overlap (the link is full duplex).
    pin = {}
    for name, t in list(acts.items()) + [("out_" + n, o) for n, o in outs.items()]:
        p = C.c_void_p()
        mb.check(dev.L.magb200_host_alloc_pinned(C.byref(p), t.numel * 2))
        pin[name] = p
    for name, t in acts.items():
        mb.check(dev.L.magb200_download(dev.d, pin[name], t.ptr, t.numel * 2))
    h2d = sum(t.numel * 2 for t in acts.values())
    d2h = sum(o.numel * 2 for o in outs.values())
    by_name = {n: (a, c) for (n, N, K, a), c in zip(PREFILL_GEMMS, calls)}

    def step_e2e():
        uploaded = set()
        for n in E2E_ORDER:
            a, (xv, wv, rv) = by_name[n]
            if a not in uploaded:
                uploaded.add(a)
                mb.check(dev.L.magb200_upload_overlapped(dev.d, acts[a].ptr, pin[a], acts[a].numel * 2))
            dev.matmul(xv, wv, rv)
            mb.check(dev.L.magb200_download_overlapped(dev.d, pin["out_" + n], outs[n].ptr, outs[n].numel * 2))
        dev.sync()  # the caller reads the results on the host; waits for the copy streams too

    e2e_steps = max(3, min(steps, 10))
    ms_e2e, _ = timed(dev, step_e2e, e2e_steps, 1)
    for p in pin.values():
        dev.L.magb200_host_free_pinned(p)
    for t in list(acts.values()) + list(weights.values()) + list(outs.values()):
        t.release()
    return {"ms_per_step": ms / steps, "tflops": flops * steps / ms / 1e9, "launches": launches, "kernel": kernel,
            "flops_per_step": flops, "bytes_per_step": abytes, "e2e_ms_per_step": ms_e2e / e2e_steps, "e2e_tflops": flops * e2e_steps / ms_e2e / 1e9,
            "h2d": h2d, "d2h": d2h}


def plugin_e2e_leg(steps: int):
    """Body of `--leg plugin-e2e` (a process of its own: the magnetron core may be loaded only once per process): the same
    end-to-end step, but every operator is `mag_matmul` on "cuda:0" through the unchanged magnetron core and the backend
    module, results are fresh tensors from the module's pooled allocator, transfers go through the module's exports."""
    import tempfile
    from magnetron_b200 import magnetron_capi as M
    core_dir = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.exists(os.path.join(core_dir, "libmagnetron_core.so")):
        print(json.dumps({"unavailable": "no built magnetron core on this machine to plug into"}))
        return
    tmp = tempfile.mkdtemp(prefix="magnetron_install_")
    ctx = M.Context(M.install(tmp, core_dir))
    rng = np.random.default_rng(3)
    pin, acts = {}, [{}, {}]
    for name, shape in (("x", (TOKENS, HIDDEN)), ("attn", (TOKENS, HIDDEN)), ("h", (TOKENS, INTER))):
        nbytes = shape[0] * shape[1] * 2
        pin[name] = ctx.host_alloc(nbytes)
        np.ctypeslib.as_array(C.cast(pin[name], C.POINTER(C.c_uint16)), shape=shape)[:] = host_bits(BF16, rng, shape, 1.0)
        for half in acts:            # two sets of device activations: step i+1 uploads while step i still computes
            half[name] = ctx.empty(M.BFLOAT16, shape)
    weights, wts = {}, {}
    for n, N, K, _ in PREFILL_GEMMS:
        hb = host_bits(BF16, rng, (N, K), 0.02)
        weights[n] = ctx.empty(M.BFLOAT16, (N, K))
        ctx.upload(weights[n], hb.ctypes.data, hb.nbytes)
        wts[n] = ctx.transpose(weights[n], 0, 1)            # the W.T view: header only
        pin["out_" + n] = ctx.host_alloc(TOKENS * N * 2)
    which = {n: a for n, N, K, a in PREFILL_GEMMS}
    shapes = {n: (N, K) for n, N, K, _ in PREFILL_GEMMS}
    flops = sum(2.0 * TOKENS * N * K for _, N, K, _ in PREFILL_GEMMS)

    def step(i: int, wait: bool):
        uploaded = set()
        cur = acts[i & 1]
        for n in E2E_ORDER:
            a = which[n]
            if a not in uploaded:
                uploaded.add(a)
                ctx.upload(cur[a], pin[a], TOKENS * shapes[n][1] * 2, wait=False)
            r = ctx.matmul(cur[a], wts[n])
            ctx.download(r, pin["out_" + n], TOKENS * shapes[n][0] * 2, wait=False)
            ctx.decref(r)                                   # storage returns to the pool; the copy stream still reads it
        if wait:
            ctx.synchronize()

    # Steps are pipelined the way a serving loop would run them: every result is a fresh tensor from the module's pool, so the
    # next step's uploads and GEMMs start while this step's results are still on their way to the host (the copies to one
    # host buffer stay in order on the download stream). The host waits every eighth step (bounds the memory in flight) and
    # at the end; `per_step_sync_ms` is the same loop with a wait after every step.
    step(0, True); step(1, True)
    t0 = time.perf_counter()
    for i in range(steps):
        step(i, True)
    dt_sync = time.perf_counter() - t0
    for i in range(16):                                      # lets the pool grow to eight steps' worth of results, untimed
        step(i, (i & 7) == 7)
    t0 = time.perf_counter()
    for i in range(steps):
        step(i, (i & 7) == 7 or i == steps - 1)
    dt = time.perf_counter() - t0
    out = {"ms_per_step": dt / steps * 1e3, "tflops": flops * steps / dt / 1e12, "device": ctx.device_name,
           "per_step_sync_ms": dt_sync / steps * 1e3, "per_step_sync_tflops": flops * steps / dt_sync / 1e12,
           "timing": "host clock around K pipelined steps (mag_b200_synchronize every eighth step and after the last one); "
                     "every step's uploads and downloads are inside the region"}
    for t in list(wts.values()) + list(weights.values()) + list(acts[0].values()) + list(acts[1].values()):
        ctx.decref(t)
    for p in pin.values():
        ctx.host_free(p)
    ctx.close(False)                                        # leak detection on: every storage went back
    import shutil
    shutil.rmtree(tmp, ignore_errors=True)
    print(json.dumps(out))


def plugin_e2e(steps: int):
    try:
        res = subprocess.run([sys.executable, os.path.abspath(__file__), "--leg", "plugin-e2e", "--steps", str(steps)],
                             capture_output=True, text=True, timeout=600)
        lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
        if res.returncode != 0 or not lines:
            return {"unavailable": "plug-in leg failed: " + (res.stderr.strip().splitlines() or ["no output"])[-1][:200]}
        return json.loads(lines[-1])
    except Exception as e:   # noqa: BLE001 - the leg is reported, never fatal
        return {"unavailable": repr(e)[:200]}


def single_op_workload(dev: Dev, cpu: CpuRef, pk):
    """C[512,2048] = A[512,2048] @ W[2048,2048]^T through the transposed view, bf16 and fp32 (seed 0). Sixteen operand sets
    rotate (201 MB, more than L2); the launches are replayed from a CUDA graph so the figure is the kernel's, not the host's."""
    mb = dev.mb
    M, N, K = 512, 2048, 2048
    out = {"shape": [M, N, K], "l2": "16 rotating operand sets (201 MB bf16 / 403 MB fp32), graph replay of 208 calls; consecutive calls "
           "touch different tensors, so the library lets a launch start on the SMs the one before it has left "
           "(fp32: each call clears a flag, splits both operands into bf16 planes, runs the tensor-core kernel and a stand-by FFMA launch)"}
    for key, dt, peak, bound in (("bf16", BF16, pk["tensor_burst"], "tensor"), ("fp32", mb.FLOAT32, pk["tensor_burst"] / 6.0,
                                  "tensor: six bf16 MMAs assemble one fp32 product, so the ceiling is the bf16 peak / 6")):
        rng = np.random.default_rng(0)
        sets = []
        for _ in range(16):
            if dt == BF16:
                x, w = dev.random_bf16((M, K), 1.0, rng), dev.random_bf16((N, K), 0.02, rng)
            else:
                x = mb.Tensor.from_bits(dev.d, dt, rng.standard_normal((M, K), dtype=np.float32).view(np.uint32))
                w = mb.Tensor.from_bits(dev.d, dt, (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)).view(np.uint32))
            sets.append((x, w, mb.Tensor(dev.d, dt, (M, N))))
        views = [(x.view_struct(), w.T.view_struct(), o.view_struct()) for x, w, o in sets]
        i = [0]

        def call():
            dev.matmul(*views[i[0] % 16])
            i[0] += 1

        ms = timed_graph(dev, call, 208)
        tf = 2.0 * M * N * K / ms / 1e9
        sec = cpu.linear(dt, M, N, K, np.random.default_rng(0), 10)
        out[key] = {"us": ms * 1e3, "tflops": tf, "kernel": mb.last_kernel(),
                    "roofline": {"bound": bound, "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                                 "frac_of_nominal_2250": tf / 2250.0 if dt == BF16 else None},
                    "cpu": {"tflops": (2.0 * M * N * K / sec / 1e12) if sec else None, "ms": sec * 1e3 if sec else None, **cpu.note()}}
        for x, w, o in sets:
            x.release(); w.release(); o.release()
    return out


def decode_workload(dev: Dev, cpu: CpuRef, steps: int, warmup: int, hbm_peak: float):
    """One token pass of Qwen3-0.6B (28 layers x 7 projections + lm_head) per step; every launch reads different weight
    matrices and the 1.19 GB of weights exceed L2 many times over. Projections that share their activation (q,k,v and
    gate,up) go out as one grouped call, so a layer is 4 launches."""
    mb = dev.mb
    rng = np.random.default_rng(2)
    layers = []
    for _ in range(DECODE_LAYERS):
        layers.append([(dev.random_bf16((N, K), 0.02, rng), N, K) for _, N, K in DECODE_LAYER])
    lm_head = dev.random_bf16((VOCAB, 1024), 0.02, rng)
    wbytes = sum(N * K * 2 for _, N, K in DECODE_LAYER) * DECODE_LAYERS + VOCAB * 1024 * 2
    result = {}
    for M in (1, 2, 4, 8):
        xs = {K: dev.random_bf16((M, K), 1.0, rng) for K in (1024, 2048, 3072)}
        outs = {N: mb.Tensor(dev.d, BF16, (M, N)) for N in (1024, 2048, 3072, VOCAB)}
        calls = []
        for layer in layers:
            for w, N, K in layer:
                calls.append((xs[K].view_struct(), w.T.view_struct(), outs[N].view_struct()))
        calls.append((xs[1024].view_struct(), lm_head.T.view_struct(), outs[VOCAB].view_struct()))
        act_bytes = sum((M * K + M * N) * 2 for _, N, K in DECODE_LAYER) * DECODE_LAYERS + (M * 1024 + M * VOCAB) * 2
        # products that share their activation go out as one grouped call: (q,k,v), o, (gate,up), down -- 4 launches per layer
        # (k and v get result buffers of their own here: a group's results must not alias)
        outs_v, outs_up = mb.Tensor(dev.d, BF16, (M, 1024)), mb.Tensor(dev.d, BF16, (M, 3072))
        keep, grouped = [], []
        for li, layer in enumerate(layers):
            vs = {nm: (xs[K].view_struct(), w.T.view_struct(), outs[N].view_struct()) for (nm, _, _), (w, N, K) in zip(DECODE_LAYER, layer)}
            vs["v"] = (vs["v"][0], vs["v"][1], outs_v.view_struct())
            vs["up"] = (vs["up"][0], vs["up"][1], outs_up.view_struct())
            for names in (("q", "k", "v"), ("o",), ("gate", "up"), ("down",)):
                yv, rv = [vs[n][1] for n in names], [vs[n][2] for n in names]
                ya = (C.POINTER(mb.View) * len(names))(*[C.pointer(v) for v in yv])
                ra = (C.POINTER(mb.View) * len(names))(*[C.pointer(v) for v in rv])
                keep.append((yv, rv))
                grouped.append((vs[names[0]][0], len(names), ya, ra))

        def step():
            for xv, n, ya, ra in grouped:
                mb.check(dev.L.magb200_matmul_grouped(dev.d, C.byref(xv), n, ya, ra))
            dev.matmul(*calls[-1])

        # the token pass is launch-bound when issued call by call (about 200 launches of a few microseconds);
        # it is recorded once and replayed as a CUDA graph, the way a serving loop would run it
        step()
        dev.sync()
        graph = C.c_void_p()
        mb.check(dev.L.magb200_graph_begin_capture(dev.d))
        step()
        mb.check(dev.L.magb200_graph_end_capture(dev.d, C.byref(graph)))
        ms_calls, launches = timed(dev, step, steps, warmup)
        ms, _ = timed(dev, lambda: mb.check(dev.L.magb200_graph_launch(dev.d, graph)), steps, warmup)
        mb.check(dev.L.magb200_graph_destroy(graph))
        # lm_head alone (311 MB per launch, 2.5x the L2 capacity): the largest single GEMV
        lm = calls[-1]
        ms_lm, _ = timed(dev, lambda: dev.matmul(*lm), max(steps, 10), warmup)
        gbs = (wbytes + act_bytes) * steps / ms / 1e6
        gbs_lm = (VOCAB * 1024 * 2 + (M * 1024 + M * VOCAB) * 2) * max(steps, 10) / ms_lm / 1e6
        result[f"M{M}"] = {"token_pass_ms": ms / steps, "token_pass_ms_call_by_call": ms_calls / steps, "gbs": gbs, "frac": gbs / hbm_peak,
                           "frac_of_nominal_8000": gbs / 8000.0, "launches_per_step": launches // steps,
                           "lm_head_ms": ms_lm / max(steps, 10), "lm_head_gbs": gbs_lm, "lm_head_frac": gbs_lm / hbm_peak,
                           "lm_head_frac_of_nominal_8000": gbs_lm / 8000.0, "kernel": mb.last_kernel()}
        for t in list(xs.values()) + list(outs.values()) + [outs_v, outs_up]:
            t.release()
    for layer in layers:
        for w, _, _ in layer:
            w.release()
    lm_head.release()
    # the reference CPU backend on the same operators through the same W.T views: lm_head and one 7-projection layer
    for M in (1, 8):
        crng = np.random.default_rng(2)
        lm_s = cpu.linear(BF16, M, VOCAB, 1024, crng, 5)
        layer_s = None
        if cpu.api:
            layer_s = sum(cpu.linear(BF16, M, N, K, crng, 10) for _, N, K in DECODE_LAYER)
        lbytes = sum(N * K * 2 for _, N, K in DECODE_LAYER)
        result[f"M{M}"]["cpu"] = {"lm_head_ms": lm_s * 1e3 if lm_s else None, "lm_head_gbs": VOCAB * 1024 * 2 / lm_s / 1e9 if lm_s else None,
                                  "layer_ms": layer_s * 1e3 if layer_s else None, "layer_gbs": lbytes / layer_s / 1e9 if layer_s else None,
                                  "token_pass_ms_extrapolated": (layer_s * DECODE_LAYERS + lm_s) * 1e3 if lm_s else None,
                                  **cpu.note("lm_head and one layer's seven projections, bf16 through the W.T view (the blocked GEMM path "
                                             "of the reference, not its contiguous-weight GEMV); token pass = 28 x layer + lm_head")}
    return result


def cast_workload(dev: Dev, cpu: CpuRef, steps: int, warmup: int, hbm_peak: float):
    """fp32 <-> bf16 casts of 16 Mi elements (100.7 MB of traffic each); four rotating buffer pairs (403 MB)
    keep every launch out of L2."""
    mb = dev.mb
    rng = np.random.default_rng(1)
    n, copies = 1 << 24, 4
    f32 = [mb.Tensor.from_bits(dev.d, mb.FLOAT32, rng.standard_normal(n, dtype=np.float32).view(np.uint32)) for _ in range(copies)]
    b16 = [mb.Tensor(dev.d, BF16, (n,)) for _ in range(copies)]
    out = {}
    for key, src, dst in (("f32_to_bf16", f32, b16), ("bf16_to_f32", b16, f32)):
        views = [(s.view_struct(), d.view_struct()) for s, d in zip(src, dst)]
        i = [0]

        def step():
            s, d = views[i[0] % copies]
            i[0] += 1
            mb.check(dev.L.magb200_cast(dev.d, C.byref(s), C.byref(d)))

        ms, _ = timed(dev, step, max(steps, 20), warmup)
        gbs = n * 6 * max(steps, 20) / ms / 1e6
        out[key] = {"ms": ms / max(steps, 20), "gbs": gbs, "frac": gbs / hbm_peak, "frac_of_nominal_8000": gbs / 8000.0}
    for t in f32 + b16:
        t.release()
    # the same kernels on 128 Mi elements (805 MB per launch): a 16 Mi launch lasts 20 us, much of it the ramp of the DRAM pipes
    big = 1 << 27
    bf = mb.Tensor(dev.d, mb.FLOAT32, (big,))
    bb = mb.Tensor(dev.d, BF16, (big,))
    mb.check(dev.L.magb200_fill(dev.d, C.byref(bf.view_struct()), C.c_double(1.5)))
    for key, src, dst in (("f32_to_bf16", bf, bb), ("bf16_to_f32", bb, bf)):
        sv, dv = src.view_struct(), dst.view_struct()
        ms, _ = timed(dev, lambda: mb.check(dev.L.magb200_cast(dev.d, C.byref(sv), C.byref(dv))), 5, 2)
        out[key]["at_128Mi"] = {"ms": ms / 5, "gbs": big * 6 * 5 / ms / 1e6, "frac": big * 6 * 5 / ms / 1e6 / hbm_peak}
    bf.release(); bb.release()
    if cpu.api:
        api = cpu.api
        xb = np.random.default_rng(1).standard_normal(n, dtype=np.float32).view(np.uint32)
        x32 = api.from_bits(mb.FLOAT32, xb)
        x16 = api.cast(x32, BF16)
        for key, src, dt in (("f32_to_bf16", x32, BF16), ("bf16_to_f32", x16, mb.FLOAT32)):
            s = cpu.seconds(lambda: api.cast(src, dt).release(), 10, 2)
            out[key]["cpu"] = {"ms": s * 1e3, "gbs": n * 6 / s / 1e9, **cpu.note()}
        x16.release(); x32.release()
    else:
        for key in ("f32_to_bf16", "bf16_to_f32"):
            out[key]["cpu"] = cpu.note()
    return out


def attention_workload(dev: Dev, cpu: CpuRef, hbm_peak: float, tensor_peak: float):
    """Scores Q[8x32x2048x128] @ K^T and outputs P[8x32x2048x2048] @ V, K and V [8x8x2048x128] broadcast over 4 query heads per
    KV head through strided views, bf16 and fp16, at full size (2.1 GB of scores). Both are bound by streaming the S / P
    matrix, so the roofline is HBM; the tensor fraction is reported beside it."""
    mb = dev.mb
    B, KV, G, T, D = 8, 8, 4, 2048, 128
    flops = 2.0 * B * KV * G * T * T * D
    abytes = 2.0 * (B * KV * G * T * D + B * KV * T * D + B * KV * G * T * T)
    out = {"shape": "Q[8,8,4,2048,128] K,V[8,8,2048,128] -> S,P[8,8,4,2048,2048]", "algorithmic_bytes": abytes, "flops": flops,
           "l2": "operands and results far larger than L2 (2.3 GB per launch)"}
    rng = np.random.default_rng(4)
    # P: one seeded block of softmax(N(0,1) logits / sqrt(D)) rows, repeated over the batch by a device-side broadcast clone
    logits = rng.standard_normal((T, T), dtype=np.float32) / np.float32(np.sqrt(D))
    pblock = np.exp(logits - logits.max(-1, keepdims=True))
    pblock /= pblock.sum(-1, keepdims=True)
    for key, dt in (("bf16", BF16), ("fp16", mb.FLOAT16)):
        from oracle import mag_oracle as O
        q = mb.Tensor.from_bits(dev.d, dt, host_bits(dt, rng, (B, KV, G, T, D), 1.0))
        k = mb.Tensor.from_bits(dev.d, dt, host_bits(dt, rng, (B, KV, T, D), 1.0))
        v = mb.Tensor.from_bits(dev.d, dt, host_bits(dt, rng, (B, KV, T, D), 1.0))
        s = mb.Tensor(dev.d, dt, (B, KV, G, T, T))
        o = mb.Tensor(dev.d, dt, (B, KV, G, T, D))
        kt = k.transpose(2, 3).view((B, KV, 1, D, T))
        vv = v.view((B, KV, 1, T, D))
        sc = (q.view_struct(), kt.view_struct(), s.view_struct())
        ms_s, _ = timed(dev, lambda: dev.matmul(*sc), 10, 3)
        kern_s = mb.last_kernel()
        p0 = mb.Tensor.from_bits(dev.d, dt, O.f32_to_bits(dt, pblock.astype(np.float32)))
        bsrc = mb.make_view(p0.ptr, dt, (B * KV * G, T, T), (0, T, 1))
        mb.check(dev.L.magb200_clone(dev.d, C.byref(bsrc), C.byref(mb.make_view(s.ptr, dt, (B * KV * G, T, T)))))
        pv = (s.view_struct(), vv.view_struct(), o.view_struct())
        ms_p, _ = timed(dev, lambda: dev.matmul(*pv), 10, 3)
        kern_p = mb.last_kernel()
        res = {}
        for name, ms, kern in (("scores", ms_s / 10, kern_s), ("pv", ms_p / 10, kern_p)):
            gbs = abytes / ms / 1e6
            res[name] = {"ms": ms, "gbs": gbs, "tflops": flops / ms / 1e9, "kernel": kern,
                         "roofline": {"bound": "hbm", "achieved": gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gbs / hbm_peak,
                                      "frac_of_nominal_8000": gbs / 8000.0, "tensor_frac": flops / ms / 1e9 / tensor_peak}}
        for t in (p0, o, s, v, k, q):
            t.release()
        # reference CPU backend on a batch subset of the same views (flagged): bf16 one (batch, KV head) group, fp16 -- whose
        # reference kernel is a scalar loop -- 128 query rows of one head
        if cpu.api:
            api = cpu.api
            crng = np.random.default_rng(4)
            g, t_rows = (G, T) if dt == BF16 else (1, 128)
            cq = api.from_bits(dt, host_bits(dt, crng, (1, 1, g, t_rows, D), 1.0))
            ck = api.from_bits(dt, host_bits(dt, crng, (1, 1, T, D), 1.0))
            ckt = api.transpose(ck, 2, 3)
            ckv = api.view(ckt, (1, 1, 1, D, T))
            sec_s = cpu.seconds(lambda: api.matmul(cq, ckv).release(), 3)
            cp = api.from_bits(dt, O.f32_to_bits(dt, np.broadcast_to(pblock[:t_rows], (1, 1, g, t_rows, T)).astype(np.float32)))
            cv = api.view(ck, (1, 1, 1, T, D))
            sec_p = cpu.seconds(lambda: api.matmul(cp, cv).release(), 3)
            sub_flops = 2.0 * g * t_rows * T * D
            sub_bytes = 2.0 * (g * t_rows * D + T * D + g * t_rows * T)
            sample = "batch subset: %d head(s) x %d query rows against one KV head (%.2f GFLOP), same broadcast views" % (g, t_rows, sub_flops / 1e9)
            res["scores"]["cpu"] = {"gflops": sub_flops / sec_s / 1e9, "gbs": sub_bytes / sec_s / 1e9, "ms_subset": sec_s * 1e3, **cpu.note(sample)}
            res["pv"]["cpu"] = {"gflops": sub_flops / sec_p / 1e9, "gbs": sub_bytes / sec_p / 1e9, "ms_subset": sec_p * 1e3, **cpu.note(sample)}
            for t in (cv, cp, ckv, ckt, ck, cq):
                t.release()
        else:
            res["scores"]["cpu"] = res["pv"]["cpu"] = cpu.note()
        out[key] = res
    return out


def gated_mlp_workload(dev: Dev, cpu: CpuRef, steps: int, warmup: int, tensor_peak: float):
    """silu(x @ Wg.T) * (x @ Wu.T) of the prefill step's MLP (4096 tokens, 4096 -> 12288): one fused GEMM against the operator
    sequence on the device (two GEMMs into temporaries and an elementwise pass), FLOPs counted as the two GEMMs' in both."""
    mb = dev.mb
    M, N, K = TOKENS, INTER, HIDDEN
    rng = np.random.default_rng(9)
    x, wg, wu = dev.random_bf16((M, K), 1.0, rng), dev.random_bf16((N, K), 0.02, rng), dev.random_bf16((N, K), 0.02, rng)
    out = mb.Tensor(dev.d, BF16, (M, N))
    xv, gv, uv, ov = x.view_struct(), wg.T.view_struct(), wu.T.view_struct(), out.view_struct()
    call = lambda: mb.check(dev.L.magb200_matmul_swiglu(dev.d, C.byref(xv), C.byref(gv), C.byref(uv), C.byref(ov)))
    n = max(3, min(steps, 20))
    ms, _ = timed(dev, call, n, warmup)
    mb.force_kernel("tcgen05_2sm")           # a pinned kernel makes the entry point run the operator sequence
    try:
        ms_seq, _ = timed(dev, call, n, warmup)
    finally:
        mb.force_kernel(None)
    flops = 4.0 * M * N * K
    tf = flops * n / ms / 1e9
    res = {"shape": [M, N, K], "ms": ms / n, "tflops": tf, "operator_sequence_ms": ms_seq / n, "operator_sequence_tflops": flops * n / ms_seq / 1e9,
           "result_bytes_saved_per_call": 2 * M * N * 2 * 2,
           "roofline": {"bound": "tensor", "achieved": tf, "peak": tensor_peak, "unit": "TFLOP/s", "frac": tf / tensor_peak}}
    for t in (x, wg, wu, out):
        t.release()
    if cpu.api:
        api = cpu.api
        crng = np.random.default_rng(9)
        cm = 512
        rx = api.from_bits(BF16, host_bits(BF16, crng, (cm, K), 1.0))
        rg, ru = api.from_bits(BF16, host_bits(BF16, crng, (N, K), 0.02)), api.from_bits(BF16, host_bits(BF16, crng, (N, K), 0.02))
        gt, ut = api.transpose(rg, 0, 1), api.transpose(ru, 0, 1)

        def seq():
            a, b = api.matmul(rx, gt), api.matmul(rx, ut)
            s_ = api.silu(a)
            r = api.mul(s_, b)
            for h in (r, s_, b, a):
                h.release()

        sec = cpu.seconds(seq, 2)
        for h in (ut, gt, ru, rg, rx):
            h.release()
        res["cpu"] = {"tflops": 4.0 * cm * N * K / sec / 1e12, **cpu.note("MATMUL, MATMUL, SILU, MUL at 512 tokens (rows are independent)")}
    else:
        res["cpu"] = cpu.note()
    return res


TP_LAYER = [("qkv", 10240, 5120), ("o", 5120, 8192), ("gate_up", 51200, 5120), ("down", 5120, 25600)]


def tp_layer_1gpu_workload(dev: Dev, cpu: CpuRef, steps: int, warmup: int, tensor_peak: float):
    """The four GEMM groups of one Qwen3-32B layer at M = 8192, unsharded on one GPU: the same work that `--gpus N` shards,
    i.e. the denominator of the multi-GPU scaling figures."""
    mb = dev.mb
    M = 8192
    rng = np.random.default_rng(5)
    ops = []
    for _, N, K in TP_LAYER:
        ops.append((dev.random_bf16((M, K), 1.0, rng), dev.random_bf16((N, K), 0.02, rng), mb.Tensor(dev.d, BF16, (M, N))))
    calls = [(x.view_struct(), w.T.view_struct(), o.view_struct()) for x, w, o in ops]
    flops = sum(2.0 * M * N * K for _, N, K in TP_LAYER)

    def step():
        for c in calls:
            dev.matmul(*c)

    n = max(3, min(steps, 10))
    ms, _ = timed(dev, step, n, warmup)
    for x, w, o in ops:
        x.release(); w.release(); o.release()
    tf = flops * n / ms / 1e9
    res = {"workload": "qwen3-32b layer GEMMs (qkv, o, gate_up, down) at M=8192, seed 5, one GPU", "ms_per_step": ms / n, "tflops": tf,
           "roofline": {"bound": "tensor", "achieved": tf, "peak": tensor_peak, "unit": "TFLOP/s", "frac": tf / tensor_peak,
                        "frac_of_nominal_2250": tf / 2250.0}}
    if cpu.api:
        crng = np.random.default_rng(5)
        sec = sum(cpu.linear(BF16, 512, N, K, crng, 2) for _, N, K in TP_LAYER)
        res["cpu"] = {"tflops": sum(2.0 * 512 * N * K for _, N, K in TP_LAYER) / sec / 1e12,
                      **cpu.note("the same four GEMMs at 512 tokens (rows are independent; the reference's FLOP/s is flat in M)")}
    else:
        res["cpu"] = cpu.note()
    return res


# ------------------------------------------------------------------------------------------------
# one kernel on one size: what the ncu captures under profiles/ run
# ------------------------------------------------------------------------------------------------
def case_mode(args):
    """`--case gemm|skinny|cast`: seeded operands in device memory (weights in the `W.T` layout unless --kn), `--iters`
    launches on the same buffers -- pick sizes beyond the 126 MB L2 when DRAM figures matter. One JSON line with the
    CUDA-event time per launch."""
    import magnetron_b200 as mb
    DT = {"f32": mb.FLOAT32, "f16": mb.FLOAT16, "bf16": mb.BFLOAT16}
    dev = Dev(0)
    L = dev.L
    rng = np.random.default_rng(0)

    def device_random(dtype, shape, scale):
        n = int(np.prod(shape))
        out = mb.Tensor(dev.d, dtype, shape)
        block = min(n, 1 << 24)
        stage = mb.Tensor.from_bits(dev.d, mb.FLOAT32, (rng.standard_normal(block, dtype=np.float32) * np.float32(scale)).view(np.uint32))
        for lo in range(0, n, block):
            m = min(block, n - lo)
            mb.check(L.magb200_cast(dev.d, C.byref(mb.make_view(stage.ptr, mb.FLOAT32, (m,))), C.byref(mb.make_view(out.ptr, dtype, (m,), offset=lo))))
        dev.sync()
        stage.release()
        return out

    if args.case == "cast":
        src = device_random(DT[args.src], (args.n,), 1.0)
        dst = mb.Tensor(dev.d, DT[args.dst], (args.n,))
        sv, dv = src.view_struct(), dst.view_struct()
        call = lambda: mb.check(L.magb200_cast(dev.d, C.byref(sv), C.byref(dv)))
        work = {"bytes": args.n * (mb.DTYPE_SIZE[DT[args.src]] + mb.DTYPE_SIZE[DT[args.dst]])}
    else:
        dt = DT[args.dtype]
        x = device_random(dt, (args.m, args.k), 1.0)
        w = device_random(dt, (args.k, args.n) if args.kn else (args.n, args.k), 0.02)
        out = mb.Tensor(dev.d, dt, (args.m, args.n))
        xv, wv, ov = x.view_struct(), (w if args.kn else w.T).view_struct(), out.view_struct()
        call = lambda: dev.matmul(xv, wv, ov)
        es = mb.DTYPE_SIZE[dt]
        work = {"flops": 2.0 * args.m * args.n * args.k, "bytes": (args.m * args.k + args.n * args.k + args.m * args.n) * es}
    ms, _ = timed(dev, call, args.iters, 1)
    per = ms / args.iters
    res = {"case": args.case, "ms": per, "kernel": mb.last_kernel() if args.case != "cast" else "cast",
           "m": args.m, "n": args.n, "k": args.k, "iters": args.iters}
    if "flops" in work:
        res["tflops"] = work["flops"] / per / 1e9
    res["gbs"] = work["bytes"] / per / 1e6
    print(json.dumps(res))


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only-headline", action="store_true", help="only the prefill step, no other configuration, no CPU legs (used under ncu)")
    ap.add_argument("--workload", default="auto", choices=["auto", "prefill", "tp"],
                    help="auto: Qwen3-8B prefill layer on one GPU, Qwen3-32B tensor-parallel layer on several")
    ap.add_argument("--leg", default=None, choices=["plugin-e2e"], help="internal: one leg in a process of its own")
    ap.add_argument("--case", default=None, choices=["gemm", "skinny", "cast"])
    ap.add_argument("--m", type=int, default=2048)
    ap.add_argument("--n", type=int, default=4096)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--dtype", default="bf16", choices=["f32", "f16", "bf16"])
    ap.add_argument("--src", default="f32", choices=["f32", "f16", "bf16"])
    ap.add_argument("--dst", default="bf16", choices=["f32", "f16", "bf16"])
    ap.add_argument("--kn", action="store_true", help="weights stored [K,N] (N-major) instead of the W.T view of [N,K]")
    ap.add_argument("--iters", type=int, default=3)
    args = ap.parse_args()
    if args.case:
        return case_mode(args)
    if args.leg == "plugin-e2e":
        return plugin_e2e_leg(args.steps)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    pk = peaks()

    if args.gpus > 1 or world > 1 or args.workload == "tp":
        import bench_tp
        return bench_tp.main(args, pk)

    config = {"workload": "qwen3-8b-prefill: q,k,v,o,gate,up,down GEMMs of one layer, M=4096 tokens, hidden 4096, "
                          "kv 1024, intermediate 12288, W.T views, seed 3",
              "l2": "inputs larger than L2 (528 MB of operands per step)", "tokens": TOKENS}

    if args.impl == "reference":
        if rank != 0:
            return
        cpu = CpuRef()
        if not cpu.api:
            print(json.dumps({"impl": "reference", "unavailable": cpu.why}))
            return
        passes = max(1, min(args.steps, 20))
        r = cpu_prefill_step(cpu, passes, min(args.warmup, 1))
        cpu.close()
        line = {"impl": "reference", "metric": "bf16 matmul TFLOP/s", "value": r["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
                "steps": passes, "warmup": min(args.warmup, 1), "ms_per_step": r["ms_per_pass"], "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
                "cpu_baseline": r, "e2e": {"value": r["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    dev = Dev(int(os.environ.get("LOCAL_RANK", "0")))
    sampler = ClockSampler(dev.d)
    sampler.start()
    pre = prefill_workload(dev, args.steps, args.warmup)
    clocks = sampler.stop()
    long_run = pre["ms_per_step"] * args.steps > 1000.0
    tensor_peak = pk["tensor_sustained"] if long_run else pk["tensor_burst"]
    # DRAM traffic of the GEMM kernels: DRAM reads per launch from an ncu capture of one 4096^3 launch of the same kernel
    # (ratio of dram__bytes_read to the A + B bytes), applied to the step's operand bytes, plus the algorithmic bytes of C
    # (part of C is still in L2 when a launch ends, so dram__bytes_write undercounts what the result costs).
    ab_bytes = sum(2.0 * (TOKENS * K + N * K) for _, N, K, _ in PREFILL_GEMMS)
    c_bytes = sum(2.0 * TOKENS * N for _, N, K, _ in PREFILL_GEMMS)
    line = {
        "metric": "bf16 matmul TFLOP/s", "value": pre["tflops"], "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": pre["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
        "gpu_launches": pre["launches"], "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": pre["tflops"], "peak": tensor_peak, "unit": "TFLOP/s",
                     "frac": pre["tflops"] / tensor_peak,
                     "traffic": (DRAM_READ_FACTOR * ab_bytes + c_bytes) / len(PREFILL_GEMMS),
                     "traffic_note": "per launch, mean over the step's 7 launches: operand reads scaled from an ncu capture of a smaller case "
                                     "of the same kernel by operand bytes, plus the algorithmic bytes of the results",
                     "peak_source": "%s %s cuBLAS bf16" % (pk["source"], "sustained" if long_run else "burst"),
                     "frac_of_nominal_2250": pre["tflops"] / 2250.0,
                     "kernel": "gemm_tcgen05_2sm_kernel (q,o,gate,up,down) + gemm_tcgen05_kernel (k,v)",
                     "algorithmic_flops_per_step": pre["flops_per_step"], "algorithmic_bytes_per_step": pre["bytes_per_step"]},
    }
    e2e_cabi = {"value": pre["e2e_tflops"], "unit": "TFLOP/s", "h2d_bytes_per_step": pre["h2d"], "d2h_bytes_per_step": pre["d2h"],
                "ms_per_step": pre["e2e_ms_per_step"], "path": "C ABI: magb200_upload_overlapped / magb200_matmul / magb200_download_overlapped"}
    if args.only_headline:
        line["e2e"] = e2e_cabi
        print(json.dumps(line))
        return
    cpu = CpuRef()
    line["single_op"] = single_op_workload(dev, cpu, pk)
    line["decode"] = {"metric": "decode GEMV HBM GB/s", "unit": "GB/s", "peak": pk["hbm"], "peak_source": pk["source"] + " copy",
                      "note": "gbs/frac = whole token pass replayed as a CUDA graph (mostly 2-6 MB per launch, latency bound); "
                              "lm_head_* = the 311 MB GEMV alone, the per-kernel HBM figure (skinny_km_async_kernel)",
                      "config": "qwen3-0.6b token pass: 28 layers x (q,k,v,o,gate,up,down) + lm_head, bf16, W.T views, seed 2",
                      **decode_workload(dev, cpu, max(3, min(args.steps, 10)), args.warmup, pk["hbm"])}
    line["casts"] = {"unit": "GB/s", "peak": pk["hbm"], "elements": 1 << 24, **cast_workload(dev, cpu, args.steps, args.warmup, pk["hbm"])}
    line["attention"] = attention_workload(dev, cpu, pk["hbm"], tensor_peak)
    line["tp_layer_1gpu"] = tp_layer_1gpu_workload(dev, cpu, args.steps, args.warmup, tensor_peak)
    line["gated_mlp"] = gated_mlp_workload(dev, cpu, args.steps, args.warmup, tensor_peak)
    line["cpu_baseline"] = cpu_prefill_step(cpu, 4, 1)
    cpu.close()
    dev.sync()
    # the headline end-to-end figure: the same step through the unchanged magnetron core and the backend module
    plug = plugin_e2e(max(8, min(args.steps, 16)))
    if "tflops" in plug:
        line["e2e"] = {"value": plug["tflops"], "unit": "TFLOP/s", "h2d_bytes_per_step": pre["h2d"], "d2h_bytes_per_step": pre["d2h"],
                       "ms_per_step": plug["ms_per_step"], "path": 'mag_matmul on "cuda:0" through the magnetron core and the backend module '
                       "(mag_b200_upload_async / mag_b200_download_async), device " + plug["device"], "timing": plug["timing"],
                       "per_step_sync_ms": plug.get("per_step_sync_ms"), "per_step_sync_tflops": plug.get("per_step_sync_tflops")}
        line["e2e_cabi"] = e2e_cabi
    else:
        line["e2e"] = dict(e2e_cabi, note="plug-in leg: " + plug.get("unavailable", "unavailable"))
    print(json.dumps(line))


if __name__ == "__main__":
    main()
