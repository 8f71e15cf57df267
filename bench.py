#!/usr/bin/env python
"""Benchmark of the matmul / cast hot path on B200 through the C ABI (include/magnetron_b200.h).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload prefill|tp]

One JSON line on stdout. A "step" is one pass of the hot path over one batch of synthetic input:

  N = 1  workload "qwen3-8b-prefill": the seven projection GEMMs of one Qwen3-8B layer at M = 4096 tokens
         (q, k, v, o, gate, up, down; bf16, fp32 accumulation, weights ~ N(0, 0.02^2) through the `W.T`
         view, activations ~ N(0,1), seed 3). `value` = TFLOP/s with everything resident in HBM;
         `e2e` = the same step with the activations coming from pinned host memory and every result
         copied back to it, both copies inside the timed region (on the library's copy streams, so they
         overlap each other and the kernels). The same line carries the decode-shaped
         sweep (`decode`: Qwen3-0.6B, one token pass over 28 layers + lm_head, M in {1,2,4,8}, HBM GB/s)
         and the 16 Mi-element casts (`casts`), each with its own roofline fraction.
  N > 1  workload "qwen3-32b-tp": the four sharded GEMM groups of one Qwen3-32B layer at M = 8192
         (QKV and gate/up column-sharded on N, o and down row-sharded on K with an NCCL all-reduce or the
         fused scatter-epilogue exchange, whichever is faster), one rank per GPU. Total work is fixed, so scaling is "strong".

`--impl reference` times the reference CPU backend (oracle/_ref, all host threads) on a bounded sample of
the same workload and prints the same line with "impl": "reference".
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
# workloads
# ------------------------------------------------------------------------------------------------
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

    # end to end: activations from pinned host memory, every result back to pinned host memory
    pin = {}
    for name, t in list(acts.items()) + [("out_" + n, o) for n, o in outs.items()]:
        p = C.c_void_p()
        mb.check(dev.L.magb200_host_alloc_pinned(C.byref(p), t.numel * 2))
        pin[name] = p
    for name, t in acts.items():
        mb.check(dev.L.magb200_download(dev.d, pin[name], t.ptr, t.numel * 2))
    h2d = sum(t.numel * 2 for t in acts.values())
    d2h = sum(o.numel * 2 for o in outs.values())

    # Each activation is uploaded right before its first consumer and each result is downloaded right after its producer,
    # on the library's copy streams: uploads, kernels and downloads of different operators overlap (the link is full
    # duplex), the GEMMs with the largest results go first so the download stream never idles.
    order = ["gate", "up", "q", "k", "v", "o", "down"]
    by_name = {n: (a, c) for (n, N, K, a), c in zip(PREFILL_GEMMS, calls)}

    def step_e2e():
        uploaded = set()
        for n in order:
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


def decode_workload(dev: Dev, steps: int, warmup: int, hbm_peak: float):
    """One token pass of Qwen3-0.6B (28 layers x 7 projections + lm_head) per step; every launch reads a
    different weight matrix and the 1.19 GB of weights exceed L2 many times over."""
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

        def step():
            for xv, wv, rv in calls:
                dev.matmul(xv, wv, rv)

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
        # lm_head alone (311 MB per launch): the largest single GEMV, timed over two alternating copies is not
        # needed -- 311 MB is 2.5x the L2 capacity
        lm = calls[-1]
        ms_lm, _ = timed(dev, lambda: dev.matmul(*lm), max(steps, 10), warmup)
        gbs = (wbytes + act_bytes) * steps / ms / 1e6
        gbs_lm = (VOCAB * 1024 * 2 + (M * 1024 + M * VOCAB) * 2) * max(steps, 10) / ms_lm / 1e6
        result[f"M{M}"] = {"token_pass_ms": ms / steps, "token_pass_ms_call_by_call": ms_calls / steps, "gbs": gbs, "frac": gbs / hbm_peak, "launches_per_step": launches // steps,
                           "lm_head_ms": ms_lm / max(steps, 10), "lm_head_gbs": gbs_lm, "lm_head_frac": gbs_lm / hbm_peak,
                           "kernel": mb.last_kernel()}
        for t in list(xs.values()) + list(outs.values()):
            t.release()
    for layer in layers:
        for w, _, _ in layer:
            w.release()
    lm_head.release()
    return result


def cast_workload(dev: Dev, steps: int, warmup: int, hbm_peak: float):
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
        out[key] = {"ms": ms / max(steps, 20), "gbs": gbs, "frac": gbs / hbm_peak}
    for t in f32 + b16:
        t.release()
    return out


# ------------------------------------------------------------------------------------------------
# CPU reference (oracle/_ref), bounded sample
# ------------------------------------------------------------------------------------------------
CPU_SAMPLE = [("q", 1024, HIDDEN, HIDDEN), ("k", 1024, KV_DIM, HIDDEN), ("gate", 512, INTER, HIDDEN), ("down", 512, HIDDEN, INTER)]


def cpu_reference(steps: int, warmup: int):
    """The unmodified reference CPU backend on a bounded sample of the prefill step: the q, k, gate and down
    GEMMs at a reduced token count (rows are independent, so FLOP/s at M = 512..1024 tokens stands for the
    full 4096-token GEMM)."""
    from oracle import mag_oracle as O
    from oracle import ref_driver as R
    if not R.available():
        return None
    api = R.MagApi("cpu", log_level=1)
    rng = np.random.default_rng(3)
    work = []
    for name, M, N, K in CPU_SAMPLE:
        x = api.from_bits(BF16, O.f32_to_bits(BF16, rng.standard_normal((M, K), dtype=np.float32)))
        w = api.from_bits(BF16, O.f32_to_bits(BF16, rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)))
        work.append((x, w, api.transpose(w, 0, 1), 2.0 * M * N * K))
    flops = sum(f for *_, f in work)

    def step():
        for x, _, wt, _ in work:
            api.matmul(x, wt).release()

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    res = {"value": flops * steps / dt / 1e12, "unit": "TFLOP/s", "cores": api.cores, "kind": "reference",
           "sample": "q,k at 1024 tokens and gate,down at 512 tokens of the Qwen3-8B prefill step (%.0f GFLOP per pass), "
                     "bf16 through the W.T view, %d passes; CPU %s" % (flops / 1e9, steps, api.cpu_name),
           "ms_per_pass": dt / steps * 1e3}
    for x, w, wt, _ in work:
        wt.release(); w.release(); x.release()
    api.close(True)
    return res


# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-decode", action="store_true", help="only the headline prefill step (used under ncu)")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--workload", default="auto", choices=["auto", "prefill", "tp"],
                    help="auto: Qwen3-8B prefill layer on one GPU, Qwen3-32B tensor-parallel layer on several")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    pk = peaks()

    if args.gpus > 1 or world > 1 or args.workload == "tp":
        from magnetron_b200 import tp_bench
        return tp_bench.main(args, pk)

    config = {"workload": "qwen3-8b-prefill: q,k,v,o,gate,up,down GEMMs of one layer, M=4096 tokens, hidden 4096, "
                          "kv 1024, intermediate 12288, W.T views, seed 3",
              "l2": "inputs larger than L2 (528 MB of operands per step)", "tokens": TOKENS}

    if args.impl == "reference":
        if rank != 0:
            return
        r = cpu_reference(max(1, min(args.steps, 40)), min(args.warmup, 2))
        if r is None:
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref is not built on this machine"}))
            return
        line = {"impl": "reference", "metric": "bf16 matmul TFLOP/s", "value": r["value"], "unit": "TFLOP/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_pass"], "higher_is_better": True,
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
    line = {
        "metric": "bf16 matmul TFLOP/s", "value": pre["tflops"], "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": pre["ms_per_step"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
        "e2e": {"value": pre["e2e_tflops"], "unit": "TFLOP/s", "h2d_bytes_per_step": pre["h2d"], "d2h_bytes_per_step": pre["d2h"],
                "ms_per_step": pre["e2e_ms_per_step"]},
        "gpu_launches": pre["launches"], "clocks": clocks,
        "roofline": {"bound": "tensor", "achieved": pre["tflops"], "peak": tensor_peak, "unit": "TFLOP/s",
                     "frac": pre["tflops"] / tensor_peak,
                     # DRAM bytes per launch: the ncu capture of one 4096^3 launch of the same kernel read+wrote 105.3 MB against
                     # 100.7 MB algorithmic (profiles/gemm_tcgen05_2sm_4096x4096x4096.md); scaled to the step's mean launch
                     "traffic": 1.046 * pre["bytes_per_step"] / len(PREFILL_GEMMS),
                     "traffic_note": "scaled from an ncu capture of a smaller case by algorithmic bytes; mean over the step's 7 launches",
                     "peak_source": "%s %s cuBLAS bf16" % (pk["source"], "sustained" if long_run else "burst"),
                     "frac_of_nominal_2250": pre["tflops"] / 2250.0,
                     "kernel": "gemm_tcgen05_2sm_kernel (q,o,gate,up,down) + gemm_tcgen05_kernel (k,v)",
                     "algorithmic_flops_per_step": pre["flops_per_step"], "algorithmic_bytes_per_step": pre["bytes_per_step"]},
    }
    if not args.skip_decode:
        line["decode"] = {"metric": "decode GEMV HBM GB/s", "unit": "GB/s", "peak": pk["hbm"], "peak_source": pk["source"] + " copy",
                          "note": "gbs/frac = whole token pass replayed as a CUDA graph (197 launches, mostly 2-6 MB each, latency bound); "
                                  "lm_head_* = the 311 MB GEMV alone, the per-kernel HBM figure (kernel skinny_km_async_kernel, "
                                  "ncu: profiles/skinny_km_async_M4_65536x4096.md)",
                          "config": "qwen3-0.6b token pass: 28 layers x (q,k,v,o,gate,up,down) + lm_head, bf16, W.T views, seed 2",
                          **decode_workload(dev, max(3, min(args.steps, 10)), args.warmup, pk["hbm"])}
        line["casts"] = {"unit": "GB/s", "peak": pk["hbm"], "elements": 1 << 24,
                         **cast_workload(dev, args.steps, args.warmup, pk["hbm"])}
    if not args.skip_cpu:
        r = cpu_reference(20, 1)
        line["cpu_baseline"] = r if r else {"value": None, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "reference",
                                            "sample": "oracle/_ref is not built on this machine"}
    print(json.dumps(line))


if __name__ == "__main__":
    main()
