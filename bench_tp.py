"""Multi-GPU leg of bench.py: the sharded GEMMs of one Qwen3-32B layer, one rank per GPU (torchrun).

`value` = whole-job TFLOP/s of the layer (7.99 TFLOP at M = 8192) with column-sharded QKV and gate/up, row-sharded o
and down, and the two exchanges of the paired schedule inside the timed region, run with the schedule that the library
itself picks (`TPLayer(exchange="auto")` -> magb200_tp_plan: which exchange, how many token chunks); time is the maximum
over ranks of CUDA-event time. The same line reports the NCCL op-by-op schedule as the baseline the fused exchange is
measured against, the variant that also all-gathers the column-sharded outputs (the configuration with gathered outputs),
a correctness check against the unsharded product, the planner's per-operator decisions and the token sweep M in
{1, 8, 512}. `--all-schedules` (an environment switch, MAGB200_TP_ALL=1) additionally times every other schedule.
`bench.py --gpus 1 --workload tp` runs the same layer unsharded (the one-GPU line of `bench.py` carries the same figure
as `tp_layer_1gpu`).
"""
from __future__ import annotations

import ctypes as C
import json
import os
import sys

import torch
import torch.distributed as dist

from magnetron_b200 import tp


def _time_steps(fn, steps, warmup, device):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(device)
    dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize(device)
    dist.barrier()
    ms = torch.tensor([a.elapsed_time(b)], device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms.item())


def _unsharded_check(layer, name, device):
    """Rank 0 rebuilds the whole activation of linear `name` from the block seeds, multiplies it with the whole weight on
    its own GPU and compares with what the sharded layer left in its output: max |difference| / max |value|."""
    spec = next(s for s in layer.specs if s.name == name)
    got = layer.y[name]
    if dist.get_rank() != 0 or name not in layer.full_w:
        return None
    x = torch.cat([tp.activation_block(layer.m, spec.granule, 5, name, j) for j in range(spec.k // spec.granule)], dim=1)
    x = x.to(got.dtype).to(device)
    w = layer.full_w[name].to(device)
    want = torch.empty((layer.m, spec.n), dtype=got.dtype, device=device)
    layer.matmul(x, w, want)
    torch.cuda.synchronize(device)
    return float((got.float() - want.float()).abs().max() / want.float().abs().max().clamp_min(1e-9))


def main(args, pk):
    import magnetron_b200 as mb
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        if rank == 0:
            import bench
            cpu = bench.CpuRef()
            r = bench.cpu_prefill_step(cpu, max(1, min(args.steps, 20)), min(args.warmup, 1)) if cpu.api else None
            cpu.close()
            line = {"impl": "reference", "metric": "bf16 matmul TFLOP/s", "value": r["value"] if r else None, "unit": "TFLOP/s",
                    "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_pass"] if r else None,
                    "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                    "config": {"workload": "qwen3-32b-tp layer GEMMs; the CPU arm times Qwen3-8B-shaped GEMMs (see cpu_baseline.sample): "
                                           "the reference's FLOP/s does not depend on which of these shapes it multiplies"},
                    "cpu_baseline": r, "e2e": {"value": r["value"] if r else None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
            print(json.dumps(line if r else {"impl": "reference", "unavailable": "oracle/_ref is not built on this machine"}))
        return
    # NCCL prints its version banner on stdout at communicator start-up; stdout must carry the JSON line only, so it is
    # pointed at stderr until the result is printed
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    # SMs the GEMMs leave free for exchange kernels on the side stream; leaving none measured best at every rank count (the
    # exchange kernels then run in the gaps between the persistent GEMMs)
    reserve = int(os.environ.get("MAGB200_TP_RESERVE_SMS", "0")) if world > 1 else 0
    if world > 1:   # before the communicator exists: a collective's kernel must fit in the SMs the GEMMs leave free
        os.environ.setdefault("NCCL_MAX_CTAS", str(max(reserve, 16)))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    # a dedicated stream: the C ABI treats a null handle (torch's default stream) as "use the library's own stream",
    # and the timing events, the matmuls and the collectives must all be ordered on one stream
    torch.cuda.set_stream(torch.cuda.Stream(device))
    if not dist.is_initialized():
        for k, v in (("MASTER_ADDR", "127.0.0.1"), ("MASTER_PORT", "29517"), ("RANK", "0"), ("WORLD_SIZE", "1")):
            os.environ.setdefault(k, v)
        dist.init_process_group("nccl", device_id=device)
    steps, warmup = args.steps, max(args.warmup, 3)
    M = 8192
    specs = tp.QWEN3_32B_LAYER
    flops = tp.layer_flops(specs, M)
    L = mb.lib()
    everything = os.environ.get("MAGB200_TP_ALL") == "1"
    extra, parts = {}, None

    # ---- the library's own choice ------------------------------------------------------------------------------------------
    layer = tp.TPLayer(specs, M, device=device, fused=world > 1, exchange="auto", side_ctas=4 * reserve, keep_full=("o",))
    if layer.fused_chunks and reserve:      # chunks in flight: the GEMMs leave SMs free for the exchange kernels on the side stream
        mb.check(L.magb200_set_cta_limit(local, 148 - reserve))
    L.magb200_launch_count_reset()
    ms = _time_steps(layer.step_auto, steps, warmup, device)
    launches = int(L.magb200_launch_count()) * steps // (steps + warmup)
    mb.check(L.magb200_set_cta_limit(local, 0))
    value = flops * steps / ms / 1e9
    plan = layer.plan
    schedule = {"exchange": layer.exchange if layer.fused else ("nccl" if world > 1 else "none"),
                "token_chunks": layer.chunks if layer.fused_chunks else 1,
                "sms_left_free_for_the_exchange": reserve if layer.fused_chunks else 0}
    check = None
    if world > 1:
        layer.step_fused() if layer.fused else layer.step(False)     # unchunked, so y["o"] holds the whole result
        torch.cuda.synchronize(device)
        check = _unsharded_check(layer, "o", device)
        if layer.fused:
            fl = [layer.fused[s_.name] for s_ in specs if s_.name in layer.fused]
            names = [s_.name for s_ in specs if s_.name in layer.fused]

            def first_half():
                for f, nm in zip(fl, names):
                    f.scatter(layer.x[nm], layer.w[nm])

            def second_half():
                for f in fl:
                    f.finish()

            parts = {"gemm_and_first_barrier_ms": _time_steps(first_half, steps, 2, device) / steps,
                     "reduce_broadcast_and_second_barrier_ms": _time_steps(second_half, steps, 2, device) / steps}
    del layer
    torch.cuda.empty_cache()

    # ---- NCCL baseline and the configuration with output all-gathers -----------------------------------------------------------
    base = tp.TPLayer(specs, M, device=device, reserve_sms=0)
    half = max(2, steps // 2)
    ms_plain = _time_steps(lambda: base.step(False), half, 2, device)
    ms_gather = _time_steps(lambda: base.step(True), half, 2, device) if world > 1 else ms_plain
    extra["op_by_op_nccl"] = {"ms_per_step": ms_plain / half, "tflops": flops * half / ms_plain / 1e9}
    extra["with_output_allgather"] = {"ms_per_step": ms_gather / half, "tflops": flops * half / ms_gather / 1e9}
    del base
    torch.cuda.empty_cache()

    if everything and world > 1:
        for ex in ("scatter", "switch"):
            for n_chunks in (1, 2, 4):
                try:
                    lay = tp.TPLayer(specs, M, device=device, fused=True, exchange=ex, chunks=n_chunks, side_ctas=0)
                    for free_sms in ((0,) if n_chunks == 1 else (0, 16)):
                        mb.check(L.magb200_set_cta_limit(local, 148 - free_sms if free_sms else 0))
                        t = _time_steps(lay.step_auto, steps, warmup, device)
                        extra[f"{ex}_chunks{n_chunks}_free{free_sms}"] = flops * steps / t / 1e9
                    mb.check(L.magb200_set_cta_limit(local, 0))
                    del lay
                except Exception as e:   # noqa: BLE001 - e.g. no multicast binding: reported, not fatal
                    extra[f"{ex}_chunks{n_chunks}"] = repr(e)[:160]
                torch.cuda.empty_cache()

    # ---- token sweep with the planner's decisions ------------------------------------------------------------------------------
    sweep = {}
    for m in (1, 8, 512):
        lay = tp.TPLayer(specs, m, device=device, fused=world > 1, exchange="auto")
        n = max(steps, 20)
        t = _time_steps(lay.step_auto, n, warmup, device)
        wbytes = sum(2 * s.n * s.k for s in specs)
        sweep[f"M{m}"] = {"ms_per_step": t / n, "tflops": tp.layer_flops(specs, m) * n / t / 1e9, "weight_gbs_all_gpus": wbytes * n / t / 1e6,
                          "exchange": lay.exchange if lay.fused else ("nccl" if world > 1 else "none"),
                          "plan": {k: {"mode": v["mode"], "exchange": v["exchange"], "pays": v["pays"], "predicted_speedup": round(v["speedup"], 2)}
                                   for k, v in (lay.plan or {}).items()}}
        del lay
        torch.cuda.empty_cache()
    dist.barrier()
    if rank == 0:
        line = {
            "metric": "bf16 matmul TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "qwen3-32b-tp: QKV [10240x5120] and gate/up [51200x5120] column-sharded on N, o [5120x8192] and "
                                   "down [5120x25600] row-sharded on K, paired schedule (one exchange per row-sharded GEMM, no gather of the "
                                   "column-sharded outputs), M=8192, seed 5", "parallelism": f"tp{world}",
                       "l2": "inputs larger than L2 (975 MB of weights per layer across ranks)"},
            "e2e": {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "host-buffer end-to-end is measured on the 1-GPU line; the sharded layer keeps activations on the device"},
            "gpu_launches": launches,
            "schedule": schedule,
            "schedule_chosen_by": "the library (magb200_tp_plan), not by timing alternatives",
            "plan": {k: {"mode": v["mode"], "exchange": v["exchange"], "chunks": v["chunks"], "pays": v["pays"],
                         "predicted_speedup": round(v["speedup"], 2)} for k, v in (plan or {}).items()},
            "max_rel_diff_vs_unsharded_o_projection": check,
            "exchange_parts": parts,
            "reserved_sms_for_collectives": reserve,
            "token_sweep": sweep,
            "roofline": {"bound": "tensor", "achieved": value / world, "peak": pk["tensor_burst"], "unit": "TFLOP/s per GPU",
                         "frac": value / world / pk["tensor_burst"], "traffic": None, "peak_source": pk["source"] + " burst cuBLAS bf16"},
            **extra,
        }
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        print(json.dumps(line), flush=True)
        os.dup2(2, 1)
    dist.barrier()
    dist.destroy_process_group()
