"""Multi-GPU leg of bench.py: the sharded GEMMs of one Qwen3-32B layer, one rank per GPU (torchrun).

`value` = whole-job TFLOP/s of the layer (7.99 TFLOP at M = 8192) with column-sharded QKV and gate/up, row-sharded o
and down, and the two all-reduces of the paired schedule inside the timed region; time is the maximum over ranks of
CUDA-event time. The same line reports the variant that also all-gathers the column-sharded outputs, the token sweep
M in {1, 8, 512}. `bench.py --gpus 1 --workload tp` runs the same layer unsharded as the scaling yardstick (the one-GPU line of
`bench.py` carries the same figure as `tp_layer_1gpu`).
"""
from __future__ import annotations

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
                    "config": {"workload": "qwen3-32b-tp layer GEMMs; CPU sample = bounded Qwen3-8B-shaped GEMMs (see cpu_baseline.sample)"},
                    "cpu_baseline": r, "e2e": {"value": r["value"] if r else None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
            print(json.dumps(line if r else {"impl": "reference", "unavailable": "oracle/_ref is not built on this machine"}))
        return
    # NCCL prints its version banner on stdout at communicator start-up; stdout must carry the JSON line only, so it is
    # pointed at stderr until the result is printed
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    if world > 1:   # before the communicator exists: the collective's kernel must fit in the SMs the GEMMs leave free
        os.environ.setdefault("NCCL_MAX_CTAS", str(max(int(os.environ.get("MAGB200_TP_RESERVE_SMS", "16")), 8)))
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
    reserve = int(os.environ.get("MAGB200_TP_RESERVE_SMS", "16")) if world > 1 else 0
    layer = tp.TPLayer(specs, M, device=device, reserve_sms=reserve)
    mb.lib().magb200_launch_count_reset()
    ms_plain = _time_steps(lambda: layer.step(False), max(2, steps // 2), 2, device)
    mb.lib().magb200_launch_count_reset()
    ms = _time_steps(layer.step_pipelined, steps, warmup, device)
    launches = int(mb.lib().magb200_launch_count()) * steps // (steps + warmup)
    ms_gather = _time_steps(lambda: layer.step(True), max(2, steps // 2), 2, device)
    fused_tflops, fused_err, fused_parts, fused_pipe_tflops, ms_fp, fp_variants = None, None, None, None, None, None
    fp_err = None
    if world > 1:
        layer = None
        torch.cuda.empty_cache()
        try:
            layer = tp.TPLayer(specs, M, device=device, reserve_sms=0, fused=True, chunks=1)
            ms_fused = _time_steps(layer.step_fused, steps, warmup, device)
            fused_tflops = flops * steps / ms_fused / 1e9
            # the same exchange with token chunks in flight: which chunk count and how many SMs left free for the
            # side-stream kernels pays depends on the rank count, so the candidates are timed and the best kept
            fp_variants = {}
            for n_chunks in (2, 4):
                lay = tp.TPLayer(specs, M, device=device, reserve_sms=0, fused=True, chunks=n_chunks)
                for free_sms in (0, reserve):
                    mb.check(mb.lib().magb200_set_cta_limit(local, 148 - free_sms if free_sms else 0))
                    t = _time_steps(lay.step_fused_pipelined, steps, warmup, device)
                    fp_variants[f"chunks{n_chunks}_free{free_sms}"] = flops * steps / t / 1e9
                    if ms_fp is None or t < ms_fp:
                        ms_fp = t
                mb.check(mb.lib().magb200_set_cta_limit(local, 0))
                # the chunked exchange against NCCL on the same operands (outputs of the last timed step)
                torch.cuda.synchronize(device)
                for s_ in specs:
                    if s_.name in lay.fused_chunks:
                        part = torch.empty((M, s_.n), dtype=torch.bfloat16, device=device)
                        lay.matmul(lay.x[s_.name], lay.w[s_.name], part)
                        acc = part.float()
                        dist.all_reduce(acc)
                        got = torch.cat([ex.out for ex in lay.fused_chunks[s_.name]], dim=0).float()
                        err = float((got - acc).abs().max() / acc.abs().max().clamp_min(1e-9))
                        fp_err = max(fp_err or 0.0, err)
                del lay
                torch.cuda.empty_cache()
            fused_pipe_tflops = flops * steps / ms_fp / 1e9
            # cross-check of the fused exchange against NCCL on the same operands
            ref = {}
            for s_ in specs:
                if s_.name in layer.fused:
                    part = torch.empty((M, s_.n), dtype=torch.bfloat16, device=device)
                    layer.matmul(layer.x[s_.name], layer.w[s_.name], part)
                    acc = part.float()
                    dist.all_reduce(acc)
                    layer.fused[s_.name](layer.x[s_.name], layer.w[s_.name])
                    torch.cuda.synchronize(device)
                    err = (layer.y[s_.name].float() - acc).abs().max() / acc.abs().max().clamp_min(1e-9)
                    ref[s_.name] = float(err)
            fused_err = ref
            # where the fused exchange spends its time: the scatter GEMMs alone, and the reduce-broadcast kernels alone
            import ctypes as C
            L = mb.lib()
            fl = [layer.fused[s_.name] for s_ in specs if s_.name in layer.fused]
            names = [s_.name for s_ in specs if s_.name in layer.fused]

            def scatter_only():
                for f, nm in zip(fl, names):
                    x, w = layer.x[nm], layer.w[nm]
                    xv = mb.make_view(x.data_ptr(), f.dt, tuple(x.shape), tuple(x.stride()))
                    wv = mb.make_view(w.data_ptr(), f.dt, (w.shape[1], w.shape[0]), (w.stride(1), w.stride(0)))
                    mb.check(L.magb200_matmul_scatter(f.dev, C.byref(xv), C.byref(wv), f.stage_ptrs, f.world, f.rank))

            def reduce_only():
                for f in fl:
                    mb.check(L.magb200_reduce_broadcast(f.dev, None, C.c_void_p(f.stage.data_ptr()), f.out_ptrs, f.world, f.rank,
                                                        f.m // f.world, f.n, f.dt))

            def barrier_only():
                for f in fl:
                    f.h_stage.barrier(channel=0)
                    f.h_out.barrier(channel=1)

            fused_parts = {"scatter_gemms_ms": _time_steps(scatter_only, steps, 2, device) / steps,
                           "reduce_broadcast_ms": _time_steps(reduce_only, steps, 2, device) / steps,
                           "four_barriers_ms": _time_steps(barrier_only, steps, 2, device) / steps}
        except Exception as e:   # symmetric memory is torch plumbing: report instead of failing the run
            fused_err = {"error": repr(e)[:300]}
    pipelined_tflops = flops * steps / ms / 1e9
    plain_tflops = flops * max(2, steps // 2) / ms_plain / 1e9
    schedule = "token chunks pipelined through the layer" if pipelined_tflops >= plain_tflops else "op by op, all-reduce chunked over M"
    if plain_tflops > pipelined_tflops:   # the headline is the fastest of the legal schedules; all are reported
        ms = ms_plain * steps / max(2, steps // 2)
    if fused_tflops and fused_tflops > max(plain_tflops, pipelined_tflops):
        schedule = "op by op, row-sharded GEMMs fused with their exchange (scatter epilogue + reduce-broadcast over peer memory)"
        ms = ms_fused
    if fused_pipe_tflops and fused_pipe_tflops > max(plain_tflops, pipelined_tflops, fused_tflops or 0.0):
        schedule = "token chunks pipelined through the layer, row-sharded GEMMs fused with their exchange (reduce-broadcast on a side stream)"
        ms = ms_fp
    value = flops * steps / ms / 1e9
    sweep = {}
    del layer
    torch.cuda.empty_cache()
    for m in (1, 8, 512):
        lay = tp.TPLayer(specs, m, device=device)
        t = _time_steps(lambda: lay.step(False), max(steps, 20), warmup, device)
        wbytes = sum(2 * s.n * s.k for s in specs)
        sweep[f"M{m}"] = {"ms_per_step": t / max(steps, 20), "tflops": tp.layer_flops(specs, m) * max(steps, 20) / t / 1e9,
                          "weight_gbs_all_gpus": wbytes * max(steps, 20) / t / 1e6}
        del lay
        torch.cuda.empty_cache()
    dist.barrier()
    if rank == 0:
        line = {
            "metric": "bf16 matmul TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": "qwen3-32b-tp: QKV [10240x5120] and gate/up [51200x5120] column-sharded on N, o [5120x8192] and "
                                   "down [5120x25600] row-sharded on K with an NCCL all-reduce (paired schedule, token chunks pipelined through the "
                                   "layer so all-reduces overlap the next chunk's GEMMs), M=8192, seed 5", "parallelism": f"tp{world}",
                       "l2": "inputs larger than L2 (975 MB of weights per layer across ranks)"},
            "e2e": {"value": None, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "host-buffer end-to-end is measured on the 1-GPU line; the sharded layer keeps activations on the device"},
            "gpu_launches": launches,
            "schedule": schedule,
            "op_by_op_schedule": {"ms_per_step": ms_plain / max(2, steps // 2), "tflops": plain_tflops},
            "pipelined_schedule": {"tflops": pipelined_tflops},
            "fused_exchange_schedule": {"tflops": fused_tflops, "max_rel_diff_vs_nccl": fused_err, "parts": fused_parts},
            "fused_exchange_pipelined_schedule": {"tflops": fused_pipe_tflops, "variants": fp_variants, "max_rel_diff_vs_nccl": fp_err},
            "reserved_sms_for_collectives": reserve,
            "with_output_allgather": {"ms_per_step": ms_gather / max(2, steps // 2), "tflops": flops * max(2, steps // 2) / ms_gather / 1e9},
            "token_sweep": sweep,
            "roofline": {"bound": "tensor", "achieved": value / world, "peak": pk["tensor_burst"], "unit": "TFLOP/s per GPU",
                         "frac": value / world / pk["tensor_burst"], "traffic": None, "peak_source": pk["source"] + " burst cuBLAS bf16"},
        }
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        print(json.dumps(line), flush=True)
        os.dup2(2, 1)
    dist.barrier()
    dist.destroy_process_group()
