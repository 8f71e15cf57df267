"""Host-side logic of the tensor-parallel layer on CPU: shard planner, and world_size-2 gloo ranks that run the
column / row sharded schedule with a stand-in local product and must reproduce the unsharded result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from magnetron_b200 import tp


def test_shard_ranges_cover_and_respect_granule():
    for total, world, g in [(10240, 8, 128), (51200, 4, 128), (8192, 8, 128), (25600, 8, 128), (5120, 3, 128), (640, 8, 128)]:
        pieces = [tp.shard_range(total, world, r, g) for r in range(world)]
        assert pieces[0][0] == 0 and pieces[-1][1] == total
        for (a, b), (c, d) in zip(pieces, pieces[1:]):
            assert b == c and a % g == 0 and b % g == 0
        sizes = [b - a for a, b in pieces]
        assert max(sizes) - min(sizes) <= g
    with pytest.raises(ValueError):
        tp.shard_range(1000, 4, 0, 128)


def test_layer_flops_and_local_shapes():
    assert tp.layer_flops(tp.QWEN3_32B_LAYER, 8192) == pytest.approx(2 * 8192 * 4.8758e8, rel=1e-3)
    qkv, o, gu, down = tp.QWEN3_32B_LAYER
    assert tp.local_shape(qkv, 8, 0) == (1280, 5120) and tp.local_shape(o, 8, 3) == (5120, 1024)
    assert tp.local_shape(gu, 4, 1) == (12800, 5120) and tp.local_shape(down, 8, 7) == (5120, 3200)


def test_no_cpu_path():
    with pytest.raises(RuntimeError):
        tp.TPLayer(tp.QWEN3_32B_LAYER[:1], 8, device=torch.device("cpu"))


SMALL = (tp.ShardedLinear("qkv", 256, 64, "col", 32), tp.ShardedLinear("o", 64, 128, "row", 32),
         tp.ShardedLinear("gate_up", 512, 64, "col", 32), tp.ShardedLinear("down", 64, 256, "row", 32))


def _standin(x, w, out):
    out.copy_((x.float() @ w.float().T).to(out.dtype))


def _rank_main(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m = 1024   # large enough for the chunked, overlapped all-reduce path (2 chunks)
        layer = tp.TPLayer(SMALL, m, device=torch.device("cpu"), dtype=torch.float32, matmul=_standin)
        assert layer.chunks == 2
        layer.step_pipelined()          # chunks travel through the layer with their all-reduces in flight
        piped = {s.name: layer.y[s.name].clone() for s in SMALL}
        for s in SMALL:
            layer.y[s.name].zero_()
        layer.step(False)
        for s in SMALL:
            assert torch.allclose(piped[s.name], layer.y[s.name], atol=1e-5, rtol=1e-5), s.name
        out = {}
        for s in SMALL:
            if s.kind == "col":
                parts = layer.column(s.name, gather=True)
                out[s.name] = torch.cat(parts, dim=1)
            else:
                out[s.name] = layer.y[s.name].clone()
        # the unsharded activation, rebuilt on its own from the block seeds: every rank must have taken ITS K slice of it
        xs = {s.name: torch.cat([tp.activation_block(m, s.granule, 5, s.name, j) for j in range(s.k // s.granule)], dim=1) for s in SMALL}
        for s in SMALL:
            lo, hi = tp.shard_range(s.k, world, rank, s.granule) if s.kind == "row" else (0, s.k)
            assert torch.equal(layer.x[s.name], xs[s.name][:, lo:hi]), s.name
        if rank == 0:
            gen = torch.Generator(device="cpu").manual_seed(5)
            ok = True
            for s in SMALL:
                full = torch.randn((s.n, s.k), generator=gen, dtype=torch.float32) * 0.02
                want = xs[s.name] @ full.T
                ok &= bool(torch.allclose(out[s.name], want, atol=1e-4, rtol=1e-4))
            ret.put(ok)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_layer():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    ret = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert ret.get(timeout=5) is True


def test_planner_decisions():
    """magb200_tp_plan: column shards never exchange; a row-sharded linear at prefill size takes a fused exchange (through the
    switch when the buffers have a multicast binding) and pays; at one token its all-reduce eats the gain, so it is marked as
    not paying, and an operator that sharding would slow down is kept whole."""
    qkv, o, gate_up, down = tp.QWEN3_32B_LAYER
    big = tp.plan_linear(down, 8192, 8, peer_access=True, multicast=True)
    assert big["mode"] == "row" and big["exchange"] == "switch" and big["pays"] and big["chunks"] == 2
    assert tp.plan_linear(down, 8192, 8, peer_access=True, multicast=False)["exchange"] == "scatter"
    assert tp.plan_linear(down, 8192, 2, peer_access=True, multicast=True)["exchange"] == "scatter"
    assert tp.plan_linear(down, 8192, 8, peer_access=False, multicast=False)["exchange"] == "nccl"
    col = tp.plan_linear(gate_up, 1, 8, peer_access=True, multicast=True)
    assert col["mode"] == "column" and col["exchange"] == "none" and col["pays"]
    tiny = tp.plan_linear(o, 1, 8, peer_access=True, multicast=True)
    assert tiny["exchange"] in ("nccl", "none") and not tiny["pays"]
    assert tp.plan_linear(o, 1, 2, peer_access=True, multicast=True)["mode"] == "replicate"
    for m in (1, 8, 512, 8192):
        for p in (2, 4, 8):
            for spec in tp.QWEN3_32B_LAYER:
                pl = tp.plan_linear(spec, m, p, peer_access=True, multicast=True)
                assert pl["sharded_us"] <= pl["single_us"] * 1.0001 and 1 <= pl["chunks"] <= 4
