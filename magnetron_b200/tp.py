"""Tensor-parallel linear layers over the GPUs of one box: one process per GPU, NCCL through torch.distributed.

magnetron has no multi-device code (its README lists multi-GPU as future work); this module is the new host
logic around the unchanged single-GPU matmul. The path shards in two ways:

  column sharding (on N)  each rank holds rows [n0, n1) of a row-major [N, K] weight and computes
                          y[:, n0:n1] = x @ W[n0:n1].T  -- independent GEMMs, no exchange; an all-gather only if
                          the caller wants the full output on every rank;
  row sharding (on K)     each rank holds columns [k0, k1) of the weight and the matching slice of the input,
                          computes a partial y over its K range, and one all-reduce (sum) makes the result.

Paired the Megatron way (column-sharded QKV / gate+up feed row-sharded o / down) a transformer layer needs two
all-reduces and no gather. To hide them the token dimension is cut into chunks that travel through the layer one after
the other (rows are independent): while the all-reduce of chunk c is on the wire, chunk c+1 multiplies. The dependencies
of a real layer are kept -- gate/up of a chunk starts only after that chunk's o-projection all-reduce -- and the GEMMs
leave a few SMs free (magb200_set_cta_limit) so that the collective's kernel can run beside the persistent GEMM.

Device memory is held in torch tensors (so NCCL can see it); the matmuls go through the C ABI of this package on
torch's current stream. There is no CPU path: `TPLayer` raises without the CUDA library. The `matmul` argument
exists so that the collective plumbing can be exercised on CPU ranks (gloo) with a stand-in product.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Callable, Sequence

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class ShardedLinear:
    name: str
    n: int            # out features of the full weight
    k: int            # in features of the full weight
    kind: str         # "col": shard N, "row": shard K
    granule: int = 128  # shard boundaries fall on multiples of this (head_dim keeps heads whole)


# One Qwen3-32B layer: hidden 5120, 64 query heads + 8 KV heads of head_dim 128, intermediate 25600
QWEN3_32B_LAYER = (
    ShardedLinear("qkv", (64 + 8 + 8) * 128, 5120, "col"),
    ShardedLinear("o", 5120, 64 * 128, "row"),
    ShardedLinear("gate_up", 2 * 25600, 5120, "col"),
    ShardedLinear("down", 5120, 25600, "row"),
)


def shard_range(total: int, world: int, rank: int, granule: int = 1) -> tuple[int, int]:
    """[lo, hi) of `total` owned by `rank`: units of `granule` dealt out as evenly as possible, the first
    `units % world` ranks taking one more."""
    if total % granule:
        raise ValueError(f"{total} is not a multiple of the shard granule {granule}")
    units = total // granule
    base, extra = divmod(units, world)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo * granule, hi * granule


def local_shape(spec: ShardedLinear, world: int, rank: int) -> tuple[int, int]:
    """(N_local, K_local) of the weight shard a rank holds."""
    if spec.kind == "col":
        lo, hi = shard_range(spec.n, world, rank, spec.granule)
        return hi - lo, spec.k
    lo, hi = shard_range(spec.k, world, rank, spec.granule)
    return spec.n, hi - lo


def layer_flops(specs: Sequence[ShardedLinear], m: int) -> float:
    return sum(2.0 * m * s.n * s.k for s in specs)


def activation_block(m: int, width: int, seed: int, name: str, index: int) -> torch.Tensor:
    """Columns [index*width, (index+1)*width) of the seeded activation of linear `name`: fp32 ~ N(0,1)."""
    g = torch.Generator(device="cpu").manual_seed(seed * 1000003 + 17 + 7919 * sum(map(ord, name)) + index)
    return torch.randn((m, width), generator=g, dtype=torch.float32)


def cabi_matmul(device: int, reserve_sms: int = 0) -> Callable[[torch.Tensor, torch.Tensor, torch.Tensor], None]:
    """out[M,N] = x[M,K] @ w[N,K].T on `device` through magb200_matmul, on torch's current stream. `reserve_sms` SMs are
    left free by the tensor-core GEMMs for a collective that runs at the same time."""
    import magnetron_b200 as mb
    L = mb.lib()
    mb.check(L.magb200_device_init(device))
    handle = torch.cuda.current_stream(device).cuda_stream
    if not handle:
        raise RuntimeError("make a torch.cuda.Stream current first: the default stream has a null handle, which the C ABI "
                           "reads as 'use the library's own stream', and matmuls would then not be ordered with the collectives")
    mb.check(L.magb200_set_stream(device, C.c_void_p(handle)))
    mb.check(L.magb200_set_cta_limit(device, 148 - reserve_sms if reserve_sms else 0))
    dt = {torch.bfloat16: mb.BFLOAT16, torch.float16: mb.FLOAT16, torch.float32: mb.FLOAT32}

    def view(t: torch.Tensor, shape=None, strides=None):
        return mb.make_view(t.data_ptr(), dt[t.dtype], shape or tuple(t.shape), strides or tuple(t.stride()))

    def matmul(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
        n, k = w.shape
        wt = view(w, (k, n), (w.stride(1), w.stride(0)))      # the W.T view: no copy
        mb.check(L.magb200_matmul(device, C.byref(view(x)), C.byref(wt), C.byref(view(out))))

    return matmul


class FusedRowLinear:
    """Row-sharded linear whose exchange is fused into the GEMM: the tensor-core kernel's epilogue stores every finished
    tile into the staging buffer of the rank that owns those rows (peer-mapped symmetric memory, under the main loop), a
    symmetric-memory barrier orders the ranks, then `magb200_reduce_broadcast` sums the partial blocks and writes the
    finished rows into every rank's output. Symmetric memory and the barrier come from torch (plumbing); both kernels are
    this package's."""

    def __init__(self, m: int, n: int, dtype, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        import magnetron_b200 as mb
        self.mb, self.L = mb, mb.lib()
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if m % self.world:
            raise ValueError(f"token count {m} must be divisible by the {self.world} ranks")
        self.m, self.n, self.dev = m, n, device.index or 0
        self.stage = symm_mem.empty((self.world, m // self.world, n), dtype=dtype, device=device)
        self.out = symm_mem.empty((m, n), dtype=dtype, device=device)
        self.h_stage = symm_mem.rendezvous(self.stage, self.group)
        self.h_out = symm_mem.rendezvous(self.out, self.group)
        self.stage_ptrs = (C.c_void_p * self.world)(*[int(p) for p in self.h_stage.buffer_ptrs])
        self.out_ptrs = (C.c_void_p * self.world)(*[int(p) for p in self.h_out.buffer_ptrs])
        self.dt = {torch.bfloat16: mb.BFLOAT16, torch.float16: mb.FLOAT16}[dtype]

    def scatter(self, x: torch.Tensor, w: torch.Tensor) -> None:
        """First half, on the current stream: the GEMM whose epilogue pushes tiles to their owners, then the barrier after
        which every rank's partial tiles have landed."""
        mb = self.mb
        n, k = w.shape
        xv = mb.make_view(x.data_ptr(), self.dt, tuple(x.shape), tuple(x.stride()))
        wv = mb.make_view(w.data_ptr(), self.dt, (k, n), (w.stride(1), w.stride(0)))
        mb.check(self.L.magb200_matmul_scatter(self.dev, C.byref(xv), C.byref(wv), self.stage_ptrs, self.world, self.rank))
        self.h_stage.barrier(channel=0)

    def finish(self) -> torch.Tensor:
        """Second half, on the current stream (which may be a side stream): sum the partial blocks, write the finished
        rows to every rank, and the barrier after which all rows have landed and the staging buffers may be reused."""
        stream = torch.cuda.current_stream(self.out.device).cuda_stream
        self.mb.check(self.L.magb200_reduce_broadcast(self.dev, C.c_void_p(stream) if stream else None,
                                                      C.c_void_p(self.stage.data_ptr()), self.out_ptrs, self.world, self.rank,
                                                      self.m // self.world, self.n, self.dt))
        self.h_out.barrier(channel=1)
        return self.out

    def __call__(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        self.scatter(x, w)
        return self.finish()


class SwitchRowLinear:
    """Row-sharded linear whose exchange goes through the NVSwitch: the GEMM writes this rank's partial product into its own
    symmetric buffer (plain epilogue, nothing crosses NVLink during the GEMM), a barrier orders the ranks, then
    `magb200_multimem_reduce_broadcast` lets the switch sum this rank's row block over all ranks (multimem.ld_reduce) and write
    the sum into every rank's output (multimem.st). Same two-step interface as FusedRowLinear. Needs a multicast binding of
    the symmetric buffers (NVLS); `available()` says whether this group has one."""

    def __init__(self, m: int, n: int, dtype, device: torch.device, matmul: Callable, group=None, max_ctas: int = 0):
        import torch.distributed._symmetric_memory as symm_mem
        import magnetron_b200 as mb
        self.mb, self.L, self.matmul, self.max_ctas = mb, mb.lib(), matmul, max_ctas
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if m % self.world:
            raise ValueError(f"token count {m} must be divisible by the {self.world} ranks")
        self.m, self.n, self.dev = m, n, device.index or 0
        self.partial = symm_mem.empty((m, n), dtype=dtype, device=device)
        self.out = symm_mem.empty((m, n), dtype=dtype, device=device)
        self.h_partial = symm_mem.rendezvous(self.partial, self.group)
        self.h_out = symm_mem.rendezvous(self.out, self.group)
        self.mc_partial, self.mc_out = int(self.h_partial.multicast_ptr or 0), int(self.h_out.multicast_ptr or 0)
        if not self.mc_partial or not self.mc_out:
            raise RuntimeError("the symmetric buffers have no multicast binding on this system")
        self.dt = {torch.bfloat16: mb.BFLOAT16, torch.float16: mb.FLOAT16}[dtype]

    @staticmethod
    def available(device: torch.device, group=None) -> bool:
        """True when a symmetric allocation of this group comes with a multicast address (probed once with a small buffer)."""
        try:
            import torch.distributed._symmetric_memory as symm_mem
            t = symm_mem.empty((4096,), dtype=torch.bfloat16, device=device)
            h = symm_mem.rendezvous(t, group if group is not None else dist.group.WORLD)
            return bool(h.multicast_ptr)
        except Exception:   # noqa: BLE001 - no symmetric memory, no NVLS: the caller picks another exchange
            return False

    def scatter(self, x: torch.Tensor, w: torch.Tensor) -> None:
        """First half on the current stream: the local GEMM into the symmetric partial buffer, then the barrier after which
        every rank's partial is complete."""
        self.matmul(x, w, self.partial)
        self.h_partial.barrier(channel=0)

    def finish(self) -> torch.Tensor:
        stream = torch.cuda.current_stream(self.out.device).cuda_stream
        self.mb.check(self.L.magb200_multimem_reduce_broadcast(self.dev, C.c_void_p(stream) if stream else None, C.c_void_p(self.mc_partial),
                                                               C.c_void_p(self.mc_out), self.world, self.rank, self.m // self.world, self.n,
                                                               self.dt, self.max_ctas))
        self.h_out.barrier(channel=1)
        return self.out

    def __call__(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        self.scatter(x, w)
        return self.finish()


def plan_linear(spec: ShardedLinear, m: int, world: int, *, peer_access: bool, multicast: bool, dtype_code: int = 2):
    """The library's decision for one linear (magb200_tp_plan): sharding mode, exchange, token chunks, and whether it pays."""
    import magnetron_b200 as mb
    pl = mb.TpPlan()
    mb.check(mb.lib().magb200_tp_plan(m, spec.n, spec.k, world, mb.TP_COLUMN if spec.kind == "col" else mb.TP_ROW, dtype_code,
                                      int(peer_access), int(multicast), C.byref(pl)))
    return {"mode": ["replicate", "column", "row"][pl.mode], "exchange": mb.TP_EXCHANGE[pl.exchange], "chunks": pl.chunks, "pays": bool(pl.pays),
            "single_us": pl.single_us, "sharded_us": pl.sharded_us, "speedup": pl.speedup}


class TPLayer:
    """The sharded linears of one layer on this rank, with resident weight shards and preallocated outputs."""

    def __init__(self, specs: Sequence[ShardedLinear], m: int, *, device: torch.device, dtype=torch.bfloat16,
                 matmul: Callable | None = None, group=None, seed: int = 5, chunks: int = 4, reserve_sms: int = 0,
                 fused: bool = False, exchange: str = "scatter", side_ctas: int = 0, keep_full: Sequence[str] = ()):
        """`fused`: row-sharded linears use a fused exchange of this package instead of NCCL; `exchange` picks it
        ("scatter": scatter epilogue + reduce-broadcast over peer memory, "switch": in-switch reduction, "auto": what
        magb200_tp_plan says, which also sets the chunk count)."""
        self.specs, self.m, self.group = tuple(specs), m, group
        self.plan = None
        self.full_w = {}
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if matmul is None:
            if device.type != "cuda":
                raise RuntimeError("TPLayer runs on CUDA devices only: there is no CPU path")
            matmul = cabi_matmul(device.index or 0, reserve_sms)
        self.matmul = matmul
        if fused and exchange == "auto" and self.world > 1:
            multicast = SwitchRowLinear.available(device, group)
            self.plan = {s.name: plan_linear(s, m, self.world, peer_access=True, multicast=multicast) for s in self.specs}
            rows = [self.plan[s.name] for s in self.specs if s.kind == "row"]
            chunks = max([r["chunks"] for r in rows] or [1])
            kinds = {r["exchange"] for r in rows}
            exchange = "switch" if "switch" in kinds else ("scatter" if "scatter" in kinds else "nccl")
            if exchange == "nccl":
                fused = False
        self.exchange = exchange
        self.chunks = max(1, min(chunks, m // 512)) if m >= 1024 else 1
        self.fused = {}
        self.fused_chunks = {}
        # linears the plan keeps whole on every rank (their exchange would cost more than sharding saves)
        self.replicated = {n for n, pl in (self.plan or {}).items() if pl["mode"] == "replicate"}
        self.side_stream = None
        gen = torch.Generator(device="cpu").manual_seed(seed)
        self.w, self.x, self.y = {}, {}, {}
        for s in self.specs:
            n_loc, k_loc = local_shape(s, self.world, self.rank)
            if s.name in self.replicated and s.n * s.k <= (1 << 27):
                n_loc, k_loc = s.n, s.k
            else:
                self.replicated.discard(s.name)
            # the full weight is drawn from one seeded stream and sliced, so every world size multiplies the
            # same matrix; only the local shard is kept on the device
            full = torch.randn((s.n, s.k), generator=gen, dtype=torch.float32) * 0.02 if s.n * s.k <= (1 << 27) else None
            if full is not None:
                if s.name in self.replicated:
                    shard = full
                elif s.kind == "col":
                    lo, hi = shard_range(s.n, self.world, self.rank, s.granule)
                    shard = full[lo:hi]
                else:
                    lo, hi = shard_range(s.k, self.world, self.rank, s.granule)
                    shard = full[:, lo:hi]
                self.w[s.name] = shard.to(dtype).contiguous().to(device)
            else:  # too large to materialise on the host in one piece: seeded per shard
                g2 = torch.Generator(device="cpu").manual_seed(seed * 1000 + self.rank)
                self.w[s.name] = (torch.randn((n_loc, k_loc), generator=g2, dtype=torch.float32) * 0.02).to(dtype).to(device)
            # the activation is one [m, K] matrix for every world size, drawn in blocks of `granule` columns with a seed per
            # block; a rank materialises only the blocks of its K range (all of them for a column-sharded linear)
            k_lo = shard_range(s.k, self.world, self.rank, s.granule)[0] if (s.kind == "row" and s.name not in self.replicated) else 0
            blocks = [activation_block(m, s.granule, seed, s.name, (k_lo + j) // s.granule) for j in range(0, k_loc, s.granule)]
            self.x[s.name] = torch.cat(blocks, dim=1).to(dtype).to(device)
            if s.name in keep_full and full is not None:
                self.full_w[s.name] = full.to(dtype)
            if fused and s.kind == "row" and s.name not in self.replicated and self.world > 1 and m % self.world == 0 and m >= 256:
                def make(rows):
                    if exchange == "switch":
                        return SwitchRowLinear(rows, s.n, dtype, device, self.matmul, group, side_ctas)
                    return FusedRowLinear(rows, s.n, dtype, device, group)
                self.fused[s.name] = make(m)
                self.y[s.name] = self.fused[s.name].out
                mc = m // self.chunks
                if self.chunks > 1 and m % self.chunks == 0 and mc % self.world == 0:
                    # one exchange object per token chunk, so chunks can be in flight at the same time
                    self.fused_chunks[s.name] = [make(mc) for _ in range(self.chunks)]
            else:
                self.y[s.name] = torch.empty((m, n_loc), dtype=dtype, device=device)

    # -- one linear ---------------------------------------------------------------------------
    def column(self, name: str, gather: bool = False):
        self.matmul(self.x[name], self.w[name], self.y[name])
        if gather and self.world > 1:
            parts = [torch.empty_like(self.y[name]) for _ in range(self.world)]
            dist.all_gather(parts, self.y[name], group=self.group)
            return parts
        return self.y[name]

    def row(self, name: str):
        """Partial product over this rank's K range, then a sum all-reduce; cut into chunks of M so that the
        all-reduce of chunk i runs while chunk i+1 multiplies."""
        x, w, y = self.x[name], self.w[name], self.y[name]
        if self.world == 1 or name in self.replicated:
            self.matmul(x, w, y)
            return y
        works = []
        step = (self.m + self.chunks - 1) // self.chunks
        for lo in range(0, self.m, step):
            hi = min(self.m, lo + step)
            self.matmul(x[lo:hi], w, y[lo:hi])
            works.append(dist.all_reduce(y[lo:hi], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        for wk in works:
            wk.wait()
        return y

    def step(self, gather_outputs: bool = False) -> None:
        for s in self.specs:
            if s.kind == "col":
                self.column(s.name, gather=gather_outputs)
            else:
                self.row(s.name)

    def step_auto(self) -> None:
        """The schedule the library picks for this layer: fused exchange with token chunks in flight when the plan asks for
        chunks, the fused exchange op by op otherwise, NCCL for shapes no fused exchange takes (few tokens)."""
        if self.fused_chunks:
            return self.step_fused_pipelined()
        if self.fused:
            return self.step_fused()
        return self.step(False)

    def step_fused(self) -> None:
        """Op by op, the row-sharded linears through the fused GEMM + exchange kernels."""
        for s in self.specs:
            if s.kind == "col":
                self.column(s.name)
            elif s.name in self.fused:
                self.fused[s.name](self.x[s.name], self.w[s.name])
            else:
                self.row(s.name)

    def step_fused_pipelined(self) -> None:
        """Token chunks through the layer with the fused exchange: the scatter GEMM of a chunk runs on the main stream, its
        reduce-broadcast on a side stream beside the next chunk's GEMMs (which leave SMs free for it); the column GEMM
        that follows a row-sharded one waits for that chunk's exchange, as in a real layer."""
        pairs = [(self.specs[i], self.specs[i + 1]) for i in range(0, len(self.specs) - 1, 2)
                 if self.specs[i].kind == "col" and self.specs[i + 1].kind == "row"]
        if 2 * len(pairs) != len(self.specs) or any(r.name not in self.fused_chunks for _, r in pairs):
            return self.step_fused()
        main = torch.cuda.current_stream()
        if self.side_stream is None:
            self.side_stream = torch.cuda.Stream(device=main.device)
        side = self.side_stream
        mc = self.m // self.chunks
        done = {}

        def run_pair(pi, ci):
            col, row = pairs[pi]
            lo, hi = ci * mc, (ci + 1) * mc
            if pi > 0:
                main.wait_event(done.pop((pi - 1, ci)))
            self.matmul(self.x[col.name][lo:hi], self.w[col.name], self.y[col.name][lo:hi])
            ex = self.fused_chunks[row.name][ci]
            ex.scatter(self.x[row.name][lo:hi], self.w[row.name])
            ready = torch.cuda.Event()
            ready.record(main)
            side.wait_event(ready)
            with torch.cuda.stream(side):
                ex.finish()
                ev = torch.cuda.Event()
                ev.record(side)
            done[(pi, ci)] = ev

        n_p, n_c = len(pairs), self.chunks
        for wave in range(n_c + n_p - 1):
            for pi in range(n_p):
                ci = wave - pi
                if 0 <= ci < n_c:
                    run_pair(pi, ci)
        for ev in done.values():
            main.wait_event(ev)

    def step_pipelined(self) -> None:
        """One layer, token chunks in flight: [col, row, all-reduce] pairs per chunk; the column GEMM that follows a
        row-sharded one waits for that chunk's all-reduce (as the next sub-block of a transformer layer must), everything
        else of the next chunk is issued first so that it overlaps the collective."""
        if self.world == 1 or self.chunks == 1:
            return self.step(False)
        pairs = [(self.specs[i], self.specs[i + 1]) for i in range(0, len(self.specs) - 1, 2)
                 if self.specs[i].kind == "col" and self.specs[i + 1].kind == "row"]
        if 2 * len(pairs) != len(self.specs):
            return self.step(False)
        step = (self.m + self.chunks - 1) // self.chunks
        bounds = [(lo, min(self.m, lo + step)) for lo in range(0, self.m, step)]
        pending = {}   # (pair index, chunk) -> work of the all-reduce that the next pair of that chunk depends on

        def run_pair(pi, ci):
            col, row = pairs[pi]
            lo, hi = bounds[ci]
            if pi > 0:
                pending.pop((pi - 1, ci)).wait()                       # this chunk's previous all-reduce
            self.matmul(self.x[col.name][lo:hi], self.w[col.name], self.y[col.name][lo:hi])
            self.matmul(self.x[row.name][lo:hi], self.w[row.name], self.y[row.name][lo:hi])
            pending[(pi, ci)] = dist.all_reduce(self.y[row.name][lo:hi], op=dist.ReduceOp.SUM, group=self.group, async_op=True)

        # skewed order: pair p of chunk c is issued together with pair p-1 of chunk c+1, so each all-reduce has one
        # pair of GEMMs of the neighbouring chunk to hide behind
        n_p, n_c = len(pairs), len(bounds)
        for wave in range(n_c + n_p - 1):
            for pi in range(n_p):
                ci = wave - pi
                if 0 <= ci < n_c:
                    run_pair(pi, ci)
        for wk in pending.values():
            wk.wait()
