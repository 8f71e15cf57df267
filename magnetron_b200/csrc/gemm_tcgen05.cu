// Prefill-shaped bf16/fp16 matmul on the 5th-generation tensor cores (sm_100a).
//
// One persistent CTA per SM walks output tiles of 128 x BN. Three warp roles:
//   warp 0     : TMA producer   -- cp.async.bulk.tensor loads of A (128 x 64) and B (BN x 64) tiles into
//                                  a ring of shared-memory stages (128-byte swizzle), completion on mbarriers
//   warp 1     : MMA issuer     -- one thread issues tcgen05.mma.kind::f16 (M=128, N=BN, K=16) straight from
//                                  shared-memory descriptors, fp32 accumulators live in TMEM; tcgen05.commit
//                                  releases each stage and finally signals the epilogue
//   warps 2..5 : epilogue       -- tcgen05.ld the accumulator (each warp owns its 32 TMEM lanes), round once
//                                  to bf16/fp16 and store to C
// TMEM holds two accumulators (2 x BN columns) so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Operand layouts: either operand may be K-major (inner dim K: the `W.T` view of an nn.Linear weight, or a
// plain row-major activation) or MN-major (inner dim M / N: a contiguous [K,N] weight, V in P.V, a
// transposed activation). The major-ness goes into the instruction descriptor and the shared-memory
// descriptors, so no operand is ever transposed or packed in memory. Batch and broadcast dims become extra
// TMA coordinates (coordinate 0 on a broadcast dim).
//
// Every wait on an mbarrier is bounded: after about a second without progress the kernel raises a status
// word, stops issuing work, drains and frees its TMEM, so a lost signal cannot wedge the device.
#include "common.cuh"

#include <cuda.h>  // CUtensorMap and enums only; the driver entry point is resolved at run time

#include <atomic>

namespace magb200 {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 x 16-bit = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kStatusTimeout = 1;
constexpr int kMaxScatterRanks = 8;

struct TcArgs {
    void *C;
    int64_t M, N, K;
    int dtype;
    int a_mn, b_mn;                     // 1: operand is MN-major
    int nbatch;
    int64_t bshape[kMaxBatchDims];
    int a_has[kMaxBatchDims], b_has[kMaxBatchDims];  // 0: operand is broadcast along this batch dim
    int64_t tiles_m, tiles_n, total_tiles;
    int num_kb;
    int *status;
    // two-SM kernel, balanced last wave: the tiles left over by the full waves are shared out by K (see WorkUnit)
    int64_t full_tiles;                 // tiles handled whole, `num_pairs` per wave
    int tail_tiles, tail_pairs;         // tiles of the partial last wave and the CTA pairs that share them (0: none)
    int num_kg;                         // K groups (stages) per tile
    int tail_slots;                     // partial-sum slots per tail tile in `sk_partial`
    float *sk_partial;                  // fp32 partial tiles of the contributors: [tail tile][slot][256 x 256]
    int *sk_counters;                   // [tail tile][2]: contributions arrived / owner warps done
    uint64_t wait_limit_ns;             // every mbarrier wait gives up after this long without progress
    int skip_kb;                        // test hook: K block of each CTA's first tile whose loads are never issued (-1: none)
    // scatter epilogue (tensor-parallel row-sharded GEMM): rows of block o go to rank o's staging buffer, slot `rank`
    int scatter_ranks;                  // 0: plain epilogue into C
    int scatter_rank;
    int64_t rows_per_rank;
    void *peer_stage[kMaxScatterRanks]; // staging buffer of every rank: [ranks][rows_per_rank][N] elements
};

// Where output row `row` of batch `batch` starts. In scatter mode the row belongs to the rank that owns its row block and
// lands in that rank's staging buffer (an ordinary store through a peer mapping), in the slot of the sending rank.
__device__ __forceinline__ uint16_t *output_row(const TcArgs &a, int64_t batch, int64_t row) {
    if (a.scatter_ranks == 0) return reinterpret_cast<uint16_t *>(a.C) + (batch * a.M + row) * a.N;
    const int64_t owner = row / a.rows_per_rank;
    const int64_t local = row - owner * a.rows_per_rank;
    return reinterpret_cast<uint16_t *>(a.peer_stage[owner < a.scatter_ranks ? owner : 0]) +
           ((int64_t)a.scatter_rank * a.rows_per_rank + local) * a.N;
}

// ---- PTX wrappers -------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait. Returns false (and raises the CTA's abort flag) when the phase did not complete in time.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, uint64_t limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_timer_ns();
    for (uint32_t spin = 0;; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 15u) == 15u) {
            if (*abort_flag) return false;
            if (global_timer_ns() - t0 > limit_ns) { *abort_flag = 1; return false; }
        }
    }
}

__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
// Bulk tensor store shared -> global (the epilogue's write-out): the box is clipped at the tensor's edges, so tails in M and N
// need no predicates. Completion is tracked by the issuing thread's bulk async-groups.
__device__ __forceinline__ void tma_store_5d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2, int c3, int c4) {
    asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// all but the newest bulk store of this thread have read their shared-memory source
__device__ __forceinline__ void tma_store_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tcgen05_mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a 128-byte-swizzled tile (start address, LBO, SBO in 16-byte units;
// bits 46-47 = descriptor version 1, bits 61-63 = 2 for SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}

// Tile order: tiles are walked in groups of kGroupM tile rows, column by column inside a group, so the CTAs that run
// at the same time share a few A row panels and a band of B column panels that together fit in L2 (walking N fastest over
// a wide N would stream all of B once per wave).
constexpr int kGroupM = 8;
__device__ __forceinline__ void decode_tile(int64_t tile, int64_t tiles_m, int64_t tiles_n, int64_t &batch, int64_t &tm, int64_t &tn) {
    const int64_t per_batch = tiles_m * tiles_n;
    batch = tile / per_batch;
    const int64_t t = tile - batch * per_batch;
    const int64_t per_group = (int64_t)kGroupM * tiles_n;
    const int64_t group = t / per_group;
    const int64_t first_m = group * kGroupM;
    const int64_t rows = (tiles_m - first_m) < kGroupM ? (tiles_m - first_m) : kGroupM;
    const int64_t local = t - group * per_group;
    tn = local / rows;
    tm = first_m + (local - tn * rows);
}

template <int BN> struct Cfg {
    static constexpr int kABytes = BM * BK * 2;
    static constexpr int kBBytes = BN * BK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
    static constexpr int kTmemCols = 2 * BN;  // two accumulators; 128 / 256 / 512 columns
    static constexpr int kEpiCols = 64;                  // output columns per staging pass: 128-byte row segments
    static constexpr int kEpiWarpBytes = 32 * kEpiCols * 2;   // one epilogue warp stages its 32 rows, chunks XOR-swizzled by row
    static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/ + 4 * kEpiWarpBytes;
};

// kSplit2: launched as clusters of two CTAs, one tile per cluster: CTA r walks the r-th half of the K blocks, then each CTA
// keeps the half of the tile's columns it owns, sends the other half of its fp32 accumulator to its peer through
// distributed shared memory (the peer's stage buffers, idle by then), adds what it received and stores its columns. For
// outputs with so few tiles that most SMs would idle (512 x 2048 x 2048: 64 tiles of 128 x 128 become 128 CTAs).
template <int BN, int DT, bool kSplit2 = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const TcArgs args) {
    using C = Cfg<BN>;
    // a GEMM launched behind this one as a programmatic dependent (the host has established that it touches nothing this one
    // reads or writes) may take over SMs as this kernel's CTAs finish: the partial last wave of one GEMM runs beside the first
    // wave of the next
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t krank = kSplit2 ? cluster_ctarank() : 0u;
    const int kb_half = (args.num_kb + 1) >> 1;
    const int kb_begin = kSplit2 ? (int)krank * kb_half : 0;
    const int kb_end = kSplit2 ? (kb_begin + kb_half < args.num_kb ? kb_begin + kb_half : args.num_kb) : args.num_kb;
    const int64_t first_tile = kSplit2 ? (int64_t)(blockIdx.x >> 1) : (int64_t)blockIdx.x;
    const int64_t tile_step = kSplit2 ? args.total_tiles : (int64_t)gridDim.x;     // split form: one tile per cluster
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;             // 1024-byte alignment for the 128B swizzle
    unsigned char *tiles_ptr = smem_raw + (tiles - raw);
    uint64_t *bars = reinterpret_cast<uint64_t *>(tiles_ptr + (size_t)C::kStages * C::kStageBytes);
    // barrier slots: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = full0 + 8u * C::kStages;
    const uint32_t tfull0 = empty0 + 8u * C::kStages;
    const uint32_t tempty0 = tfull0 + 16u;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars + 2 * C::kStages + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * C::kStages + 5);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) { mbar_init(full0 + 8u * s, 1); mbar_init(empty0 + 8u * s, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(tfull0 + 8u * i, 1); mbar_init(tempty0 + 8u * i, 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
    }
    if (warp == 1) {  // TMEM allocation is a warp-wide operation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void *)tmem_slot)), "r"((uint32_t)C::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ===================== TMA producer (one thread) =====================
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int64_t tile = first_tile; ok && tile < args.total_tiles; tile += tile_step) {
                int64_t batch, tm, tn;
                decode_tile(tile, args.tiles_m, args.tiles_n, batch, tm, tn);
                const int m0 = (int)(tm * BM), n0 = (int)(tn * BN);
                int bc[kMaxBatchDims] = {0, 0, 0};
                {
                    int64_t rem = batch;
                    for (int d = args.nbatch - 1; d >= 0; --d) {
                        int64_t q = rem / args.bshape[d];
                        bc[d] = (int)(rem - q * args.bshape[d]);
                        rem = q;
                    }
                }
                // TMA coordinates are fastest-dim first: {inner, outer, b2, b1, b0}
                const int a2 = args.a_has[2] ? bc[2] : 0, a1 = args.a_has[1] ? bc[1] : 0, a0 = args.a_has[0] ? bc[0] : 0;
                const int b2 = args.b_has[2] ? bc[2] : 0, b1 = args.b_has[1] ? bc[1] : 0, b0 = args.b_has[0] ? bc[0] : 0;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait(empty0 + 8u * stage, phase ^ 1u, abort_flag, args.wait_limit_ns)) { ok = false; break; }
                    if (kb == args.skip_kb && tile == (int64_t)blockIdx.x) {   // test hook: this stage is never armed, its consumer's wait runs out
                        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                        continue;
                    }
                    const uint32_t full = full0 + 8u * stage;
                    const uint32_t sa = tiles + (uint32_t)stage * C::kStageBytes;
                    const uint32_t sb = sa + C::kABytes;
                    mbar_arrive_expect_tx(full, (uint32_t)C::kStageBytes);
                    const int k0 = kb * BK;
                    if (!args.a_mn) {
                        tma_load_5d(sa, &tmA, full, k0, m0, a2, a1, a0);               // box {64 k, 128 m}
                    } else {
#pragma unroll
                        for (int c = 0; c < BM / 64; ++c)                                 // boxes {64 m, 64 k}
                            tma_load_5d(sa + c * 8192, &tmA, full, m0 + c * 64, k0, a2, a1, a0);
                    }
                    if (!args.b_mn) {
                        tma_load_5d(sb, &tmB, full, k0, n0, b2, b1, b0);               // box {64 k, BN n}
                    } else {
#pragma unroll
                        for (int c = 0; c < BN / 64; ++c)                                 // boxes {64 n, 64 k}
                            tma_load_5d(sb + c * 8192, &tmB, full, n0 + c * 64, k0, b2, b1, b0);
                    }
                    if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
        if constexpr (kSplit2) { cluster_sync_all(); cluster_sync_all(); }   // the two meeting points of the epilogue warps
    } else if (warp == 1) {
        // ===================== MMA issuer (one thread) =====================
        if (lane == 0) {
            // instruction descriptor: fp32 accumulate, A/B format, major-ness, N>>3 at bit 17, M>>4 at bit 24
            const uint32_t fmt = (DT == MAGB200_BF16) ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)args.a_mn << 15) |
                                   ((uint32_t)args.b_mn << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            // K-major tile: rows of 128 bytes, 8-row swizzle atoms 1024 bytes apart (SBO), K step = 32 bytes.
            // MN-major tile: chunks of 64 (MN) x 64 (K): 8-row K atoms 1024 bytes apart (SBO), MN chunks 8192
            // bytes apart (LBO), K step of 16 rows = 2048 bytes.
            const uint32_t a_lbo = args.a_mn ? 8192u : 16u, a_step = args.a_mn ? 2048u : 32u;
            const uint32_t b_lbo = args.b_mn ? 8192u : 16u, b_step = args.b_mn ? 2048u : 32u;
            int stage = 0;
            uint32_t phase = 0;
            uint32_t titer = 0;
            bool ok = true;
            for (int64_t tile = first_tile; ok && tile < args.total_tiles; tile += tile_step, ++titer) {
                const uint32_t acc = titer & 1u, acc_phase = (titer >> 1) & 1u;
                if (!mbar_wait(tempty0 + 8u * acc, acc_phase ^ 1u, abort_flag, args.wait_limit_ns)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN;
                for (int kb = kb_begin; kb < kb_end; ++kb) {
                    if (!mbar_wait(full0 + 8u * stage, phase, abort_flag, args.wait_limit_ns)) { ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t sa = tiles + (uint32_t)stage * C::kStageBytes;
                    const uint32_t sb = sa + C::kABytes;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t ad = make_smem_desc(sa + k * a_step, a_lbo, 1024u);
                        const uint64_t bd = make_smem_desc(sb + k * b_step, b_lbo, 1024u);
                        tcgen05_mma_f16(tmem_d, ad, bd, idesc, ((kb - kb_begin) | k) ? 1u : 0u);
                    }
                    tcgen05_commit(empty0 + 8u * stage);   // stage is free once these MMAs have read it
                    if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) tcgen05_commit(tfull0 + 8u * acc);  // accumulator complete
            }
        }
        if constexpr (kSplit2) { cluster_sync_all(); cluster_sync_all(); }
    } else {
        // ===================== epilogue (4 warps, 32 TMEM lanes each) =====================
        const int quarter = warp & 3;  // a warp may only touch TMEM lanes [32*(warp%4), +32)
        uint32_t titer = 0;
        bool ok = true;
        const bool vec_ok = (args.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(args.C) & 15u) == 0);
        const bool staged = args.total_tiles > (int64_t)gridDim.x || args.scatter_ranks > 0;
        for (int64_t tile = first_tile; ok && tile < args.total_tiles; tile += tile_step, ++titer) {
            const uint32_t acc = titer & 1u, acc_phase = (titer >> 1) & 1u;
            int64_t batch, tm, tn;
            decode_tile(tile, args.tiles_m, args.tiles_n, batch, tm, tn);
            const int64_t row = tm * BM + quarter * 32 + lane;
            const int64_t n0 = tn * BN;
            // every lane waits (each needs the acquire), then the warp agrees on one outcome so that the
            // warp-wide tcgen05.ld below is never reached by a partial warp
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(tfull0 + 8u * acc, acc_phase, abort_flag, args.wait_limit_ns));
            if constexpr (kSplit2) {
                // both halves of K are complete in the two CTAs' TMEM and nobody reads the stage buffers any more
                tcgen05_fence_after();
                cluster_sync_all();
                constexpr int kOwn = BN / 2;                                  // columns this CTA finishes: [krank * kOwn, +kOwn)
                const uint32_t tb = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
                const uint32_t slot = (uint32_t)(quarter * 32 + lane) * 4u;   // element (row, col) of a half: (col * 128 + row) * 4 bytes
                if (ok) {
                    const uint32_t remote = map_to_cta(tiles, krank ^ 1u);
#pragma unroll 1
                    for (int c = 0; c < kOwn; c += 32) {
                        uint32_t r[32];
                        tmem_ld_32x32(tb + (krank ^ 1u) * kOwn + c, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(remote + (uint32_t)(c + j) * 512u + slot), "r"(r[j]) : "memory");
                    }
                }
                cluster_sync_all();                                           // the peer's half of my columns has arrived
                if (ok) {
                    uint16_t *crow = output_row(args, batch, row < args.M ? row : 0) + n0 + krank * kOwn;
#pragma unroll 1
                    for (int c = 0; c < kOwn; c += 32) {
                        uint32_t r[32];
                        tmem_ld_32x32(tb + krank * kOwn + c, r);
                        tmem_ld_wait();
                        float f[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            f[j] = __uint_as_float(r[j]) + *reinterpret_cast<const float *>(tiles_ptr + (size_t)(c + j) * 512 + slot);
                        if (row < args.M) {
                            const int64_t col0 = n0 + krank * kOwn + c;
                            if (vec_ok) {
#pragma unroll
                                for (int v = 0; v < 4; ++v)
                                    if (col0 + 8 * v < args.N) {
                                        uint4 o;
                                        o.x = pack2_rn<DT>(f[8 * v + 0], f[8 * v + 1]);
                                        o.y = pack2_rn<DT>(f[8 * v + 2], f[8 * v + 3]);
                                        o.z = pack2_rn<DT>(f[8 * v + 4], f[8 * v + 5]);
                                        o.w = pack2_rn<DT>(f[8 * v + 6], f[8 * v + 7]);
                                        *reinterpret_cast<uint4 *>(crow + c + 8 * v) = o;
                                    }
                            } else {
#pragma unroll
                                for (int j = 0; j < 32; ++j)
                                    if (col0 + j < args.N) store_from_f32<DT>(crow, c + j, f[j]);
                            }
                        }
                    }
                }
                break;                                                        // one tile per cluster
            }
            if (!ok) break;
            tcgen05_fence_after();
            if (vec_ok && !staged) {
                // single wave: nothing follows this tile, so the shortest path to global memory wins (16-byte stores per lane)
                uint16_t *crow = output_row(args, batch, row < args.M ? row : 0) + n0;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + c, r);
                    tmem_ld_wait();
                    if (row < args.M) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {
                            if (n0 + c + 8 * v < args.N) {
                                uint4 o;
                                o.x = pack2_rn<DT>(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
                                o.y = pack2_rn<DT>(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
                                o.z = pack2_rn<DT>(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
                                o.w = pack2_rn<DT>(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
                                *reinterpret_cast<uint4 *>(crow + c + 8 * v) = o;
                            }
                        }
                    }
                }
            } else if (vec_ok) {
                // Staged epilogue: TMEM -> registers -> this warp's shared-memory patch (row = lane, 16-byte chunk c of a row
                // kept at chunk c ^ (row & 7)), then 8 lanes write one row's 128 contiguous bytes. The next TMEM loads are
                // issued before the write-out.
                unsigned char *stg = tiles_ptr + (size_t)C::kStages * C::kStageBytes + 256 + (size_t)quarter * C::kEpiWarpBytes;
                const int64_t row0 = tm * BM + quarter * 32;
                const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
                uint32_t ra[32], rb[32];
                tmem_ld_32x32(tbase, ra);
                tmem_ld_32x32(tbase + 32, rb);
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += C::kEpiCols) {
                    tmem_ld_wait();
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint4 o, q;
                        o.x = pack2_rn<DT>(__uint_as_float(ra[8 * v + 0]), __uint_as_float(ra[8 * v + 1]));
                        o.y = pack2_rn<DT>(__uint_as_float(ra[8 * v + 2]), __uint_as_float(ra[8 * v + 3]));
                        o.z = pack2_rn<DT>(__uint_as_float(ra[8 * v + 4]), __uint_as_float(ra[8 * v + 5]));
                        o.w = pack2_rn<DT>(__uint_as_float(ra[8 * v + 6]), __uint_as_float(ra[8 * v + 7]));
                        q.x = pack2_rn<DT>(__uint_as_float(rb[8 * v + 0]), __uint_as_float(rb[8 * v + 1]));
                        q.y = pack2_rn<DT>(__uint_as_float(rb[8 * v + 2]), __uint_as_float(rb[8 * v + 3]));
                        q.z = pack2_rn<DT>(__uint_as_float(rb[8 * v + 4]), __uint_as_float(rb[8 * v + 5]));
                        q.w = pack2_rn<DT>(__uint_as_float(rb[8 * v + 6]), __uint_as_float(rb[8 * v + 7]));
                        *reinterpret_cast<uint4 *>(stg + lane * (C::kEpiCols * 2) + ((v ^ (lane & 7)) << 4)) = o;
                        *reinterpret_cast<uint4 *>(stg + lane * (C::kEpiCols * 2) + (((v + 4) ^ (lane & 7)) << 4)) = q;
                    }
                    if (c0 + C::kEpiCols < BN) {   // in flight during the write-out
                        tmem_ld_32x32(tbase + c0 + C::kEpiCols, ra);
                        tmem_ld_32x32(tbase + c0 + C::kEpiCols + 32, rb);
                    }
                    __syncwarp();
                    const int64_t col = n0 + c0 + (lane & 7) * 8;
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int rr = it * 4 + (lane >> 3);
                        const int64_t grow = row0 + rr;
                        if (grow < args.M && col < args.N) {
                            const uint4 v = *reinterpret_cast<const uint4 *>(stg + rr * (C::kEpiCols * 2) + (((lane & 7) ^ (rr & 7)) << 4));
                            *reinterpret_cast<uint4 *>(output_row(args, batch, grow) + col) = v;
                        }
                    }
                    __syncwarp();
                }
            } else {
                uint16_t *crow = output_row(args, batch, row < args.M ? row : 0) + n0;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + c, r);
                    tmem_ld_wait();
                    if (row < args.M && n0 + c < args.N) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n0 + c + j < args.N) store_from_f32<DT>(crow, c + j, __uint_as_float(r[j]));
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8u * acc);
        }
    }

    // ---- teardown: everyone meets here (all waits above are bounded), then the allocating warp frees TMEM
    tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0 && args.status) atomicExch(args.status, kStatusTimeout);
        // let copies and MMAs that were already issued land before the shared memory and TMEM go away
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols) : "memory");
    }
}


// =====================================================================================================================
// Two-SM variant: a cluster of two CTAs computes one 256 x 256 tile with tcgen05.mma.cta_group::2.
//
// Why: a single-CTA 128 x 256 tile pulls 48 KB through L2 -> shared memory per 64-wide K block, about 96 bytes per clock
// per SM, which is what bounds the one-CTA kernel. In a pair, CTA r loads only its 128 rows of A and its 128-column half of
// B (32 KB per K block per SM); the MMA issued by the leader CTA reads both halves of B from the two shared memories and
// writes each CTA's 128 accumulator rows into that CTA's TMEM. Loads are plain (non-multicast) TMA in the cta_group::2 form,
// whose completion may be counted on the leader's mbarrier.
//
// Signalling across the pair (no multicast form is used anywhere):
//   full[s]    lives in the leader; both CTAs' TMA loads complete on it; the leader's producer arms it with the byte count
//              of both CTAs.
//   empty[s]   one per CTA; the leader's MMA thread issues two tcgen05.commit per K block, one to its own barrier and one
//              to the peer's (a shared::cluster address), so both producers learn at once that the stage is free.
//   tfull[a]   accumulator a complete: likewise committed to both CTAs' barriers.
//   tempty[a]  accumulator a drained: the 8 epilogue warps of BOTH CTAs arrive on the leader's barrier (count 16).
//
// A stage holds 128 K values (two 64-wide sub-blocks, each a 128-byte-swizzled tile as TMA writes it), so one barrier round
// trip of the MMA thread covers eight tcgen05.mma instead of four. That thread is the scarce resource: issuing one MMA costs
// it about 65 clocks, a wait, two commits and the loop bookkeeping about 350 more, against 128 clocks of tensor-pipe time per
// MMA. With four MMAs per round trip the thread needed about 610 clocks for 512 clocks of tensor work (measured with the
// loads switched off: the pipe was idle 16 % of the time whatever the memory system did); with eight it needs about 870 for
// 1024 and the pipe is the limit.
// =====================================================================================================================
constexpr int kThreads2 = 320;  // warp 0 TMA, warp 1 MMA (leader only), warps 2-9 epilogue (two per TMEM lane quarter)
constexpr int BN2 = 256;

template <int KSUB> struct Cfg2 {
    static constexpr int kSub = KSUB;                            // 64-wide K sub-blocks per stage (2: the long-K default)
    static constexpr int kSubABytes = BM * BK * 2;               // this CTA's 128 rows of A, one sub-block
    static constexpr int kSubBBytes = (BN2 / 2) * BK * 2;        // this CTA's 128 columns of B, one sub-block
    static constexpr int kABytes = kSub * kSubABytes;
    static constexpr int kBBytes = kSub * kSubBBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;        // 64 KB
    static constexpr int kStages = 6 / KSUB;
    static constexpr int kTmemCols = 2 * BN2;
    static constexpr int kEpiWarps = 8;                           // two warps per TMEM lane quarter, 128 columns each
    static constexpr int kEpiCols = 64;                           // output columns per staging pass: 128-byte row segments
    static constexpr int kEpiPitch = kEpiCols * 2;                // no padding: 16-byte chunks are XOR-swizzled by row instead
    static constexpr int kEpiWarpBytes = 32 * kEpiPitch;          // one epilogue warp stages its 32 rows
    static constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + 1024 + 256 + kEpiWarps * kEpiWarpBytes;
};

__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Same arrive without the release fence. A release at cluster scope waits until the warp's earlier global stores are
// performed; an epilogue warp that only hands back an accumulator it has finished reading (tcgen05.wait::ld has returned)
// has nothing to publish, and with the fence every tile paid a store round trip before the next MMA could start.
__device__ __forceinline__ void mbar_arrive_remote_relaxed(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_5d_2sm(uint32_t dst, const CUtensorMap *map, uint32_t bar_cluster_addr,
                                                int c0, int c1, int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
__device__ __forceinline__ void tcgen05_commit_2sm(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- balanced last wave ---------------------------------------------------------------------------------------------------
// A persistent grid of P CTA pairs finishes T tiles in ceil(T / P) tile times; the pairs without a tile in the last wave idle
// (256 tiles on 74 pairs: 3.46 waves of work take 4). Narrower tiles do not help: a tcgen05.mma occupies the issuing thread
// and the pipe about as long at N = 64 as at N = 256. So the r = T mod P tiles of the last wave are shared out along K
// instead: their r * num_kg K groups are dealt to Q pairs in equal contiguous runs. A run that starts at K group 0 of a tile
// makes its pair the tile's owner; any other run is a contribution: its pair writes the fp32 accumulator to a scratch slot
// and raises the tile's counter, the owner adds the contributions in run order (fixed, so results do not depend on timing),
// rounds once and stores. A pair's run may cross from the end of one tile into the start of the next: then it contributes
// first and owns second, so an owner only ever waits for pairs that are not waiting for anybody.
struct WorkUnit {
    int64_t tile;
    int kg0, kg1;        // K groups [kg0, kg1) of the tile
    int part, parts;     // run index within the tile (0: owner) and number of runs
    int tail_idx;        // index among the tail tiles (-1: a whole tile)
};
__device__ __forceinline__ int tail_pair_of(const TcArgs &a, int64_t kg_index) {   // pair whose run holds this K group
    const int64_t R = (int64_t)a.tail_tiles * a.num_kg;
    return (int)(((kg_index + 1) * a.tail_pairs + R - 1) / R - 1);
}
// The u-th unit of `pair` (u = 0, 1, ...); false when the pair has no further work.
__device__ __forceinline__ bool work_unit(const TcArgs &a, int64_t pair, int64_t num_pairs, int u, WorkUnit &w) {
    const int64_t whole = pair + (int64_t)u * num_pairs;
    if (whole < a.full_tiles) { w.tile = whole; w.kg0 = 0; w.kg1 = a.num_kg; w.part = 0; w.parts = 1; w.tail_idx = -1; return true; }
    const int v = u - (int)(a.full_tiles / num_pairs);   // full_tiles is a multiple of num_pairs: every pair had as many whole tiles
    if (a.tail_pairs == 0 || pair >= a.tail_pairs || v > 1) return false;
    const int64_t R = (int64_t)a.tail_tiles * a.num_kg;
    const int64_t lo = pair * R / a.tail_pairs, hi = (pair + 1) * R / a.tail_pairs;
    const int64_t ta = lo / a.num_kg;
    const int64_t end_a = hi < (ta + 1) * a.num_kg ? hi : (ta + 1) * a.num_kg;
    int64_t t, k0, k1;
    if (v == 0) { t = ta; k0 = lo - ta * a.num_kg; k1 = end_a - ta * a.num_kg; }
    else {
        if (end_a >= hi) return false;
        t = ta + 1; k0 = 0; k1 = hi - t * a.num_kg;
    }
    const int owner = tail_pair_of(a, t * a.num_kg), last = tail_pair_of(a, (t + 1) * a.num_kg - 1);
    w.tile = a.full_tiles + t; w.kg0 = (int)k0; w.kg1 = (int)k1;
    w.part = (int)pair - owner; w.parts = last - owner + 1; w.tail_idx = (int)t;
    return true;
}

// tcgen05.mma with each shared-memory descriptor given as (low word, high word): from one K step, sub-block or stage to the
// next only the low word (the start address in 16-byte units) moves, one integer add per operand on the issuing thread.
__device__ __forceinline__ void tcgen05_mma_f16_2sm_split(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate) : "memory");
}

// kShare: this launch shares its last wave out (see WorkUnit). A separate instantiation, because the sharing paths cost the
// epilogue of every tile about 15 % on short-K shapes even when they are never taken (registers and scheduling of the
// drain loop: measured on Q.K^T with K = 128, 0.66 ms against 0.56 ms).
// kTmaStore: the staged 32 x 64 patches leave through cp.async.bulk.tensor stores (one instruction per patch instead of
// eight shared loads and eight predicated 16-byte global stores per lane); used whenever the result is a plain local
// tensor TMA can describe. The scatter epilogue (peer stores) and the shared last wave keep the per-lane write-out.
// kSwiGLU: the gated-MLP form out = silu(x @ Wg) * (x @ Wu). A tile is 256 rows x 128 OUTPUT columns: CTA 0 of the pair loads
// the 128 gate rows of Wg (tmB), CTA 1 the 128 up rows of Wu (tmB2) for the same outputs, so accumulator columns [0,128) hold
// x @ Wg and [128,256) x @ Wu, and the drain combines column j with column 128 + j (with the roundings of the unfused
// operator sequence) before the bulk store: half the result bytes of two GEMMs, and no pass over them afterwards.
template <int DT, int KSUB, bool kShare, bool kTmaStore, bool kSwiGLU>
__global__ void __launch_bounds__(kThreads2, 1)
gemm_tcgen05_2sm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                        const __grid_constant__ CUtensorMap tmB2, const __grid_constant__ CUtensorMap tmC, const TcArgs args) {
    static_assert(!kSwiGLU || (kTmaStore && !kShare), "the gated form leaves through the bulk-store epilogue, whole tiles only");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // see gemm_tcgen05_kernel
    constexpr int kTileN = kSwiGLU ? BN2 / 2 : BN2;      // output columns of a tile
    using C = Cfg2<KSUB>;
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    unsigned char *tiles_ptr = smem_raw + (tiles - raw);
    // layout: [stages][epilogue patches, 4 KB per warp, 1024-byte aligned as the 128-byte swizzle wants][barriers]
    uint64_t *bars = reinterpret_cast<uint64_t *>(tiles_ptr + (size_t)C::kStages * C::kStageBytes + (size_t)C::kEpiWarps * C::kEpiWarpBytes);
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = full0 + 8u * C::kStages;
    const uint32_t tfull0 = empty0 + 8u * C::kStages;
    const uint32_t tempty0 = tfull0 + 16u;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars + 2 * C::kStages + 4);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 2 * C::kStages + 5);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();          // 0: leader (issues the MMAs), 1: peer
    const bool leader = rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) { mbar_init(full0 + 8u * s, 1); mbar_init(empty0 + 8u * s, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(tfull0 + 8u * i, 1); mbar_init(tempty0 + 8u * i, 2 * C::kEpiWarps); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
        if constexpr (kSwiGLU) prefetch_tmap(&tmB2);
    }
    if (warp == 1) {  // both CTAs of the pair allocate, same warp index in each
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void *)tmem_slot)), "r"((uint32_t)C::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync_all();                                // barriers of both CTAs exist before anyone signals across
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t num_pairs = gridDim.x >> 1;
    const int64_t pair = blockIdx.x >> 1;

    if (warp == 0) {
        // ===================== TMA producer (one thread per CTA) =====================
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint32_t full_leader0 = map_to_cta(full0, 0);
            WorkUnit w;
            for (int u = 0; ok && work_unit(args, pair, num_pairs, u, w); ++u) {
                int64_t batch, tm, tn;
                decode_tile(w.tile, args.tiles_m, args.tiles_n, batch, tm, tn);
                const int m0 = (int)(tm * 2 * BM) + (int)rank * BM;        // this CTA's 128 rows of the 256-row tile
                // this CTA's 128 columns of B: half of a 256-column tile, or (gated form) the tile's gate / up columns
                const int n0 = kSwiGLU ? (int)(tn * kTileN) : (int)(tn * BN2) + (int)rank * (BN2 / 2);
                const CUtensorMap *mapB = (kSwiGLU && rank == 1) ? &tmB2 : &tmB;
                int bc[kMaxBatchDims] = {0, 0, 0};
                {
                    int64_t rem = batch;
                    for (int d = args.nbatch - 1; d >= 0; --d) {
                        int64_t q = rem / args.bshape[d];
                        bc[d] = (int)(rem - q * args.bshape[d]);
                        rem = q;
                    }
                }
                const int a2 = args.a_has[2] ? bc[2] : 0, a1 = args.a_has[1] ? bc[1] : 0, a0 = args.a_has[0] ? bc[0] : 0;
                const int b2 = args.b_has[2] ? bc[2] : 0, b1 = args.b_has[1] ? bc[1] : 0, b0 = args.b_has[0] ? bc[0] : 0;
                for (int kg = w.kg0; kg < w.kg1; ++kg) {   // a sub-block past the end of K is zero-filled by TMA
                    if (!mbar_wait(empty0 + 8u * stage, phase ^ 1u, abort_flag, args.wait_limit_ns)) { ok = false; break; }
                    if (kg == args.skip_kb && u == 0) {   // test hook: neither CTA loads or arms this stage, the MMA thread's wait runs out
                        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                        continue;
                    }
                    const uint32_t full = full_leader0 + 8u * stage;
                    const uint32_t sa = tiles + (uint32_t)stage * C::kStageBytes;
                    const uint32_t sb = sa + C::kABytes;
                    if (leader) {
                        mbar_arrive_expect_tx(full0 + 8u * stage, 2u * (uint32_t)C::kStageBytes);
                    }
#pragma unroll
                    for (int sub = 0; sub < C::kSub; ++sub) {
                        const int k0 = (kg * C::kSub + sub) * BK;
                        const uint32_t ssa = sa + sub * C::kSubABytes, ssb = sb + sub * C::kSubBBytes;
                        if (!args.a_mn) {
                            tma_load_5d_2sm(ssa, &tmA, full, k0, m0, a2, a1, a0);
                        } else {
#pragma unroll
                            for (int c = 0; c < BM / 64; ++c) tma_load_5d_2sm(ssa + c * 8192, &tmA, full, m0 + c * 64, k0, a2, a1, a0);
                        }
                        if (!args.b_mn) {
                            tma_load_5d_2sm(ssb, mapB, full, k0, n0, b2, b1, b0);
                        } else {
#pragma unroll
                            for (int c = 0; c < (BN2 / 2) / 64; ++c) tma_load_5d_2sm(ssb + c * 8192, mapB, full, n0 + c * 64, k0, b2, b1, b0);
                        }
                    }
                    if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ===================== MMA issuer (one thread of the leader CTA) =====================
        if (leader && lane == 0) {
            const uint32_t fmt = (DT == MAGB200_BF16) ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)args.a_mn << 15) |
                                   ((uint32_t)args.b_mn << 16) | ((uint32_t)(BN2 >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
            const uint32_t a_lbo = args.a_mn ? 8192u : 16u, a_step = args.a_mn ? 2048u : 32u;
            const uint32_t b_lbo = args.b_mn ? 8192u : 16u, b_step = args.b_mn ? 2048u : 32u;
            const uint32_t empty_peer0 = map_to_cta(empty0, 1), tfull_peer0 = map_to_cta(tfull0, 1);
            // descriptors of stage 0, sub-block 0
            const uint64_t adesc0 = make_smem_desc(tiles, a_lbo, 1024u), bdesc0 = make_smem_desc(tiles + C::kABytes, b_lbo, 1024u);
            const uint32_t a_hi = (uint32_t)(adesc0 >> 32), b_hi = (uint32_t)(bdesc0 >> 32);
            const uint32_t a_k = a_step >> 4, b_k = b_step >> 4;                                      // one K step of 16
            constexpr uint32_t kStage16 = (uint32_t)C::kStageBytes >> 4;
            constexpr uint32_t kSubA16 = (uint32_t)C::kSubABytes >> 4, kSubB16 = (uint32_t)C::kSubBBytes >> 4;
            int stage = 0;
            uint32_t phase = 0, titer = 0;
            uint32_t a_lo = (uint32_t)adesc0, b_lo = (uint32_t)bdesc0;                                // of the current stage
            uint32_t full = full0, empty_own = empty0, empty_peer = empty_peer0;
            bool ok = true;
            WorkUnit w;
            for (int u = 0; ok && work_unit(args, pair, num_pairs, u, w); ++u, ++titer) {
                const uint32_t acc = titer & 1u, acc_phase = (titer >> 1) & 1u;
                if (!mbar_wait(tempty0 + 8u * acc, acc_phase ^ 1u, abort_flag, args.wait_limit_ns)) { ok = false; break; }
                tcgen05_fence_after();
                const uint32_t tmem_d = tmem_base + acc * BN2;
                for (int kg = w.kg0; kg < w.kg1; ++kg) {
                    if (!mbar_wait(full, phase, abort_flag, args.wait_limit_ns)) { ok = false; break; }
                    tcgen05_fence_after();
                    tcgen05_mma_f16_2sm_split(tmem_d, a_lo, a_hi, b_lo, b_hi, idesc, kg != w.kg0 ? 1u : 0u);
                    tcgen05_mma_f16_2sm_split(tmem_d, a_lo + a_k, a_hi, b_lo + b_k, b_hi, idesc, 1u);
                    tcgen05_mma_f16_2sm_split(tmem_d, a_lo + 2 * a_k, a_hi, b_lo + 2 * b_k, b_hi, idesc, 1u);
                    tcgen05_mma_f16_2sm_split(tmem_d, a_lo + 3 * a_k, a_hi, b_lo + 3 * b_k, b_hi, idesc, 1u);
                    if constexpr (KSUB == 2) {
                        tcgen05_mma_f16_2sm_split(tmem_d, a_lo + kSubA16, a_hi, b_lo + kSubB16, b_hi, idesc, 1u);
                        tcgen05_mma_f16_2sm_split(tmem_d, a_lo + kSubA16 + a_k, a_hi, b_lo + kSubB16 + b_k, b_hi, idesc, 1u);
                        tcgen05_mma_f16_2sm_split(tmem_d, a_lo + kSubA16 + 2 * a_k, a_hi, b_lo + kSubB16 + 2 * b_k, b_hi, idesc, 1u);
                        tcgen05_mma_f16_2sm_split(tmem_d, a_lo + kSubA16 + 3 * a_k, a_hi, b_lo + kSubB16 + 3 * b_k, b_hi, idesc, 1u);
                    }
                    tcgen05_commit_2sm(empty_own);        // stage free: tell this CTA's producer ...
                    tcgen05_commit_2sm(empty_peer);       // ... and the peer's
                    if (++stage == C::kStages) {
                        stage = 0; phase ^= 1u;
                        a_lo = (uint32_t)adesc0; b_lo = (uint32_t)bdesc0; full = full0; empty_own = empty0; empty_peer = empty_peer0;
                    } else {
                        a_lo += kStage16; b_lo += kStage16; full += 8u; empty_own += 8u; empty_peer += 8u;
                    }
                }
                if (ok) { tcgen05_commit_2sm(tfull0 + 8u * acc); tcgen05_commit_2sm(tfull_peer0 + 8u * acc); }
            }
        }
    } else {
        // ===================== epilogue (8 warps per CTA, this CTA's 128 accumulator rows) =====================
        const int quarter = warp & 3;
        uint32_t titer = 0;
        bool ok = true;
        const bool vec_ok = (args.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(args.C) & 15u) == 0);
        const uint32_t tempty_leader0 = map_to_cta(tempty0, 0);
        WorkUnit w;
        for (int u = 0; ok && work_unit(args, pair, num_pairs, u, w); ++u, ++titer) {
            const uint32_t acc = titer & 1u, acc_phase = (titer >> 1) & 1u;
            int64_t batch, tm, tn;
            decode_tile(w.tile, args.tiles_m, args.tiles_n, batch, tm, tn);
            const int64_t row = tm * 2 * BM + (int64_t)rank * BM + quarter * 32 + lane;
            const int64_t n0 = tn * kTileN;
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(tfull0 + 8u * acc, acc_phase, abort_flag, args.wait_limit_ns));
            if (!ok) break;
            tcgen05_fence_after();
            const int chalf = (warp - 2) >> 2;            // which 128-column half of the tile this warp drains
            if constexpr (kSwiGLU) {
                // this warp's 32 rows x 64 output columns [chalf * 64, +64): gate from accumulator column c, up from column 128 + c
                unsigned char *stg = tiles_ptr + (size_t)C::kStages * C::kStageBytes + (size_t)(warp - 2) * C::kEpiWarpBytes;
                const int64_t row0 = tm * 2 * BM + (int64_t)rank * BM + quarter * 32;
                const uint32_t tb = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN2 + chalf * 64;
#pragma unroll 1
                for (int h = 0; h < 2; ++h) {
                    uint32_t g[32], up[32];
                    tmem_ld_32x32(tb + h * 32, g);
                    tmem_ld_32x32(tb + BN2 / 2 + h * 32, up);
                    tmem_ld_wait();
                    if (h == 1) {                        // the accumulator has been read completely: hand it back
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_remote_relaxed(tempty_leader0 + 8u * acc);
                    }
                    if (lane == 0) tma_store_wait_read_but_one();   // the store that last used this half of the patch has read it
                    __syncwarp();
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint4 o;
                        o.x = swiglu_pack2<DT>(pack2_rn<DT>(__uint_as_float(g[8 * v + 0]), __uint_as_float(g[8 * v + 1])),
                                               pack2_rn<DT>(__uint_as_float(up[8 * v + 0]), __uint_as_float(up[8 * v + 1])));
                        o.y = swiglu_pack2<DT>(pack2_rn<DT>(__uint_as_float(g[8 * v + 2]), __uint_as_float(g[8 * v + 3])),
                                               pack2_rn<DT>(__uint_as_float(up[8 * v + 2]), __uint_as_float(up[8 * v + 3])));
                        o.z = swiglu_pack2<DT>(pack2_rn<DT>(__uint_as_float(g[8 * v + 4]), __uint_as_float(g[8 * v + 5])),
                                               pack2_rn<DT>(__uint_as_float(up[8 * v + 4]), __uint_as_float(up[8 * v + 5])));
                        o.w = swiglu_pack2<DT>(pack2_rn<DT>(__uint_as_float(g[8 * v + 6]), __uint_as_float(g[8 * v + 7])),
                                               pack2_rn<DT>(__uint_as_float(up[8 * v + 6]), __uint_as_float(up[8 * v + 7])));
                        *reinterpret_cast<uint4 *>(stg + h * 2048 + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) = o;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0 && row0 < args.M && n0 + chalf * 64 + h * 32 < args.N)
                        tma_store_5d(&tmC, smem_u32(stg + h * 2048), (int)(n0 + chalf * 64 + h * 32), (int)row0, (int)batch, 0, 0);
                }
                continue;
            }
            // This warp's 32 x 128 block of a partial tile in scratch: [32-column chunk][accumulator register][lane], so that
            // the 32 lanes of every store and load touch 128 contiguous bytes. Contributor and owner use the same mapping.
            const size_t warp_block = ((size_t)rank * C::kEpiWarps + (size_t)(warp - 2)) * (32 * (BN2 / 2));
            if (kShare && w.part > 0) {
                // ---- contribution: the fp32 accumulator goes to this run's scratch slot, then the tile's counter is raised
                float *slot = args.sk_partial + ((size_t)w.tail_idx * args.tail_slots + (size_t)(w.part - 1)) * (size_t)(2 * BM * BN2) + warp_block;
                const uint32_t tb = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN2 + chalf * (BN2 / 2);
#pragma unroll 1
                for (int c = 0; c < BN2 / 2; c += 32) {
                    uint32_t r[32];
                    tmem_ld_32x32(tb + c, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) __stcg(slot + (size_t)c * 32 + i * 32 + lane, __uint_as_float(r[i]));
                }
                tcgen05_fence_before();
                __threadfence();                           // the stores are visible device-wide before the counter moves
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_remote_relaxed(tempty_leader0 + 8u * acc);
                    atomicAdd(args.sk_counters + 2 * w.tail_idx, 1);
                }
                continue;
            }
            if (kShare && w.parts > 1) {
                // ---- owner of a shared tile: wait (bounded) until every contributing warp has delivered
                const int want = (w.parts - 1) * 2 * C::kEpiWarps;
                const volatile int *cnt = args.sk_counters + 2 * w.tail_idx;
                bool there = *cnt >= want;
                if (!there) {
                    const uint64_t t0 = global_timer_ns();
                    for (uint32_t spin = 0; !(there = (*cnt >= want)); ++spin) {
                        __nanosleep(64);
                        if ((spin & 15u) == 15u && (*abort_flag || global_timer_ns() - t0 > args.wait_limit_ns)) { *abort_flag = 1; break; }
                    }
                }
                ok = __all_sync(0xFFFFFFFFu, there);
                if (!ok) break;
                __threadfence();                           // acquire: the contributions are read after the counter
            }
            const float *contrib = args.sk_partial + (size_t)(w.tail_idx < 0 ? 0 : w.tail_idx) * args.tail_slots * (size_t)(2 * BM * BN2) + warp_block;
            if constexpr (kTmaStore) {
                // Bulk-store epilogue: the warp's 4 KB patch is two halves of 32 rows x 32 columns, each laid out as a
                // 64-byte-swizzled box (row = lane, 16-byte chunk c kept at chunk c ^ ((row >> 1) & 3): conflict-free stores).
                // A half is converted and handed to one bulk tensor store while the store of the other half is still reading
                // its shared memory and the next TMEM load is in flight; rows beyond M and columns beyond N are clipped by TMA.
                unsigned char *stg = tiles_ptr + (size_t)C::kStages * C::kStageBytes + (size_t)(warp - 2) * C::kEpiWarpBytes;
                const int64_t row0 = tm * 2 * BM + (int64_t)rank * BM + quarter * 32;
                const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN2 + chalf * (BN2 / 2);
                uint32_t ra[32];
                tmem_ld_32x32(tbase, ra);
#pragma unroll 1
                for (int c0 = 0; c0 < BN2 / 2; c0 += 32) {
                    unsigned char *half = stg + ((c0 >> 5) & 1) * 2048;
                    tmem_ld_wait();
                    uint4 o[4];
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        o[v].x = pack2_rn<DT>(__uint_as_float(ra[8 * v + 0]), __uint_as_float(ra[8 * v + 1]));
                        o[v].y = pack2_rn<DT>(__uint_as_float(ra[8 * v + 2]), __uint_as_float(ra[8 * v + 3]));
                        o[v].z = pack2_rn<DT>(__uint_as_float(ra[8 * v + 4]), __uint_as_float(ra[8 * v + 5]));
                        o[v].w = pack2_rn<DT>(__uint_as_float(ra[8 * v + 6]), __uint_as_float(ra[8 * v + 7]));
                    }
                    if (c0 + 32 < BN2 / 2) {
                        tmem_ld_32x32(tbase + c0 + 32, ra);          // in flight during the write-out
                    } else {
                        // the accumulator has been read completely: hand it back before the last write-out, so the next
                        // tile's MMAs do not wait for this tile's stores
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_remote_relaxed(tempty_leader0 + 8u * acc);
                    }
                    if (lane == 0) tma_store_wait_read_but_one();   // the store that last used this half has read it
                    __syncwarp();
#pragma unroll
                    for (int v = 0; v < 4; ++v)
                        *reinterpret_cast<uint4 *>(half + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) = o[v];
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0 && row0 < args.M && n0 + chalf * (BN2 / 2) + c0 < args.N)
                        tma_store_5d(&tmC, smem_u32(half), (int)(n0 + chalf * (BN2 / 2) + c0), (int)row0, (int)batch, 0, 0);
                }
            } else if (vec_ok) {
                // Staged epilogue: TMEM -> registers -> this warp's shared-memory patch (row = lane, 16-byte chunk c of a row
                // kept at chunk c ^ (row & 7), conflict-free both ways), then 8 lanes write one row's 128 contiguous bytes, so
                // global and peer stores are whole 128-byte segments. The next TMEM loads are issued before the write-out.
                unsigned char *stg = tiles_ptr + (size_t)C::kStages * C::kStageBytes + (size_t)(warp - 2) * C::kEpiWarpBytes;
                const int64_t row0 = tm * 2 * BM + (int64_t)rank * BM + quarter * 32;
                const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN2 + chalf * (BN2 / 2);
                uint32_t ra[32], rb[32];
                tmem_ld_32x32(tbase, ra);
                tmem_ld_32x32(tbase + 32, rb);
#pragma unroll 1
                for (int c0 = 0; c0 < BN2 / 2; c0 += C::kEpiCols) {
                    tmem_ld_wait();
                    for (int j = 1; kShare && j < w.parts; ++j) {      // contributions in run order: the sum does not depend on timing
                        const float *pj = contrib + (size_t)(j - 1) * (size_t)(2 * BM * BN2) + (size_t)c0 * 32 + lane;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            ra[i] = __float_as_uint(__uint_as_float(ra[i]) + __ldcg(pj + i * 32));
                            rb[i] = __float_as_uint(__uint_as_float(rb[i]) + __ldcg(pj + 1024 + i * 32));
                        }
                    }
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        uint4 o, q;
                        o.x = pack2_rn<DT>(__uint_as_float(ra[8 * v + 0]), __uint_as_float(ra[8 * v + 1]));
                        o.y = pack2_rn<DT>(__uint_as_float(ra[8 * v + 2]), __uint_as_float(ra[8 * v + 3]));
                        o.z = pack2_rn<DT>(__uint_as_float(ra[8 * v + 4]), __uint_as_float(ra[8 * v + 5]));
                        o.w = pack2_rn<DT>(__uint_as_float(ra[8 * v + 6]), __uint_as_float(ra[8 * v + 7]));
                        q.x = pack2_rn<DT>(__uint_as_float(rb[8 * v + 0]), __uint_as_float(rb[8 * v + 1]));
                        q.y = pack2_rn<DT>(__uint_as_float(rb[8 * v + 2]), __uint_as_float(rb[8 * v + 3]));
                        q.z = pack2_rn<DT>(__uint_as_float(rb[8 * v + 4]), __uint_as_float(rb[8 * v + 5]));
                        q.w = pack2_rn<DT>(__uint_as_float(rb[8 * v + 6]), __uint_as_float(rb[8 * v + 7]));
                        *reinterpret_cast<uint4 *>(stg + lane * C::kEpiPitch + ((v ^ (lane & 7)) << 4)) = o;
                        *reinterpret_cast<uint4 *>(stg + lane * C::kEpiPitch + (((v + 4) ^ (lane & 7)) << 4)) = q;
                    }
                    if (c0 + C::kEpiCols < BN2 / 2) {   // in flight during the write-out
                        tmem_ld_32x32(tbase + c0 + C::kEpiCols, ra);
                        tmem_ld_32x32(tbase + c0 + C::kEpiCols + 32, rb);
                    } else {
                        // the accumulator has been read completely: hand it back before the last write-out, so the next
                        // tile's MMAs do not wait for this tile's stores
                        tcgen05_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_remote_relaxed(tempty_leader0 + 8u * acc);
                    }
                    {
                    __syncwarp();
                    const int64_t col = n0 + chalf * (BN2 / 2) + c0 + (lane & 7) * 8;
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int rr = it * 4 + (lane >> 3);
                        const int64_t grow = row0 + rr;
                        if (grow < args.M && col < args.N) {
                            const uint4 v = *reinterpret_cast<const uint4 *>(stg + rr * C::kEpiPitch + (((lane & 7) ^ (rr & 7)) << 4));
                            *reinterpret_cast<uint4 *>(output_row(args, batch, grow) + col) = v;
                        }
                    }
                    __syncwarp();
                    }
                }
            } else {
            uint16_t *crow = output_row(args, batch, row < args.M ? row : 0) + n0;
#pragma unroll 1
            for (int c = chalf * (BN2 / 2); c < (chalf + 1) * (BN2 / 2); c += 32) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN2 + c, r);
                tmem_ld_wait();
                for (int j = 1; kShare && j < w.parts; ++j) {
                    const float *pj = contrib + (size_t)(j - 1) * (size_t)(2 * BM * BN2) + (size_t)(c - chalf * (BN2 / 2)) * 32 + lane;
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __ldcg(pj + i * 32));
                }
                if (row < args.M && n0 + c < args.N) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (n0 + c + j < args.N) store_from_f32<DT>(crow, c + j, __uint_as_float(r[j]));
                }
            }
                tcgen05_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_remote(tempty_leader0 + 8u * acc);   // leader's barrier counts all 16 epilogue warps of the pair
            }
            if (kShare && w.parts > 1) {
                // every contribution has been read by this warp; the last of the pair's 16 epilogue warps to get here clears the
                // tile's counters for the next launch (no contribution can still arrive: all were counted before the reads)
                __threadfence();
                __syncwarp();
                if (lane == 0 && atomicAdd(args.sk_counters + 2 * w.tail_idx + 1, 1) == 2 * C::kEpiWarps - 1) {
                    args.sk_counters[2 * w.tail_idx] = 0;
                    args.sk_counters[2 * w.tail_idx + 1] = 0;
                }
            }
        }
        if constexpr (kTmaStore) {      // the shared-memory patches must outlive the bulk stores that read them
            if (lane == 0) tma_store_wait_all();
        }
    }

    // ---- teardown: both CTAs meet (every wait above is bounded), then each frees its half of the allocation
    tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0 && args.status) atomicExch(args.status, kStatusTimeout);
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)C::kTmemCols) : "memory");
    }
}

// =====================================================================================================================
// float32 on the tensor cores: split operands.
//
// Every fp32 operand element is the sum of three bf16 values, a = a0 + a1 + a2 with 8 significant bits each (cast.cu writes
// the three planes), so a * b = a0 b0 + (a0 b1 + a1 b0) + (a0 b2 + a1 b1 + a2 b0) + terms below 2^-26 |a b|: six bf16 MMAs
// whose products are exact in the fp32 accumulator. What decides the accuracy is the accumulation, and a tensor-core
// accumulator that walked all of K would do no better than a plain fp32 chain (which misses the reference's accuracy by a
// factor of five). So the leading products a0 b0 of one 64-wide K block go to a FRESH accumulator (four MMAs), which the
// eight drain warps then fold into per-thread running totals with an error-free TwoSum while the tensor core is already
// filling the other of two such accumulators; the five small products (2^-8 and 2^-16 of the leading one) collect in a third
// accumulator over all of K, where their own rounding is far below the result's last place, and are added once at the end.
//
// One 128 x 128 tile per CTA. A stage holds one K block of all six planes (96 KB), two stages. Warp 0 lane 0: TMA producer;
// warp 1 lane 0: MMA issue (24 per K block); warps 2-9: drain (warp w owns TMEM lanes 32 (w % 4) .. +31 and 64 columns).
// A drain thread keeps its 64 running totals in registers; their 64 low parts, touched once per K block, live in the
// fourth quarter of TMEM (tcgen05.ld / tcgen05.st of the thread's own lane and columns), because ten warps leave a thread
// 168 registers (three warps share one scheduler's 16 K).
// TMEM columns: [0,128) and [128,256) the two leading-product accumulators, [256,384) the small products, [384,512) low parts.
//
// What bounds it: a 128 x 128 x 16 MMA reads 8 KB of shared memory for 64 clocks of tensor work, which is the whole 128 bytes
// per clock a shared memory delivers, and the TMA writes of the next stage come on top; a wider tile would need more than the
// 512 TMEM columns (two fresh accumulators, the small products and the low parts for every column).
// =====================================================================================================================
constexpr int kF3Threads = 320;
constexpr int kF3BN = 128;
constexpr int kF3PlaneBytes = BM * BK * 2;                 // one plane of one operand: 128 rows x 64 K values
constexpr int kF3StageBytes = 6 * kF3PlaneBytes;
constexpr int kF3Stages = 2;
constexpr uint32_t kF3TmemCols = 512;
constexpr size_t kF3SmemBytes = (size_t)kF3Stages * kF3StageBytes + 1024 + 256;

struct F3Args {
    float *C;
    int64_t M, N, K;
    int nbatch;
    int64_t bshape[kMaxBatchDims];
    int a_has[kMaxBatchDims], b_has[kMaxBatchDims];
    int64_t tiles_m, tiles_n;
    int num_kb;
    int *status;
    const int *skip_if_set;
    uint64_t wait_limit_ns;
};

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// s + e == a + b exactly
__device__ __forceinline__ void two_sum_f3(float a, float b, float &s, float &e) {
    const float sum = __fadd_rn(a, b);
    const float bp = __fsub_rn(sum, a);
    e = __fadd_rn(__fsub_rn(a, __fsub_rn(sum, bp)), __fsub_rn(b, bp));
    s = sum;
}

// kSplitK: launched as clusters of two CTAs that share one tile: CTA r of the pair walks the r-th half of the K blocks, and
// at the end CTA 1 hands its (total, low) pairs to CTA 0 through distributed shared memory (CTA 0's stage buffers, idle by
// then), where they are added with one more TwoSum: an output with fewer tiles than half the SMs keeps twice as many busy.
template <bool kSplitK>
__global__ void __launch_bounds__(kF3Threads, 1)
gemm_f32x3_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const F3Args args) {
    extern __shared__ unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t tiles = (raw + 1023u) & ~1023u;
    unsigned char *tiles_ptr = smem_raw + (tiles - raw);
    uint64_t *bars = reinterpret_cast<uint64_t *>(tiles_ptr + (size_t)kF3Stages * kF3StageBytes);
    // barrier slots: full[2], empty[2], mfull[2] (leading accumulator complete), mfree[2] (drained), cfull (small products complete)
    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = full0 + 16u, mfull0 = full0 + 32u, mfree0 = full0 + 48u, cfull = full0 + 64u;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(bars + 9);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bars + 10);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(full0 + 8u * i, 1); mbar_init(empty0 + 8u * i, 1);
            mbar_init(mfull0 + 8u * i, 1); mbar_init(mfree0 + 8u * i, 8);
        }
        mbar_init(cfull, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        prefetch_tmap(&tmA);
        prefetch_tmap(&tmB);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void *)tmem_slot)), "r"(kF3TmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // Launched as a programmatic dependent of the split pass: everything above ran beside it; its planes and its verdict are
    // read only from here on. The stand-by FFMA launch behind this kernel may set itself up now (it waits before it reads).
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // the operands cannot be split: nothing to do here, the FFMA kernel computes the product (same answer in every thread
    // of both CTAs of a cluster, so the cluster's meeting points below are skipped by all of them)
    const bool skip = args.skip_if_set && *reinterpret_cast<const volatile int *>(args.skip_if_set) != 0;

    int64_t batch, tm, tn;
    decode_tile(kSplitK ? (int64_t)(blockIdx.x >> 1) : (int64_t)blockIdx.x, args.tiles_m, args.tiles_n, batch, tm, tn);
    const int m0 = (int)(tm * BM), n0 = (int)(tn * kF3BN);
    const uint32_t krank = kSplitK ? cluster_ctarank() : 0u;
    const int kb_half = (args.num_kb + 1) >> 1;
    const int kb_begin = kSplitK ? (int)krank * kb_half : 0;
    const int kb_end = kSplitK ? (kb_begin + kb_half < args.num_kb ? kb_begin + kb_half : args.num_kb) : args.num_kb;
    const int nkb = kb_end - kb_begin;                 // K blocks of this CTA

    if (skip) {
        // straight to the teardown
    } else if (warp == 0) {
        if (lane == 0) {
            int bc[kMaxBatchDims] = {0, 0, 0};
            {
                int64_t rem = batch;
                for (int d = args.nbatch - 1; d >= 0; --d) {
                    int64_t q = rem / args.bshape[d];
                    bc[d] = (int)(rem - q * args.bshape[d]);
                    rem = q;
                }
            }
            const int a2 = args.a_has[2] ? bc[2] : 0, a1 = args.a_has[1] ? bc[1] : 0, a0 = args.a_has[0] ? bc[0] : 0;
            const int b2 = args.b_has[2] ? bc[2] : 0, b1 = args.b_has[1] ? bc[1] : 0, b0 = args.b_has[0] ? bc[0] : 0;
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = 0; kb < nkb; ++kb) {
                if (!mbar_wait(empty0 + 8u * stage, phase ^ 1u, abort_flag, args.wait_limit_ns)) break;
                const uint32_t full = full0 + 8u * stage;
                const uint32_t sa = tiles + (uint32_t)stage * kF3StageBytes;
                mbar_arrive_expect_tx(full, (uint32_t)kF3StageBytes);
                const int k0 = (kb_begin + kb) * BK;
#pragma unroll
                for (int pl = 0; pl < 3; ++pl) {   // plane pl of an operand starts pl * rows further down the stacked row dim
                    tma_load_5d(sa + pl * kF3PlaneBytes, &tmA, full, k0, pl * (int)args.M + m0, a2, a1, a0);
                    tma_load_5d(sa + (3 + pl) * kF3PlaneBytes, &tmB, full, k0, pl * (int)args.N + n0, b2, b1, b0);
                }
                if (++stage == kF3Stages) { stage = 0; phase ^= 1u; }
            }
        }
        if constexpr (kSplitK) { cluster_sync_all(); cluster_sync_all(); }
    } else if (warp == 1) {
        if (lane == 0) {
            // bf16 operands, fp32 accumulate, both K-major, N = 128, M = 128
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kF3BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            const uint64_t dbase = make_smem_desc(tiles, 16u, 1024u);   // K-major, 128-byte rows, 8-row swizzle atoms 1024 bytes apart
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = 0; ok && kb < nkb; ++kb) {
                const uint32_t mb = (uint32_t)kb & 1u;
                if (!mbar_wait(full0 + 8u * stage, phase, abort_flag, args.wait_limit_ns)) { ok = false; break; }
                if (!mbar_wait(mfree0 + 8u * mb, (((uint32_t)kb >> 1) & 1u) ^ 1u, abort_flag, args.wait_limit_ns)) { ok = false; break; }
                tcgen05_fence_after();
                // descriptors differ only in their start-address field (16-byte units, no carry out of it below 256 KB): one add each
                const uint64_t da = dbase + (uint64_t)(((uint32_t)stage * kF3StageBytes) >> 4);
                const uint64_t db = da + (uint64_t)((3 * kF3PlaneBytes) >> 4);
                // leading products into the fresh accumulator of this K block
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                    tcgen05_mma_f16(tmem_base + mb * kF3BN, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, k ? 1u : 0u);
                tcgen05_commit(mfull0 + 8u * mb);
                // the five small products, smallest first, into the accumulator that spans all of K
#pragma unroll
                for (int t = 0; t < 5; ++t) {
                    const int pa = (t == 0) ? 2 : (t == 1) ? 1 : (t == 2) ? 0 : (t == 3) ? 1 : 0;
                    const int pb = (t == 0) ? 0 : (t == 1) ? 1 : (t == 2) ? 2 : (t == 3) ? 0 : 1;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        tcgen05_mma_f16(tmem_base + 2 * kF3BN, da + (uint64_t)((pa * kF3PlaneBytes + k * 32) >> 4),
                                        db + (uint64_t)((pb * kF3PlaneBytes + k * 32) >> 4), idesc, (kb | t | k) ? 1u : 0u);
                }
                tcgen05_commit(empty0 + 8u * stage);
                if (++stage == kF3Stages) { stage = 0; phase ^= 1u; }
            }
            if (ok) tcgen05_commit(cfull);
        }
        if constexpr (kSplitK) { cluster_sync_all(); cluster_sync_all(); }   // the two meeting points of the drain warps below
    } else {
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)half * 64u;
        const uint32_t low_base = lane_base + 3 * kF3BN;
        float total[64];
#pragma unroll
        for (int j = 0; j < 64; ++j) total[j] = 0.f;
        bool ok = true;
        for (int kb = 0; kb < nkb; ++kb) {
            const uint32_t mb = (uint32_t)kb & 1u;
            ok = __all_sync(0xFFFFFFFFu, mbar_wait(mfull0 + 8u * mb, ((uint32_t)kb >> 1) & 1u, abort_flag, args.wait_limit_ns));
            if (!ok) break;
            tcgen05_fence_after();
            // chunk c + 1 is on its way from TMEM while chunk c is folded (tcgen05.wait::ld covers every load issued so far)
            uint32_t r[2][16], lo[2][16];
            tmem_ld_32x16(lane_base + mb * kF3BN, r[0]);
            if (kb > 0) tmem_ld_32x16(low_base, lo[0]);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                tmem_ld_wait();
                if (c < 3) {
                    tmem_ld_32x16(lane_base + mb * kF3BN + (c + 1) * 16, r[(c + 1) & 1]);
                    if (kb > 0) tmem_ld_32x16(low_base + (c + 1) * 16, lo[(c + 1) & 1]);
                } else {                            // everything of this accumulator is in registers: the tensor core may refill it
                    tcgen05_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(mfree0 + 8u * mb);
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float e;
                    two_sum_f3(total[c * 16 + j], __uint_as_float(r[c & 1][j]), total[c * 16 + j], e);
                    lo[c & 1][j] = __float_as_uint(kb > 0 ? __fadd_rn(__uint_as_float(lo[c & 1][j]), e) : e);
                }
                tmem_st_32x16(low_base + c * 16, lo[c & 1]);
            }
            tmem_st_wait();
        }
        if (ok) ok = __all_sync(0xFFFFFFFFu, mbar_wait(cfull, 0u, abort_flag, args.wait_limit_ns));
        tcgen05_fence_after();
        // slot of element (row, col) of the tile in CTA 0's idle stage buffers: 8 bytes, rows fastest (a warp's lanes are rows)
        const uint32_t slot0 = (uint32_t)((half * 64) * 128 + quarter * 32 + lane) * 8u;
        if constexpr (kSplitK) {
            cluster_sync_all();                     // both CTAs' MMAs have completed: nothing reads CTA 0's stages any more
            if (krank == 1u && ok) {
                const uint32_t remote = map_to_cta(tiles, 0u);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[16], lo[16];
                    tmem_ld_32x16(lane_base + 2 * kF3BN + c * 16, r);
                    tmem_ld_32x16(low_base + c * 16, lo);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float l = __fadd_rn(__uint_as_float(lo[j]), __uint_as_float(r[j]));
                        asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};"
                                     ::"r"(remote + slot0 + (uint32_t)(c * 16 + j) * 1024u), "f"(total[c * 16 + j]), "f"(l) : "memory");
                    }
                }
            }
            cluster_sync_all();                     // CTA 1's pairs are in CTA 0's shared memory
        }
        if (ok && krank == 0u) {
            const int64_t row = (int64_t)m0 + quarter * 32 + lane;
            float *crow = args.C + (batch * args.M + (row < args.M ? row : 0)) * args.N;
            const bool vec_ok = (args.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(args.C) & 15u) == 0);
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t r[16], lo[16];
                tmem_ld_32x16(lane_base + 2 * kF3BN + c * 16, r);
                tmem_ld_32x16(low_base + c * 16, lo);
                tmem_ld_wait();
                const int64_t col0 = (int64_t)n0 + half * 64 + c * 16;
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    float t = total[c * 16 + j];
                    float l = __fadd_rn(__uint_as_float(lo[j]), __uint_as_float(r[j]));
                    if constexpr (kSplitK) {
                        const float2 other = *reinterpret_cast<const float2 *>(tiles_ptr + slot0 + (uint32_t)(c * 16 + j) * 1024u);
                        float e;
                        two_sum_f3(t, other.x, t, e);
                        l = __fadd_rn(__fadd_rn(l, other.y), e);
                    }
                    v[j] = (fabsf(t) == __int_as_float(0x7F800000)) ? t : __fadd_rn(t, l);
                }
                if (row < args.M) {
                    if (vec_ok && col0 + 16 <= args.N) {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            *reinterpret_cast<float4 *>(crow + col0 + 4 * q) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (col0 + j < args.N) crow[col0 + j] = v[j];
                    }
                }
            }
        }
    }

    tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0 && args.status) atomicExch(args.status, kStatusTimeout);
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 2000000ull) { }
        __syncthreads();
    }
    if (warp == 1) {
        __syncwarp();
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kF3TmemCols) : "memory");
    }
}

// ---- host side ----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// One operand as TMA sees it: inner dim (unit stride), outer dim (pitch), up to three batch dims.
struct OperandDesc {
    const void *base;
    int64_t inner_extent, outer_extent, outer_pitch;  // elements
    int64_t bext[kMaxBatchDims], bstride[kMaxBatchDims];
    int has[kMaxBatchDims];
    uint32_t box_inner, box_outer;
    int swizzle64 = 0;                                // 1: 64-byte swizzle (box_inner of 32 elements), else 128-byte
};

bool operand_ok(const OperandDesc &o) {
    if ((uintptr_t)o.base & 15u) return false;
    if (o.outer_extent > 1 && (o.outer_pitch <= 0 || (o.outer_pitch * 2) % 16)) return false;
    if (o.inner_extent >= (1ll << 32) || o.outer_extent >= (1ll << 32)) return false;
    if (o.outer_pitch * 2 >= (1ll << 40)) return false;
    for (int d = 0; d < kMaxBatchDims; ++d)
        if (o.has[d] && (o.bstride[d] <= 0 || (o.bstride[d] * 2) % 16 || o.bstride[d] * 2 >= (1ll << 40) || o.bext[d] >= (1ll << 32)))
            return false;
    return true;
}

int encode_uncached(const OperandDesc &o, int dtype, CUtensorMap *out);

// A tensor map depends only on the operand's address, extents, pitches and box, so the driver call that builds it
// (about a microsecond, two per matmul) is remembered per host thread: a decode loop or a layer that multiplies the same
// weights again finds its maps here. An entry can never be stale: equal key, equal encoding.
struct MapKey {
    const void *base;
    int64_t inner_extent, outer_extent, outer_pitch;
    int64_t bext[kMaxBatchDims], bstride[kMaxBatchDims];
    int32_t has[kMaxBatchDims];
    uint32_t box_inner, box_outer;
    int32_t dtype, swizzle64;
};
constexpr int kMapCacheSlots = 128;
struct MapCache {
    MapKey keys[kMapCacheSlots];
    CUtensorMap maps[kMapCacheSlots];
    uint64_t hash[kMapCacheSlots];
    bool used[kMapCacheSlots];
};
uint64_t hash_key(const MapKey &k) {
    uint64_t h = 1469598103934665603ull;
    const unsigned char *b = reinterpret_cast<const unsigned char *>(&k);
    for (size_t i = 0; i < sizeof(MapKey); ++i) { h ^= b[i]; h *= 1099511628211ull; }
    return h;
}
int encode(const OperandDesc &o, int dtype, CUtensorMap *out) {
    static thread_local MapCache *cache = nullptr;
    if (!cache) cache = new MapCache();   // zero-initialised; lives as long as the thread
    MapKey k;
    memset(&k, 0, sizeof(k));             // padding bytes take part in the hash
    k.base = o.base; k.inner_extent = o.inner_extent; k.outer_extent = o.outer_extent; k.outer_pitch = o.outer_pitch;
    for (int d = 0; d < kMaxBatchDims; ++d) { k.bext[d] = o.bext[d]; k.bstride[d] = o.has[d] ? o.bstride[d] : 0; k.has[d] = o.has[d]; }
    k.box_inner = o.box_inner; k.box_outer = o.box_outer; k.dtype = dtype; k.swizzle64 = o.swizzle64;
    const uint64_t h = hash_key(k);
    const int s0 = (int)(h % kMapCacheSlots), s1 = (int)((h >> 20) % kMapCacheSlots);   // two candidate slots per key
    for (int s : {s0, s1})
        if (cache->used[s] && cache->hash[s] == h && memcmp(&cache->keys[s], &k, sizeof(k)) == 0) { *out = cache->maps[s]; return MAGB200_OK; }
    int rc = encode_uncached(o, dtype, out);
    if (rc) return rc;
    const int s = cache->used[s0] ? s1 : s0;
    cache->keys[s] = k; cache->maps[s] = *out; cache->hash[s] = h; cache->used[s] = true;
    return MAGB200_OK;
}

int encode_uncached(const OperandDesc &o, int dtype, CUtensorMap *out) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return MAGB200_ERR_CUDA; }
    // fastest dim first: {inner, outer, b2, b1, b0}
    cuuint64_t dims[5] = {(cuuint64_t)o.inner_extent, (cuuint64_t)o.outer_extent, 1, 1, 1};
    cuuint64_t strides[4];
    // A dim of extent 1 still needs a legal stride (multiple of 16 bytes); use the packed size below it.
    uint64_t packed = (uint64_t)((o.inner_extent * 2 + 15) / 16 * 16);
    strides[0] = o.outer_extent > 1 ? (cuuint64_t)o.outer_pitch * 2 : packed;
    uint64_t prev = strides[0] * (uint64_t)o.outer_extent;
    for (int i = 0; i < kMaxBatchDims; ++i) {
        const int d = kMaxBatchDims - 1 - i;  // b2 is the fastest batch dim
        if (o.has[d]) { dims[2 + i] = (cuuint64_t)o.bext[d]; strides[1 + i] = (cuuint64_t)o.bstride[d] * 2; }
        else { dims[2 + i] = 1; strides[1 + i] = prev; }
        if (strides[1 + i] >= (1ull << 40)) strides[1 + i] = 16;  // extent-1 dim: the value is never used
        prev = strides[1 + i] * dims[2 + i];
    }
    cuuint32_t box[5] = {o.box_inner, o.box_outer, 1, 1, 1};
    cuuint32_t estr[5] = {1, 1, 1, 1, 1};
    CUresult r = fn(out, dtype == MAGB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 5,
                    const_cast<void *>(o.base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    o.swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with %d (dims %llu %llu %llu %llu %llu, strides %llu %llu %llu %llu, box %u %u)", (int)r,
                  (unsigned long long)dims[0], (unsigned long long)dims[1], (unsigned long long)dims[2], (unsigned long long)dims[3],
                  (unsigned long long)dims[4], (unsigned long long)strides[0], (unsigned long long)strides[1],
                  (unsigned long long)strides[2], (unsigned long long)strides[3], box[0], box[1]);
        return MAGB200_ERR_CUDA;
    }
    return MAGB200_OK;
}

// Layout of one operand for the tensor-core path, or false when TMA cannot describe it.
bool describe(const GemmProblem &p, bool is_a, int BN, OperandDesc &o, int &mn_major) {
    const int64_t s_mn = is_a ? p.sAm : p.sBn, s_k = is_a ? p.sAk : p.sBk;
    const int64_t e_mn = is_a ? p.M : p.N;
    o.base = is_a ? p.A : p.B;
    if (s_k == 1 || p.K == 1) {            // K-major (with K == 1 the K stride is never stepped)
        mn_major = 0;
        o.inner_extent = p.K; o.outer_extent = e_mn; o.outer_pitch = s_mn;
        o.box_inner = BK; o.box_outer = is_a ? BM : BN;
    } else if (s_mn == 1 || e_mn == 1) {   // MN-major
        mn_major = 1;
        o.inner_extent = e_mn; o.outer_extent = p.K; o.outer_pitch = s_k;
        o.box_inner = 64; o.box_outer = BK;
    } else {
        return false;
    }
    for (int d = 0; d < kMaxBatchDims; ++d) {
        const int64_t st = d < p.nbatch ? (is_a ? p.bsA[d] : p.bsB[d]) : 0;
        const int64_t ex = d < p.nbatch ? p.bshape[d] : 1;
        o.has[d] = (ex > 1 && st != 0) ? 1 : 0;
        o.bext[d] = o.has[d] ? ex : 1;
        o.bstride[d] = st;
    }
    return operand_ok(o);
}

int pick_bn(const GemmProblem &p) {
    // Estimated time = waves x cost of one tile. A 128x256 tile is the efficient one (the narrower tiles read as many
    // bytes of A per MMA but produce half / a quarter of the output, so they run into shared-memory and L2 bandwidth);
    // narrower tiles only win when they save whole waves on a small output.
    const int64_t tm = (p.M + BM - 1) / BM;
    int best = 256;
    double best_cost = 1e300;
    const int cand[3] = {256, 128, 64};
    const double tile_cost[3] = {1.0, 0.62, 0.40};
    for (int i = 0; i < 3; ++i) {
        const int bn = cand[i];
        if (bn > 64 && p.N <= bn / 2) continue;  // more than half of the tile would be padding
        const int64_t tiles = tm * ((p.N + bn - 1) / bn) * p.batch_total;
        const double waves = (double)((tiles + num_sms() - 1) / num_sms());
        const double cost = waves * tile_cost[i];
        if (cost < best_cost - 1e-9) { best_cost = cost; best = bn; }
    }
    return best;
}

// Set by launch_gemm_tcgen05 / _2sm for the launch they are about to make: launch as a programmatic dependent of the kernel
// before it on the stream (no wait inside: the caller has checked that the two are independent).
thread_local bool t_launch_overlapped = false;
inline void add_overlap_attr(cudaLaunchAttribute *attr, unsigned &n) {
    if (!t_launch_overlapped) return;
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
}

// ---- run-time knobs (set through the C ABI) ---------------------------------------------------------------------------
std::atomic<uint64_t> g_wait_limit_ns{1000ull * 1000ull * 1000ull};
std::atomic<int> g_skip_kb_once{-1};      // consumed by the next tensor-core launch
std::atomic<int> g_balance_tail{1};       // sharing of a partial last wave along K: 0 off, 1 when it pays, 2 whenever possible
std::atomic<int> g_split_small{1};        // one-CTA kernel: CTA pairs split K when the output has few tiles (0: never)

// cudaFuncSetAttribute applies to the current device only, so the opt-in to more than 48 KB of dynamic shared memory is
// remembered per (kernel, device): bit d of `done` is set once device d has it.
template <typename K>
int ensure_smem_optin(K kernel, size_t bytes, std::atomic<uint32_t> &done) {
    int dev = 0;
    MAGB200_CUDA_TRY(cudaGetDevice(&dev));
    const uint32_t bit = 1u << (dev & 31);
    if (!(done.load(std::memory_order_acquire) & bit)) {
        MAGB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        done.fetch_or(bit, std::memory_order_release);
    }
    return MAGB200_OK;
}

void fill_knobs(TcArgs &args) {
    args.wait_limit_ns = g_wait_limit_ns.load();
    args.skip_kb = g_skip_kb_once.exchange(-1);
}

// Few tiles and a long K: clusters of two CTAs split K (128 x 128 tiles only)
template <int DT>
int launch_cfg_split2(const GemmProblem &p, const CUtensorMap &ta, const CUtensorMap &tb, TcArgs &args, cudaStream_t st) {
    using C = Cfg<128>;
    auto kernel = gemm_tcgen05_kernel<128, DT, true>;
    static std::atomic<uint32_t> optin{0};
    if (int rc = ensure_smem_optin(kernel, C::kSmemBytes, optin)) return rc;
    fill_knobs(args);
    args.skip_kb = -1;                                   // the unarmed-stage hook belongs to the persistent kernels
    args.tiles_m = (p.M + BM - 1) / BM;
    args.tiles_n = (p.N + 127) / 128;
    args.total_tiles = args.tiles_m * args.tiles_n * p.batch_total;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)(2 * args.total_tiles), 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    add_overlap_attr(attr, cfg.numAttrs);
    MAGB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, ta, tb, args));
    count_launch();
    return MAGB200_OK;
}

template <int BN, int DT>
int launch_cfg(const GemmProblem &p, const CUtensorMap &ta, const CUtensorMap &tb, TcArgs &args, cudaStream_t st, int cta_limit) {
    using C = Cfg<BN>;
    auto kernel = gemm_tcgen05_kernel<BN, DT>;
    static std::atomic<uint32_t> optin{0};  // per template instantiation
    if (int rc = ensure_smem_optin(kernel, C::kSmemBytes, optin)) return rc;
    fill_knobs(args);
    args.tiles_m = (p.M + BM - 1) / BM;
    args.tiles_n = (p.N + BN - 1) / BN;
    args.total_tiles = args.tiles_m * args.tiles_n * p.batch_total;
    const int64_t max_ctas = cta_limit > 0 ? cta_limit : num_sms();
    const unsigned grid = (unsigned)(args.total_tiles < max_ctas ? args.total_tiles : max_ctas);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    add_overlap_attr(attr, cfg.numAttrs);
    MAGB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, ta, tb, args));
    count_launch();
    return MAGB200_OK;
}


// Host mirror of tail_pair_of (device): pair whose run holds K group `kg_index` of the tail.
int host_tail_pair_of(int64_t kg_index, int64_t R, int64_t Q) { return (int)(((kg_index + 1) * Q + R - 1) / R - 1); }

// Decide how the tiles of a partial last wave are shared out (see WorkUnit). Fills full_tiles, tail_*, num_kg, sk_*.
void plan_tail(TcArgs &args, int64_t pairs, const SplitWorkspace *ws, int ksub) {
    const int64_t T = args.total_tiles;
    args.num_kg = (args.num_kb + ksub - 1) / ksub;
    const int64_t r = T % pairs;
    args.full_tiles = T - r;
    args.tail_tiles = (int)r;
    args.tail_pairs = (int)r;            // default: one pair per left-over tile, the others idle
    args.tail_slots = 0;
    args.sk_partial = nullptr; args.sk_counters = nullptr;
    if (r == 0) { args.tail_pairs = 0; return; }
    const bool vec_ok = (args.N % 8 == 0) && (((uintptr_t)args.C & 15u) == 0);
    if (!g_balance_tail.load() || !ws || !ws->partial || !ws->counters || !vec_ok || r > ws->max_tiles) return;
    // Sharing costs a round trip of fp32 tiles through L2 and a serial sum in the owner (measured: about 8 us at 2-3 runs per
    // tile), and under the board's power limit an idle pair is not a total loss (the busy ones clock higher). It pays when
    // most pairs would idle and a tile is long: 2560 x 2048 x 8192 (6 of 80 tiles left over) +9 %, 4096^2 x 8192 +1 %,
    // 4096^2 x 2048 -14 % with sharing forced. So: at most a quarter of the pairs busy without it, K >= 4096, at most four
    // runs per tile (or whenever `force` asks for it, which the tests use to reach every path).
    const bool force = g_balance_tail.load() == 2;
    int cap = args.num_kg / 4;
    if (cap > (force ? 8 : 4)) cap = force ? 8 : 4;
    if (cap < 2) return;
    if (!force && (r * 4 > pairs || args.num_kg < 32)) return;
    int64_t Q = r * cap < pairs ? r * cap : pairs;
    if (Q <= r) return;
    const int64_t R = r * args.num_kg;
    int max_parts = 1;
    for (int64_t t = 0; t < r; ++t) {
        const int parts = host_tail_pair_of((t + 1) * args.num_kg - 1, R, Q) - host_tail_pair_of(t * args.num_kg, R, Q) + 1;
        if (parts > max_parts) max_parts = parts;
    }
    const size_t need = (size_t)r * (size_t)(max_parts - 1) * (size_t)(2 * BM * BN2) * sizeof(float);
    if (max_parts < 2 || need > ws->partial_bytes) return;
    args.tail_pairs = (int)Q;
    args.tail_slots = max_parts - 1;
    args.sk_partial = ws->partial;
    args.sk_counters = ws->counters;
}

template <int DT, int KSUB, bool kShare, bool kTmaStore, bool kSwiGLU = false>
int launch_2sm_kernel(const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap &tb2, const CUtensorMap &tc, const TcArgs &args,
                      const cudaLaunchConfig_t &cfg) {
    auto kernel = gemm_tcgen05_2sm_kernel<DT, KSUB, kShare, kTmaStore, kSwiGLU>;
    static std::atomic<uint32_t> optin{0};
    if (int rc = ensure_smem_optin(kernel, Cfg2<KSUB>::kSmemBytes, optin)) return rc;
    MAGB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, ta, tb, tb2, tc, args));
    return MAGB200_OK;
}

// `tc`: tensor map of the result for the bulk-store epilogue, or null when the result cannot leave that way
// `tb_up`: tensor map of the up-projection weights for the gated form (then `tc` is required), else null
template <int DT, int KSUB>
int launch_2sm(const GemmProblem &p, const CUtensorMap &ta, const CUtensorMap &tb, const CUtensorMap *tc, TcArgs &args, cudaStream_t st,
               int cta_limit, const SplitWorkspace *ws, const CUtensorMap *tb_up = nullptr) {
    fill_knobs(args);
    args.tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
    args.tiles_n = tb_up ? (p.N + BN2 / 2 - 1) / (BN2 / 2) : (p.N + BN2 - 1) / BN2;
    args.total_tiles = args.tiles_m * args.tiles_n * p.batch_total;
    const int64_t max_pairs = (cta_limit > 1 ? cta_limit : num_sms()) / 2;
    const unsigned pairs = (unsigned)(args.total_tiles < max_pairs ? args.total_tiles : max_pairs);
    plan_tail(args, pairs, tb_up ? nullptr : ws, KSUB);     // the gated form never shares a tile along K
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(kThreads2, 1, 1);
    cfg.dynamicSmemBytes = Cfg2<KSUB>::kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    add_overlap_attr(attr, cfg.numAttrs);
    int rc;
    if (tb_up) rc = launch_2sm_kernel<DT, KSUB, false, true, true>(ta, tb, *tb_up, *tc, args, cfg);
    else if (args.tail_slots > 0) rc = launch_2sm_kernel<DT, KSUB, true, false>(ta, tb, tb, ta, args, cfg);
    else if (tc) rc = launch_2sm_kernel<DT, KSUB, false, true>(ta, tb, tb, *tc, args, cfg);
    else rc = launch_2sm_kernel<DT, KSUB, false, false>(ta, tb, tb, ta, args, cfg);
    if (rc) return rc;
    count_launch();
    return MAGB200_OK;
}

}  // namespace

void set_wait_limit_ns(uint64_t ns) { g_wait_limit_ns.store(ns); }
uint64_t get_wait_limit_ns() { return g_wait_limit_ns.load(); }
void set_skip_kb_once(int kb) { g_skip_kb_once.store(kb); }
void set_balance_tail(int mode) { g_balance_tail.store(mode); }   // 0: off, 1: when it pays, 2: whenever possible
void set_split_small(int on) { g_split_small.store(on ? 1 : 0); }

bool tcgen05_supported(const GemmProblem &p) {
    if (p.dtype != MAGB200_BF16 && p.dtype != MAGB200_F16) return false;
    if (p.M < 1 || p.N < 1 || p.K < 1) return false;
    if (p.M >= (1ll << 31) || p.N >= (1ll << 31) || p.K >= (1ll << 31)) return false;
    OperandDesc a, b;
    int amn, bmn;
    return describe(p, true, 128, a, amn) && describe(p, false, 128, b, bmn);
}


bool tcgen05_operand_ok(const GemmProblem &p, bool is_a) {
    OperandDesc o;
    int mn;
    return describe(p, is_a, 128, o, mn);
}

// The two-SM kernel pays when the output has at least one full wave of 256 x 256 tiles for the 74 CTA pairs; smaller
// problems keep the one-CTA kernel with its narrower tiles (measured: 4096 x 1024 x 4096, 64 tiles, is 12 % faster there).
bool tcgen05_2sm_supported(const GemmProblem &p) {
    if (!tcgen05_supported(p)) return false;
    if (p.M < 256 || p.N < 256) return false;
    return true;
}
bool tcgen05_2sm_preferred(const GemmProblem &p) {
    if (!tcgen05_2sm_supported(p)) return false;
    const int64_t tiles = ((p.M + 255) / 256) * ((p.N + 255) / 256) * p.batch_total;
    return tiles >= num_sms() / 2;
}

int launch_gemm_tcgen05_2sm(const GemmProblem &p, cudaStream_t st, int cta_limit, int *status_word_dev, const ScatterTarget *scatter,
                            const SplitWorkspace *ws, bool overlapped) {
    struct Scope { Scope(bool v) { t_launch_overlapped = v; } ~Scope() { t_launch_overlapped = false; } } scope(overlapped && !scatter);
    if (overlapped) ws = nullptr;             // the shared last wave uses a workspace that the kernel before this one may be using
    OperandDesc a, b;
    int amn = 0, bmn = 0;
    if (!describe(p, true, 128, a, amn) || !describe(p, false, 128, b, bmn)) {
        set_error("tcgen05 matmul: operand layout cannot be described by a TMA tensor map");
        return MAGB200_ERR_INVALID_ARG;
    }
    CUtensorMap ta, tb;
    int rc;
    if ((rc = encode(a, p.dtype, &ta)) || (rc = encode(b, p.dtype, &tb))) return rc;
    TcArgs args;
    memset(&args, 0, sizeof(args));
    args.C = p.C; args.M = p.M; args.N = p.N; args.K = p.K; args.dtype = p.dtype;
    args.a_mn = amn; args.b_mn = bmn; args.nbatch = p.nbatch;
    for (int d = 0; d < kMaxBatchDims; ++d) {
        args.bshape[d] = d < p.nbatch ? p.bshape[d] : 1;
        args.a_has[d] = a.has[d]; args.b_has[d] = b.has[d];
    }
    args.num_kb = (int)((p.K + BK - 1) / BK);
    args.status = status_word_dev;
    if (scatter) {
        args.scatter_ranks = scatter->ranks; args.scatter_rank = scatter->rank; args.rows_per_rank = scatter->rows_per_rank;
        for (int i = 0; i < scatter->ranks; ++i) args.peer_stage[i] = scatter->stage[i];
    }
    // the result as TMA sees it: [batch][M][N] contiguous -> boxes of 32 columns x 32 rows (64-byte swizzle) for the epilogue's bulk stores
    CUtensorMap tcm;
    const CUtensorMap *tc = nullptr;
    if (!scatter && p.N % 8 == 0) {
        OperandDesc c;
        memset(&c, 0, sizeof(c));
        c.base = p.C; c.inner_extent = p.N; c.outer_extent = p.M; c.outer_pitch = p.N;
        c.box_inner = 32; c.box_outer = 32; c.swizzle64 = 1;
        for (int d = 0; d < kMaxBatchDims; ++d) { c.bext[d] = 1; c.bstride[d] = 0; c.has[d] = 0; }
        if (p.batch_total > 1) { c.bext[kMaxBatchDims - 1] = p.batch_total; c.bstride[kMaxBatchDims - 1] = p.M * p.N; c.has[kMaxBatchDims - 1] = 1; }
        if (operand_ok(c) && encode(c, p.dtype, &tcm) == MAGB200_OK) tc = &tcm;
    }
    return p.dtype == MAGB200_BF16 ? launch_2sm<MAGB200_BF16, 2>(p, ta, tb, tc, args, st, cta_limit, ws)
                                   : launch_2sm<MAGB200_F16, 2>(p, ta, tb, tc, args, st, cta_limit, ws);
}

// ---- gated MLP: out = silu(x @ Wg) * (x @ Wu) in one launch -----------------------------------------------------------------
namespace {
// the result [batch][M][N] as boxes of 32 columns x 32 rows (64-byte swizzle) for the epilogue's bulk stores
bool describe_result(const GemmProblem &p, OperandDesc &c) {
    if (p.N % 8) return false;
    memset(&c, 0, sizeof(c));
    c.base = p.C; c.inner_extent = p.N; c.outer_extent = p.M; c.outer_pitch = p.N;
    c.box_inner = 32; c.box_outer = 32; c.swizzle64 = 1;
    for (int d = 0; d < kMaxBatchDims; ++d) { c.bext[d] = 1; c.bstride[d] = 0; c.has[d] = 0; }
    if (p.batch_total > 1) { c.bext[kMaxBatchDims - 1] = p.batch_total; c.bstride[kMaxBatchDims - 1] = p.M * p.N; c.has[kMaxBatchDims - 1] = 1; }
    return operand_ok(c);
}
}  // namespace

bool swiglu_fused_supported(const GemmProblem &p, const void *b_up) {
    if (!tcgen05_supported(p) || p.M < 256 || p.N < 128) return false;
    GemmProblem q = p;
    q.B = b_up;
    OperandDesc o;
    int mn;
    if (!describe(q, false, 128, o, mn)) return false;
    return describe_result(p, o) && ((uintptr_t)p.C & 15u) == 0;
}

int launch_gemm_swiglu(const GemmProblem &p, const void *b_up, cudaStream_t st, int cta_limit, int *status_word_dev) {
    GemmProblem q = p;
    q.B = b_up;
    OperandDesc a, b, b2, c;
    int amn = 0, bmn = 0, b2mn = 0;
    if (!describe(p, true, 128, a, amn) || !describe(p, false, 128, b, bmn) || !describe(q, false, 128, b2, b2mn) || bmn != b2mn ||
        !describe_result(p, c)) {
        set_error("gated matmul: operand layout cannot be described by TMA tensor maps");
        return MAGB200_ERR_INVALID_ARG;
    }
    CUtensorMap ta, tb, tb2, tc;
    int rc;
    if ((rc = encode(a, p.dtype, &ta)) || (rc = encode(b, p.dtype, &tb)) || (rc = encode(b2, p.dtype, &tb2)) || (rc = encode(c, p.dtype, &tc))) return rc;
    TcArgs args;
    memset(&args, 0, sizeof(args));
    args.C = p.C; args.M = p.M; args.N = p.N; args.K = p.K; args.dtype = p.dtype;
    args.a_mn = amn; args.b_mn = bmn; args.nbatch = p.nbatch;
    for (int d = 0; d < kMaxBatchDims; ++d) {
        args.bshape[d] = d < p.nbatch ? p.bshape[d] : 1;
        args.a_has[d] = a.has[d]; args.b_has[d] = b.has[d];
    }
    args.num_kb = (int)((p.K + BK - 1) / BK);
    args.status = status_word_dev;
    return p.dtype == MAGB200_BF16 ? launch_2sm<MAGB200_BF16, 2>(p, ta, tb, &tc, args, st, cta_limit, nullptr, &tb2)
                                   : launch_2sm<MAGB200_F16, 2>(p, ta, tb, &tc, args, st, cta_limit, nullptr, &tb2);
}

int launch_gemm_tcgen05(const GemmProblem &p, cudaStream_t st, int cta_limit, int *status_word_dev, const ScatterTarget *scatter,
                        bool overlapped) {
    struct Scope { Scope(bool v) { t_launch_overlapped = v; } ~Scope() { t_launch_overlapped = false; } } scope(overlapped && !scatter);
    // an output of at most 74 tiles of 128 x 128 with K >= 1024: pairs of CTAs split K, twice as many SMs work
    const int64_t tiles128 = ((p.M + BM - 1) / BM) * ((p.N + 127) / 128) * p.batch_total;
    const bool split2 = !scatter && cta_limit <= 0 && p.N > 64 && tiles128 * 2 <= num_sms() && p.K >= 1024 && g_split_small.load() && g_skip_kb_once.load() < 0;
    const int bn = split2 ? 128 : pick_bn(p);
    OperandDesc a, b;
    int amn = 0, bmn = 0;
    if (!describe(p, true, bn, a, amn) || !describe(p, false, bn, b, bmn)) {
        set_error("tcgen05 matmul: operand layout cannot be described by a TMA tensor map");
        return MAGB200_ERR_INVALID_ARG;
    }
    CUtensorMap ta, tb;
    int rc;
    if ((rc = encode(a, p.dtype, &ta)) || (rc = encode(b, p.dtype, &tb))) return rc;
    TcArgs args;
    memset(&args, 0, sizeof(args));
    args.C = p.C; args.M = p.M; args.N = p.N; args.K = p.K; args.dtype = p.dtype;
    args.a_mn = amn; args.b_mn = bmn; args.nbatch = p.nbatch;
    for (int d = 0; d < kMaxBatchDims; ++d) {
        args.bshape[d] = d < p.nbatch ? p.bshape[d] : 1;
        args.a_has[d] = a.has[d]; args.b_has[d] = b.has[d];
    }
    args.num_kb = (int)((p.K + BK - 1) / BK);
    args.status = status_word_dev;
    if (scatter) {
        args.scatter_ranks = scatter->ranks; args.scatter_rank = scatter->rank; args.rows_per_rank = scatter->rows_per_rank;
        for (int i = 0; i < scatter->ranks; ++i) args.peer_stage[i] = scatter->stage[i];
    }
    if (split2)
        return p.dtype == MAGB200_BF16 ? launch_cfg_split2<MAGB200_BF16>(p, ta, tb, args, st) : launch_cfg_split2<MAGB200_F16>(p, ta, tb, args, st);
#define LAUNCH(BNV)                                                                                   \
    return p.dtype == MAGB200_BF16 ? launch_cfg<BNV, MAGB200_BF16>(p, ta, tb, args, st, cta_limit)                \
                                   : launch_cfg<BNV, MAGB200_F16>(p, ta, tb, args, st, cta_limit)
    if (bn == 256) { LAUNCH(256); }
    if (bn == 128) { LAUNCH(128); }
    LAUNCH(64);
#undef LAUNCH
}

// ---- float32 through split operands ---------------------------------------------------------------------------------
namespace {
bool describe_planes(const GemmProblem &p, bool is_a, const void *planes, OperandDesc &o) {
    const PlaneLayout l = plane_layout(p, is_a);
    o.base = planes;
    o.inner_extent = p.K; o.outer_extent = 3 * l.rows; o.outer_pitch = l.kpad;
    o.box_inner = BK; o.box_outer = BM;
    for (int d = 0; d < kMaxBatchDims; ++d) {
        o.has[d] = (d < p.nbatch && l.bstride[d] != 0) ? 1 : 0;
        o.bext[d] = o.has[d] ? p.bshape[d] : 1;
        o.bstride[d] = l.bstride[d];
    }
    return operand_ok(o);
}
}  // namespace

bool f32x3_supported(const GemmProblem &p) {
    if (p.dtype != MAGB200_F32) return false;
    if (p.M < 1 || p.N < 1 || p.K < 1) return false;
    if (3 * p.M >= (1ll << 31) || 3 * p.N >= (1ll << 31) || p.K >= (1ll << 31)) return false;
    const int64_t tiles = ((p.M + BM - 1) / BM) * ((p.N + kF3BN - 1) / kF3BN) * p.batch_total;
    if (tiles >= (1ll << 31)) return false;
    for (int d = 0; d < p.nbatch; ++d)
        if (p.bshape[d] >= (1ll << 31)) return false;
    OperandDesc a, b;
    return describe_planes(p, true, nullptr, a) && describe_planes(p, false, nullptr, b);
}

int launch_gemm_f32x3(const GemmProblem &p, const void *planes_a, const void *planes_b, const int *skip_if_set, int *status_word_dev,
                      cudaStream_t st) {
    OperandDesc a, b;
    if (!describe_planes(p, true, planes_a, a) || !describe_planes(p, false, planes_b, b)) {
        set_error("matmul: the split-operand planes cannot be described to TMA");
        return MAGB200_ERR_INVALID_ARG;
    }
    CUtensorMap ta, tb;
    int rc;
    if ((rc = encode(a, MAGB200_BF16, &ta)) || (rc = encode(b, MAGB200_BF16, &tb))) return rc;
    F3Args args;
    memset(&args, 0, sizeof(args));
    args.C = reinterpret_cast<float *>(p.C);
    args.M = p.M; args.N = p.N; args.K = p.K;
    args.nbatch = p.nbatch;
    for (int d = 0; d < kMaxBatchDims; ++d) {
        args.bshape[d] = d < p.nbatch ? p.bshape[d] : 1;
        args.a_has[d] = a.has[d];
        args.b_has[d] = b.has[d];
    }
    args.tiles_m = (p.M + BM - 1) / BM;
    args.tiles_n = (p.N + kF3BN - 1) / kF3BN;
    args.num_kb = (int)((p.K + BK - 1) / BK);
    args.status = status_word_dev;
    args.skip_if_set = skip_if_set;
    args.wait_limit_ns = g_wait_limit_ns.load();
    const int64_t tiles = args.tiles_m * args.tiles_n * p.batch_total;
    // a programmatic dependent of the split pass: its set-up (barriers, TMEM, tensor maps) runs beside that pass's tail
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.blockDim = dim3(kF3Threads, 1, 1);
    cfg.dynamicSmemBytes = kF3SmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    if (tiles * 2 <= num_sms() && args.num_kb >= 8) {      // few tiles, long K: pairs of CTAs share a tile along K
        static std::atomic<uint32_t> optin_split{0};
        if ((rc = ensure_smem_optin(gemm_f32x3_kernel<true>, kF3SmemBytes, optin_split))) return rc;
        cfg.gridDim = dim3((unsigned)(2 * tiles), 1, 1);
        cfg.numAttrs = 2;
        MAGB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_f32x3_kernel<true>, ta, tb, args));
        count_launch();
        return MAGB200_OK;
    }
    static std::atomic<uint32_t> optin{0};
    if ((rc = ensure_smem_optin(gemm_f32x3_kernel<false>, kF3SmemBytes, optin))) return rc;
    cfg.gridDim = dim3((unsigned)tiles, 1, 1);
    cfg.numAttrs = 1;
    MAGB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_f32x3_kernel<false>, ta, tb, args));
    count_launch();
    MAGB200_CUDA_TRY(cudaGetLastError());
    return MAGB200_OK;
}

}  // namespace magb200
