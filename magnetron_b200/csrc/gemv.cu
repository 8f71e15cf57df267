// Decode-shaped products (M <= 8): weight-streaming kernels bound by HBM bandwidth.
//
// C[M,N] = A[M,K] . B[K,N] with a handful of activation rows and a large weight matrix B. Every
// weight element is read from HBM exactly once with 128-bit loads that bypass L1; the activations
// are staged once per CTA in shared memory; accumulation is fp32 over the whole K with one rounding.
//
//  * skinny_km_mma (bf16 / fp16): B is K-major (the `W.T` view of a row-major [N,K] nn.Linear weight:
//    sBk == 1). A warp owns 16 consecutive weight rows and feeds them, straight from its 128-bit global
//    loads, into mma.sync.m16n8k16 as the A operand; the (up to 8) activation rows are the 8 columns of
//    the B operand. Because a dot product does not care in which order K is visited, the 8 consecutive K
//    values that one 128-bit load brings are assigned to the instruction's K slots by a fixed permutation
//    that A and B share, so no shuffle or shared-memory transpose of the weights is needed. The FP32 pipe
//    is then idle: M = 8 costs the same as M = 1 and the kernel stays HBM bound across the batch sweep.
//  * skinny_km (float32, and layouts the MMA variant cannot take): one warp owns R consecutive weight
//    rows; its 32 lanes stride along K in 16-byte vectors, FFMA, warp-shuffle reduction.
//  * skinny_nm: B is N-major (contiguous [K,N], the layout the reference's own GEMV path needs,
//    magnetron/cpu/mag_cpu_impl_ops_matmul.inl:2940). One thread owns 16 bytes of consecutive
//    columns, the 8 warps of a CTA split the CTA's K range, partial sums meet in shared memory.
//
// When K is too long for the activation tile to fit in shared memory, or N is too small to occupy
// 148 SMs, K is split across CTAs (grid.y): each split writes fp32 partials to a scratch buffer
// [split][batch][M][N] and a second tiny kernel sums the splits in a fixed order and rounds once,
// so results do not depend on scheduling.
#include "common.cuh"

#include <atomic>

namespace magb200 {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;

template <int DT> struct Elem { static constexpr int size = 2; static constexpr int vec = 8; using bits = uint16_t; };
template <> struct Elem<MAGB200_F32> { static constexpr int size = 4; static constexpr int vec = 4; using bits = uint32_t; };

constexpr int kMaxGroups = 4;
struct SkinnyArgs {
    const void *A, *B;
    void *C;            // result [batch][M][N] in the operand dtype (used when nsplit == 1)
    float *partial;     // fp32 scratch [nsplit][batch][M][N] (used when nsplit > 1)
    int64_t N, K;
    int64_t sAm, sAk;   // activation strides (elements)
    int64_t ldb;        // pitch of B's slow dim (elements): sBn for K-major, sBk for N-major
    int64_t kch;        // K elements per split (multiple of the vector width)
    int nsplit;
    int nbatch;
    int64_t bshape[kMaxBatchDims], bsA[kMaxBatchDims], bsB[kMaxBatchDims];
    int64_t batch_total;
    int early_weights;  // 1: the weights were not written by a kernel that may still be running; they may be fetched before pdl_wait()
    // grouped launch (skinny_km_mma_kernel only): several weight matrices against the same activation rows, e.g. the q, k and
    // v projections of a decode step. Group i owns the 16-row tiles [gtile0[i], gtile0[i+1]) of the launch.
    int ngroups;        // 0: a single problem described by B, C, N, ldb above
    const void *gB[kMaxGroups];
    void *gC[kMaxGroups];
    int64_t gN[kMaxGroups], gldb[kMaxGroups];
    int64_t gtile0[kMaxGroups + 1];
};

// Programmatic dependent launch: a kernel launched with the programmatic-serialization attribute may start while its
// predecessor in the stream is still running. Everything that does not depend on the predecessor's output (index set-up,
// the first weight loads) runs before pdl_wait(); the activations are read only after it. pdl_launch_dependents() lets
// the successor start its own independent part early. Decode is a chain of microsecond kernels, so this hides most of
// the launch latency between them. Because every kernel here lets its successor start at once, a kernel can be running
// while kernels several launches back have not finished: weights are fetched ahead of pdl_wait() only when the host has
// established that none of those kernels writes them (SkinnyArgs::early_weights); a weight operand that is itself a fresh
// result -- K in q @ K^T right after the k projection -- is read after the wait like the activations.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
int launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, int cluster, Args &&...args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cluster > 1) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = (unsigned)cluster; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    MAGB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
    return MAGB200_OK;
}
template <typename... KArgs, typename... Args>
int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args &&...args) {
    return launch_pdl_cluster(kernel, grid, block, smem, st, 1, static_cast<Args &&>(args)...);
}

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}

__device__ __forceinline__ uint4 ldg_stream(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// 16 bytes of storage -> fp32 lanes
template <int DT> __device__ __forceinline__ void unpack(const uint4 &v, float (&f)[Elem<DT>::vec]) {
    if constexpr (DT == MAGB200_F32) {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    } else if constexpr (DT == MAGB200_BF16) {
        f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xFFFF0000u);
        f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xFFFF0000u);
        f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xFFFF0000u);
        f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xFFFF0000u);
    } else {
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
    }
}

__device__ __forceinline__ void batch_offsets(const SkinnyArgs &a, int64_t batch, int64_t &offA, int64_t &offB) {
    offA = 0; offB = 0;
    int64_t rem = batch;
    for (int d = a.nbatch - 1; d >= 0; --d) {
        int64_t q = rem / a.bshape[d];
        int64_t idx = rem - q * a.bshape[d];
        offA += idx * a.bsA[d];
        offB += idx * a.bsB[d];
        rem = q;
    }
}

template <int DT> __device__ __forceinline__ void store_result(const SkinnyArgs &a, int64_t batch, int split, int m, int M,
                                                               int64_t n, float v) {
    if (a.nsplit == 1) store_from_f32<DT>(a.C, (batch * M + m) * a.N + n, v);
    else a.partial[(((int64_t)split * a.batch_total + batch) * M + m) * a.N + n] = v;
}

// ------------------------------------------------------------------------------------------------
// K-major weights: grid = (row blocks, nsplit, batch)
// ------------------------------------------------------------------------------------------------
template <int DT, int M, int R>
__global__ void __launch_bounds__(kThreads) skinny_km_kernel(const SkinnyArgs a) {
    using E = Elem<DT>;
    constexpr int V = E::vec;
    extern __shared__ __align__(16) unsigned char smem[];
    typename E::bits *xs = reinterpret_cast<typename E::bits *>(smem);  // [M][kch]

    const int split = blockIdx.y;
    const int64_t batch = blockIdx.z;
    const int64_t k0 = (int64_t)split * a.kch;
    const int64_t kc = min(a.kch, a.K - k0);
    int64_t offA, offB;
    batch_offsets(a, batch, offA, offB);

    // stage the activation chunk (raw bits, any strides)
    {
        const typename E::bits *A = reinterpret_cast<const typename E::bits *>(a.A) + offA;
        for (int m = 0; m < M; ++m)
            for (int64_t k = threadIdx.x; k < kc; k += kThreads) xs[m * a.kch + k] = A[m * a.sAm + (k0 + k) * a.sAk];
    }
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t kvecs = kc / V;
    const int64_t kchv = a.kch / V;
    const uint4 *xv = reinterpret_cast<const uint4 *>(xs);
    const typename E::bits *Bbase = reinterpret_cast<const typename E::bits *>(a.B) + offB + k0;

    for (int64_t row0 = ((int64_t)blockIdx.x * kWarps + warp) * R; row0 < a.N; row0 += (int64_t)gridDim.x * kWarps * R) {
        float acc[R][M];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) acc[r][m] = 0.f;
        const uint4 *wrow[R];
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int64_t row = min(row0 + r, a.N - 1);  // clamp: tail rows are computed twice, stored once
            wrow[r] = reinterpret_cast<const uint4 *>(Bbase + row * a.ldb);
        }
#pragma unroll 2
        for (int64_t kv = lane; kv < kvecs; kv += 32) {
            uint4 w[R];
#pragma unroll
            for (int r = 0; r < R; ++r) w[r] = ldg_stream(wrow[r] + kv);
            float wf[R][V];
#pragma unroll
            for (int r = 0; r < R; ++r) unpack<DT>(w[r], wf[r]);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float xf[V];
                unpack<DT>(xv[m * kchv + kv], xf);
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int j = 0; j < V; ++j) acc[r][m] = fmaf(wf[r][j], xf[j], acc[r][m]);
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float v = acc[r][m];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
                acc[r][m] = v;
            }
        // lane (r*M + m) stores one value, so the R*M results leave the warp in one pass
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M; ++m)
                if (lane == ((r * M + m) & 31) && row0 + r < a.N) store_result<DT>(a, batch, split, m, M, row0 + r, acc[r][m]);
    }
}

// ------------------------------------------------------------------------------------------------
// K-major 16-bit weights on mma.sync: grid = (row-tile groups, nsplit, batch)
// ------------------------------------------------------------------------------------------------
template <int DT> __device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                            uint32_t b0, uint32_t b1) {
    if constexpr (DT == MAGB200_BF16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
}

// Stage the (up to 8) activation rows of this CTA's K range in shared memory. All rows are copied in one flattened loop
// whose loads are issued four at a time before their stores: a row-by-row loop pays one L2 round trip per row, which made a
// small projection take 8.3 us at M = 8 against 5.6 us at M = 1 for the same weight bytes.
__device__ __forceinline__ void stage_activations(const SkinnyArgs &a, int M, int xstride, int64_t offA, int64_t k0, int kc, uint16_t *xs) {
    const uint16_t *A = reinterpret_cast<const uint16_t *>(a.A) + offA + k0 * a.sAk;
    const bool vec = a.sAk == 1 && ((reinterpret_cast<uintptr_t>(A) & 15u) == 0) && (M == 1 || a.sAm % 8 == 0);
    if (vec) {
        // asynchronous 16-byte copies, all in flight at once (eight rows of K = 4096 are 16 copies per thread: through registers,
        // four at a time, that was four L2 round trips on the critical path of every CTA), then one wait; the wait also covers
        // the weight copies a streaming kernel has issued before, which it needs next anyway
        const int chunks = kc >> 3;                 // whole groups of 8 K values (callers whose K is not a multiple of 8 add the rest)
        const int total = M * chunks;
        for (int i = threadIdx.x; i < total; i += kThreads) {
            const int m = i / chunks, c = i - m * chunks;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(xs + m * xstride + c * 8);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(A + (int64_t)m * a.sAm + c * 8) : "memory");
        }
        asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
    } else {
        for (int m = 0; m < M; ++m)
            for (int k = threadIdx.x; k < kc; k += kThreads) xs[m * xstride + k] = A[(int64_t)m * a.sAm + (int64_t)k * a.sAk];
    }
}

// KW warps of the CTA split the CTA's K range, RW = 8 / KW warps take different 16-row tiles.
// CL > 1: a cluster of CL CTAs shares the same tiles and splits K once more (a weight matrix with few 16-row tiles, e.g.
// the 1024-row o and down projections of a small model, otherwise keeps most SMs idle): CTA r of the cluster takes K slices
// [r * KW, (r + 1) * KW), the CTAs r > 0 hand their sums to CTA 0 through distributed shared memory (two buffers alternating
// by round, one cluster barrier per round), and CTA 0 adds them in rank order and stores.
// Fragment bookkeeping (g = lane / 4, t = lane % 4): the thread loads K values [k, k+8) of weight rows
// r0+g and r0+g+8 and of activation row g. Instruction 1 takes K values k+0..3, instruction 2 takes
// k+4..7: slots (2t, 2t+1) <- first pair, slots (2t+8, 2t+9) <- second pair, the same in A and B.
template <int DT, int KW, int CL>
__global__ void __launch_bounds__(kThreads, 2) skinny_km_mma_kernel(const SkinnyArgs a, const int M, const int xstride) {
    constexpr int RW = kWarps / KW;
    constexpr int kPre = 4;                                                  // weight steps loaded ahead of the activations
    extern __shared__ __align__(16) unsigned char smem[];
    uint16_t *xs = reinterpret_cast<uint16_t *>(smem);                      // [M][xstride]
    float *red = reinterpret_cast<float *>(smem + (size_t)M * xstride * 2);  // [KW][RW][128] when KW > 1
    float *red2 = red + (KW > 1 ? kWarps * 128 : 0);                         // [2][CL - 1][RW][128] when CL > 1
    const int cr = CL > 1 ? (int)cluster_rank() : 0;

    pdl_launch_dependents();
    const int split = blockIdx.y;
    const int64_t batch = blockIdx.z;
    const int64_t k0 = (int64_t)split * a.kch;
    const int kc = (int)min(a.kch, a.K - k0);      // a CTA's K range always fits 32 bits (bounded by shared memory)
    int64_t offA, offB;
    batch_offsets(a, batch, offA, offB);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rw = warp / KW, kw = warp % KW;
    const int g = lane >> 2, t = lane & 3;
    int per = (kc + KW * CL - 1) / (KW * CL);
    per = (per + 31) / 32 * 32;
    const int ks = min(kc, (cr * KW + kw) * per), ke = min(kc, ks + per);
    const int nfull = (ke - ks) >> 5;
    const uint16_t *xrow = xs + g * xstride;
    const bool has_x = g < M;
    // which weight matrix a tile of the launch belongs to (one matrix unless the launch is grouped)
    const uint16_t *Bbase;
    uint16_t *Cg;
    int64_t Ng, ldbg, tile_first;
    auto select_group = [&](int64_t tile) {
        int gi = 0;
        if (a.ngroups > 1) {
            while (gi + 1 < a.ngroups && tile >= a.gtile0[gi + 1]) ++gi;
            Bbase = reinterpret_cast<const uint16_t *>(a.gB[gi]) + k0;
            Cg = reinterpret_cast<uint16_t *>(a.gC[gi]); Ng = a.gN[gi]; ldbg = a.gldb[gi]; tile_first = a.gtile0[gi];
        } else {
            Bbase = reinterpret_cast<const uint16_t *>(a.B) + offB + k0;
            Cg = reinterpret_cast<uint16_t *>(a.C); Ng = a.N; ldbg = a.ldb; tile_first = 0;
        }
    };

    // 16-row tiles are dealt out evenly: unit u (a row-warp slot of some CTA) takes tiles [u*T/U, (u+1)*T/U).
    // Every warp of a CTA runs the same number of rounds (the K-slice reduction below has CTA barriers).
    const int64_t T = a.ngroups > 1 ? a.gtile0[a.ngroups] : (a.N + 15) / 16;
    const int64_t U = (int64_t)(gridDim.x / CL) * RW;
    const int64_t u = (int64_t)(blockIdx.x / CL) * RW + rw;
    const int64_t t_begin = u * T / U, t_end = (u + 1) * T / U;
    const int64_t rounds = (T + U - 1) / U;

    // The weights do not depend on the previous kernel: the first steps of the first tile are in flight before the
    // activations are even staged (and, under programmatic dependent launch, before the previous kernel has finished).
    if (!a.early_weights) pdl_wait();
    uint4 pre_a[kPre], pre_b[kPre];
    const int npre = (t_begin < t_end) ? min(nfull, kPre) : 0;
    select_group(t_begin < T ? t_begin : 0);
    if (npre > 0) {
        const int64_t rp = (t_begin - tile_first) * 16;
        const uint4 *qa = reinterpret_cast<const uint4 *>(Bbase + min(rp + g, Ng - 1) * ldbg + ks) + t;
        const uint4 *qb = reinterpret_cast<const uint4 *>(Bbase + min(rp + g + 8, Ng - 1) * ldbg + ks) + t;
#pragma unroll
        for (int i = 0; i < kPre; ++i)
            if (i < npre) { pre_a[i] = ldg_stream(qa + 4 * i); pre_b[i] = ldg_stream(qb + 4 * i); }
    }

    pdl_wait();
    stage_activations(a, M, xstride, offA, k0, kc, xs);
    __syncthreads();

    for (int64_t round = 0; round < rounds; ++round) {
        const int64_t tile = t_begin + round;
        const bool active = tile < t_end;
        if (active) select_group(tile);
        const int64_t r0 = (tile - tile_first) * 16;
        float c[4] = {0.f, 0.f, 0.f, 0.f};
        if (active) {
            const uint16_t *pa = Bbase + min(r0 + g, Ng - 1) * ldbg;       // clamp: tail rows are loaded twice, stored once
            const uint16_t *pb = Bbase + min(r0 + g + 8, Ng - 1) * ldbg;
            // The trip count is the same for all 32 lanes (mma.sync needs the whole warp). Full 32-wide K chunks run
            // without predicates so the compiler can keep eight 16-byte loads in flight per lane; the ragged last
            // chunk (K slice not a multiple of 32) is one predicated step in which out-of-range lanes feed zeros.
            const uint4 *pa4 = reinterpret_cast<const uint4 *>(pa + ks) + t;
            const uint4 *pb4 = reinterpret_cast<const uint4 *>(pb + ks) + t;
            const uint4 *px4 = reinterpret_cast<const uint4 *>(xrow + ks) + t;
            int first = 0;
            if (round == 0) {
#pragma unroll
                for (int i = 0; i < kPre; ++i) {
                    if (i < npre) {
                        uint4 xv = make_uint4(0u, 0u, 0u, 0u);
                        if (has_x) xv = px4[4 * i];
                        mma_16816<DT>(c, pre_a[i].x, pre_b[i].x, pre_a[i].y, pre_b[i].y, xv.x, xv.y);
                        mma_16816<DT>(c, pre_a[i].z, pre_b[i].z, pre_a[i].w, pre_b[i].w, xv.z, xv.w);
                    }
                }
                first = npre;
            }
#pragma unroll 4
            for (int i = first; i < nfull; ++i) {
                const uint4 wa = ldg_stream(pa4 + 4 * i);
                const uint4 wb = ldg_stream(pb4 + 4 * i);
                uint4 xv = make_uint4(0u, 0u, 0u, 0u);
                if (has_x) xv = px4[4 * i];
                mma_16816<DT>(c, wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
                mma_16816<DT>(c, wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
            }
            if ((ke - ks) & 31) {
                const int k = ks + (nfull << 5) + t * 8;
                uint4 wa = make_uint4(0u, 0u, 0u, 0u), wb = wa, xv = wa;
                if (k < ke) {
                    wa = ldg_stream(reinterpret_cast<const uint4 *>(pa + k));
                    wb = ldg_stream(reinterpret_cast<const uint4 *>(pb + k));
                    if (has_x) xv = *reinterpret_cast<const uint4 *>(xrow + k);
                }
                mma_16816<DT>(c, wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
                mma_16816<DT>(c, wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
            }
        }
        if constexpr (KW > 1) {
            // sum the K slices in slice order (reproducible), then the kw == 0 warp stores
            float *mine = red + (kw * RW + rw) * 128 + lane * 4;
            mine[0] = c[0]; mine[1] = c[1]; mine[2] = c[2]; mine[3] = c[3];
            __syncthreads();
            if (kw == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float s = 0.f;
                    for (int w = 0; w < KW; ++w) s += red[(w * RW + rw) * 128 + lane * 4 + i];
                    c[i] = s;
                }
            }
            __syncthreads();
        }
        if constexpr (CL > 1) {
            float *buf = red2 + (size_t)(round & 1) * (CL - 1) * RW * 128;
            if (cr != 0 && kw == 0) {
                const uint32_t local = (uint32_t)__cvta_generic_to_shared(buf + ((cr - 1) * RW + rw) * 128 + lane * 4);
                uint32_t remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0));
                asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(remote), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]) : "memory");
            }
            cluster_barrier();
            if (cr == 0 && kw == 0) {
#pragma unroll
                for (int r = 0; r < CL - 1; ++r) {
                    const float4 o = *reinterpret_cast<const float4 *>(buf + (r * RW + rw) * 128 + lane * 4);
                    c[0] += o.x; c[1] += o.y; c[2] += o.z; c[3] += o.w;
                }
            }
        }
        if (active && kw == 0 && cr == 0) {
            // c[0], c[1]: weight row r0+g, tokens 2t, 2t+1;  c[2], c[3]: weight row r0+g+8
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int64_t n = r0 + g + (i >> 1) * 8;
                const int m = 2 * t + (i & 1);
                if (n < Ng && m < M) {
                    if (a.ngroups > 1) store_from_f32<DT>(Cg, (int64_t)m * Ng + n, c[i]);
                    else store_result<DT>(a, batch, split, m, M, n, c[i]);
                }
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// K-major 16-bit weights, cp.async-pipelined: grid = (persistent CTAs, nsplit, batch)
// ------------------------------------------------------------------------------------------------
// Same fragment scheme as skinny_km_mma_kernel, for problems with plenty of 16-row tiles. The 128-bit weight loads
// do not go to registers: each lane keeps a private ring of kAsyncDepth steps in shared memory. A step covers 64 K
// values of the lane's two rows (four 16-byte cp.async copies; the four lanes of a row fetch 128 contiguous bytes of
// it), so 16 loads per lane -- 8 KB per warp -- are in flight without costing registers, and the ring runs on across
// tile boundaries (the sequence of (tile, K step) pairs of a warp is flattened), so there is no drain between tiles.
// Slots are private to a lane: cp.async.wait_group is all the synchronisation the ring needs.
constexpr int kAsyncDepth = 4;
constexpr size_t kAsyncRingBytes = (size_t)kAsyncDepth * 4 * kThreads * 16;   // 64 KB

template <int DT>
__global__ void __launch_bounds__(kThreads, 2) skinny_km_async_kernel(const SkinnyArgs a, const int M, const int xstride) {
    extern __shared__ __align__(16) unsigned char smem[];
    uint4 *ring = reinterpret_cast<uint4 *>(smem);                                  // [depth][4][256 lanes]
    uint16_t *xs = reinterpret_cast<uint16_t *>(smem + kAsyncRingBytes);            // [M][xstride]

    pdl_launch_dependents();
    const int split = blockIdx.y;
    const int64_t batch = blockIdx.z;
    const int64_t k0 = (int64_t)split * a.kch;
    const int kc = (int)min(a.kch, a.K - k0);
    int64_t offA, offB;
    batch_offsets(a, batch, offA, offB);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t T = (a.N + 15) / 16;
    const int64_t W = (int64_t)gridDim.x * kWarps;
    const int64_t w = (int64_t)blockIdx.x * kWarps + warp;
    const int64_t t_begin = w * T / W, t_end = (w + 1) * T / W;      // a contiguous, even share of the tiles
    const int nk = (kc + 63) >> 6;                                     // 64-wide K steps per tile
    const uint16_t *Bbase = reinterpret_cast<const uint16_t *>(a.B) + offB + k0;
    const uint16_t *xrow = xs + g * xstride;
    const bool has_x = g < M;
    const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(ring) + (uint32_t)threadIdx.x * 16u;

    // issue cursor (tile, K step, ring slot), advanced incrementally: no divisions in the steady state
    int64_t i_tile = t_begin;
    int i_ks = 0, i_slot = 0;
    const uint16_t *pa = Bbase + min(i_tile * 16 + g, a.N - 1) * a.ldb;     // clamp: tail rows are loaded twice, stored once
    const uint16_t *pb = Bbase + min(i_tile * 16 + g + 8, a.N - 1) * a.ldb;
    auto issue = [&]() {
        if (i_tile < t_end) {
            const int k = i_ks * 64 + t * 8, k2 = k + 32;
            const uint32_t n1 = (k < kc) ? 16u : 0u, n2 = (k2 < kc) ? 16u : 0u;   // beyond the K range: zero-fill, nothing is read
            const int kk = (k < kc) ? k : 0, kk2 = (k2 < kc) ? k2 : 0;
            const uint32_t dst = ring_u32 + (uint32_t)i_slot * (4u * kThreads * 16u);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(pa + kk), "r"(n1) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + kThreads * 16u), "l"(pa + kk2), "r"(n2) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + 2u * kThreads * 16u), "l"(pb + kk), "r"(n1) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + 3u * kThreads * 16u), "l"(pb + kk2), "r"(n2) : "memory");
            if (++i_ks == nk) {
                i_ks = 0;
                ++i_tile;
                pa = Bbase + min(i_tile * 16 + g, a.N - 1) * a.ldb;
                pb = Bbase + min(i_tile * 16 + g + 8, a.N - 1) * a.ldb;
            }
        }
        i_slot = (i_slot + 1) & (kAsyncDepth - 1);
        asm volatile("cp.async.commit_group;" ::: "memory");          // one group per step, empty past the end
    };

    if (!a.early_weights) pdl_wait();
    for (int q = 0; q < kAsyncDepth; ++q) issue();

    // the weight copies above do not depend on a kernel still in flight (or came after the wait); the activations may
    pdl_wait();
    stage_activations(a, M, xstride, offA, k0, kc, xs);
    __syncthreads();
    float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};   // two chains: consecutive mma do not wait on each other
    int c_ks = 0, c_slot = 0;
    for (int64_t tile = t_begin; tile < t_end;) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kAsyncDepth - 1) : "memory");
        const uint4 *slot = ring + (size_t)c_slot * 4 * kThreads + threadIdx.x;
        const uint4 wa = slot[0], wa2 = slot[kThreads];
        const uint4 wb = slot[2 * kThreads], wb2 = slot[3 * kThreads];
        const int k = c_ks * 64 + t * 8;
        uint4 xv = make_uint4(0u, 0u, 0u, 0u), xv2 = make_uint4(0u, 0u, 0u, 0u);
        if (has_x && k < kc) xv = *reinterpret_cast<const uint4 *>(xrow + k);
        if (has_x && k + 32 < kc) xv2 = *reinterpret_cast<const uint4 *>(xrow + k + 32);
        mma_16816<DT>(c, wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
        mma_16816<DT>(c2, wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
        mma_16816<DT>(c, wa2.x, wb2.x, wa2.y, wb2.y, xv2.x, xv2.y);
        mma_16816<DT>(c2, wa2.z, wb2.z, wa2.w, wb2.w, xv2.z, xv2.w);
        c_slot = (c_slot + 1) & (kAsyncDepth - 1);
        issue();
        if (++c_ks == nk) {
            const int64_t r0 = tile * 16;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int64_t n = r0 + g + (i >> 1) * 8;
                const int m = 2 * t + (i & 1);
                if (n < a.N && m < M) store_result<DT>(a, batch, split, m, M, n, c[i] + c2[i]);
                c[i] = 0.f;
                c2[i] = 0.f;
            }
            c_ks = 0;
            ++tile;
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ------------------------------------------------------------------------------------------------
// K-major 16-bit weights, row-contiguous streaming: grid = (one CTA per SM, nsplit, batch)
// ------------------------------------------------------------------------------------------------
// Same arithmetic as skinny_km_async_kernel, other memory access: there a cp.async instruction of a warp fetches 64 bytes
// from each of 8 rows (every lane keeps to its own two rows), here it fetches 512 CONTIGUOUS bytes of ONE row -- 256 K values,
// 16 bytes per lane -- and sixteen such instructions bring one step of a 16-row tile into a ring slot that belongs to the
// warp ([16 rows][512 + 64 bytes]: the pitch of 64 mod 128 makes the fragment reads, 16 bytes per lane from rows g and g + 8,
// conflict-free). Two slots per warp: 16 KB per warp, 128 KB per SM in flight, as before; the lanes meet (__syncwarp) after
// their copies have landed and again before the slot is refilled.
constexpr int kRowsCh = 256;                                   // K values of a row per step
constexpr int kRowsPitch = kRowsCh * 2 + 64;                   // bytes
constexpr int kRowsDepth = 2;
constexpr size_t kRowsSlotBytes = (size_t)16 * kRowsPitch;     // 9216
constexpr size_t kRowsRingBytes = (size_t)kWarps * kRowsDepth * kRowsSlotBytes;   // 144 KB

template <int DT>
__global__ void __launch_bounds__(kThreads, 1) skinny_km_rows_kernel(const SkinnyArgs a, const int M, const int xstride) {
    extern __shared__ __align__(16) unsigned char smem[];
    uint16_t *xs = reinterpret_cast<uint16_t *>(smem + kRowsRingBytes);            // [M][xstride]

    pdl_launch_dependents();
    const int split = blockIdx.y;
    const int64_t batch = blockIdx.z;
    const int64_t k0 = (int64_t)split * a.kch;
    const int kc = (int)min(a.kch, a.K - k0);
    int64_t offA, offB;
    batch_offsets(a, batch, offA, offB);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t T = (a.N + 15) / 16;
    const int64_t W = (int64_t)gridDim.x * kWarps;
    const int64_t w = (int64_t)blockIdx.x * kWarps + warp;
    const int64_t t_begin = w * T / W, t_end = (w + 1) * T / W;      // a contiguous, even share of the tiles
    const int nk = (kc + kRowsCh - 1) / kRowsCh;                       // steps per tile
    const uint16_t *Bbase = reinterpret_cast<const uint16_t *>(a.B) + offB + k0;
    const uint16_t *xrow = xs + g * xstride;
    const bool has_x = g < M;
    unsigned char *ring = smem + (size_t)warp * kRowsDepth * kRowsSlotBytes;
    const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(ring) + (uint32_t)lane * 16u;

    int64_t i_tile = t_begin;
    int i_ks = 0, i_slot = 0;
    auto issue = [&]() {
        if (i_tile < t_end) {
            const int k = i_ks * kRowsCh + lane * 8;
            const uint32_t nbytes = (k < kc) ? 16u : 0u;               // beyond the K range: zero-fill, nothing is read
            const uint16_t *src = Bbase + ((k < kc) ? k : 0);
            const uint32_t dst = ring_u32 + (uint32_t)i_slot * (uint32_t)kRowsSlotBytes;
            const int64_t r0 = i_tile * 16;
#pragma unroll
            for (int r = 0; r < 16; ++r) {
                const int64_t row = min(r0 + r, a.N - 1);              // clamp: tail rows are loaded twice, stored once
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + (uint32_t)(r * kRowsPitch)), "l"(src + row * a.ldb), "r"(nbytes) : "memory");
            }
            if (++i_ks == nk) { i_ks = 0; ++i_tile; }
        }
        i_slot ^= 1;
        asm volatile("cp.async.commit_group;" ::: "memory");          // one group per step, empty past the end
    };

    if (!a.early_weights) pdl_wait();
    for (int q = 0; q < kRowsDepth; ++q) issue();

    pdl_wait();
    stage_activations(a, M, xstride, offA, k0, kc, xs);
    __syncthreads();
    float c[4] = {0.f, 0.f, 0.f, 0.f}, c2[4] = {0.f, 0.f, 0.f, 0.f};
    int c_ks = 0, c_slot = 0;
    for (int64_t tile = t_begin; tile < t_end;) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kRowsDepth - 1) : "memory");
        __syncwarp();                                                   // every lane's copies of this step have landed
        const unsigned char *slot = ring + (size_t)c_slot * kRowsSlotBytes;
        const int kbase = c_ks * kRowsCh;
#pragma unroll
        for (int sub = 0; sub < kRowsCh / 32; ++sub) {
            if (kbase + sub * 32 < kc) {                                // uniform over the warp
                const int k = kbase + sub * 32 + t * 8;
                const uint4 wa = *reinterpret_cast<const uint4 *>(slot + g * kRowsPitch + (sub * 32 + t * 8) * 2);
                const uint4 wb = *reinterpret_cast<const uint4 *>(slot + (g + 8) * kRowsPitch + (sub * 32 + t * 8) * 2);
                uint4 xv = make_uint4(0u, 0u, 0u, 0u);
                if (has_x && k < kc) xv = *reinterpret_cast<const uint4 *>(xrow + k);
                mma_16816<DT>(c, wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
                mma_16816<DT>(c2, wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
            }
        }
        __syncwarp();                                                   // the slot has been read by every lane
        c_slot ^= 1;
        issue();
        if (++c_ks == nk) {
            const int64_t r0 = tile * 16;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int64_t n = r0 + g + (i >> 1) * 8;
                const int m = 2 * t + (i & 1);
                if (n < a.N && m < M) store_result<DT>(a, batch, split, m, M, n, c[i] + c2[i]);
                c[i] = 0.f;
                c2[i] = 0.f;
            }
            c_ks = 0;
            ++tile;
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ------------------------------------------------------------------------------------------------
// N-major 16-bit weights (a contiguous [K, N] matrix) through mma.sync: grid = (one CTA per SM, nsplit, batch)
// ------------------------------------------------------------------------------------------------
// A warp owns strips of 128 weight columns and streams its CTA's K chunk of them: a cp.async instruction copies two K rows
// of the strip (2 x 256 contiguous bytes), eight of them one step of 16 K rows into a ring slot owned by the warp
// ([16 K rows][256 + 16 bytes]; two slots per warp, sixteen warps per SM). ldmatrix.x4.trans turns a 16 x 16 block of the slot
// into the A fragment of mma.sync.m16n8k16 (rows = weight columns, K along the fragment's K), the activation rows are the
// B operand straight from shared memory; eight mma per step, 32 accumulators per thread. The ring runs on across strips.
// With few strips K is split across CTAs (fp32 partial sums, summed in split order by skinny_finalize_kernel).
// The FFMA kernel below did 8 x M FMAs plus the unpacking per 16-byte load and fell from 5.6 TB/s at M = 1 to 2.2-3.4 at
// M = 2..8; it stays for float32 and for layouts this kernel does not take.
constexpr int kNmCols = 128;                                   // columns of a strip
constexpr int kNmPitch = kNmCols * 2 + 16;                     // bytes: 16 mod 128 keeps the 8 row addresses of an ldmatrix apart
constexpr int kNmDepth = 2;                                    // two CTAs per SM: 16 warps x 8 KB in flight
constexpr size_t kNmSlotBytes = (size_t)16 * kNmPitch;         // 4352
constexpr size_t kNmRingBytes = (size_t)kWarps * kNmDepth * kNmSlotBytes;   // 136 KB

template <int DT>
__global__ void __launch_bounds__(kThreads, 2) skinny_nm_mma_kernel(const SkinnyArgs a, const int M, const int xstride) {
    extern __shared__ __align__(16) unsigned char smem[];
    uint16_t *xs = reinterpret_cast<uint16_t *>(smem + kNmRingBytes);               // [M][xstride]

    pdl_launch_dependents();
    const int split = blockIdx.y;
    const int64_t batch = blockIdx.z;
    const int64_t k0 = (int64_t)split * a.kch;
    const int kc = (int)min(a.kch, a.K - k0);
    int64_t offA, offB;
    batch_offsets(a, batch, offA, offB);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int64_t S = (a.N + kNmCols - 1) / kNmCols;                 // strips
    const int64_t W = (int64_t)gridDim.x * kWarps;
    const int64_t w = (int64_t)blockIdx.x * kWarps + warp;
    const int64_t s_begin = w * S / W, s_end = (w + 1) * S / W;       // a contiguous, even share of the strips
    const int nk = (kc + 15) >> 4;                                     // steps of 16 K rows per strip
    const uint16_t *Bbase = reinterpret_cast<const uint16_t *>(a.B) + offB + k0 * a.ldb;
    unsigned char *ring = smem + (size_t)warp * kNmDepth * kNmSlotBytes;
    const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(ring);
    // this lane's 16 bytes of a copy instruction: K row (lane >> 4) of the pair, columns (lane & 15) * 8 .. + 7 of the strip
    const int cp_row = lane >> 4, cp_col = (lane & 15) * 8;
    const uint32_t cp_dst = ring_u32 + (uint32_t)(cp_row * kNmPitch + cp_col * 2);
    // this lane's row address of an ldmatrix.x4.trans: matrix (lane >> 3) = {K rows 0-7 | 8-15} x {columns 0-7 | 8-15} of a tile
    const uint32_t lm_off = (uint32_t)((((lane >> 4) & 1) * 8 + (lane & 7)) * kNmPitch + ((lane >> 3) & 1) * 16);

    int64_t i_strip = s_begin;
    int i_ks = 0, i_slot = 0;
    auto issue = [&]() {
        if (i_strip < s_end) {
            const int64_t col = i_strip * kNmCols + cp_col;
            const bool col_ok = col < a.N;                            // N is a multiple of 8: a lane's 8 columns are all in or all out
            const uint16_t *src = Bbase + (col_ok ? col : 0);
            const uint32_t dst = cp_dst + (uint32_t)i_slot * (uint32_t)kNmSlotBytes;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int k = i_ks * 16 + 2 * i + cp_row;
                const bool ok = col_ok && k < kc;                     // outside the matrix: zero-fill, nothing is read
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + (uint32_t)(2 * i * kNmPitch)),
                             "l"(src + (int64_t)(ok ? k : 0) * a.ldb), "r"(ok ? 16u : 0u) : "memory");
            }
            if (++i_ks == nk) { i_ks = 0; ++i_strip; }
        }
        i_slot = (i_slot + 1) & (kNmDepth - 1);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    if (!a.early_weights) pdl_wait();
    for (int q = 0; q < kNmDepth; ++q) issue();

    pdl_wait();
    stage_activations(a, M, xstride, offA, k0, kc, xs);
    {
        // K need not be a multiple of 8 in this layout: the last K % 8 values, which the 16-byte staging loop leaves out, one by
        // one; then zeros up to the next multiple of 16 (a step always multiplies 16 K rows)
        const uint16_t *A = reinterpret_cast<const uint16_t *>(a.A) + offA + k0 * a.sAk;
        for (int i = threadIdx.x; i < M * 8; i += kThreads) {
            const int m = i >> 3, k = (kc & ~7) + (i & 7);
            if (k < kc) xs[m * xstride + k] = A[(int64_t)m * a.sAm + (int64_t)k * a.sAk];
        }
        for (int i = threadIdx.x; i < M * 16; i += kThreads) {
            const int m = i >> 4, k = kc + (i & 15);
            if (k < ((kc + 15) & ~15)) xs[m * xstride + k] = 0;
        }
    }
    __syncthreads();
    const uint16_t *xrow = xs + g * xstride;
    const bool has_x = g < M;
    float c[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) { c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f; }
    int c_ks = 0, c_slot = 0;
    for (int64_t strip = s_begin; strip < s_end;) {
        asm volatile("cp.async.wait_group %0;" ::"n"(kNmDepth - 1) : "memory");
        __syncwarp();                                                   // every lane's copies of this step have landed
        const uint32_t slot = ring_u32 + (uint32_t)c_slot * (uint32_t)kNmSlotBytes + lm_off;
        uint32_t b0 = 0u, b1 = 0u;
        if (has_x) {
            b0 = *reinterpret_cast<const uint32_t *>(xrow + c_ks * 16 + 2 * t);
            b1 = *reinterpret_cast<const uint32_t *>(xrow + c_ks * 16 + 2 * t + 8);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            uint32_t a0, a1, a2, a3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                         : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3) : "r"(slot + (uint32_t)(j * 32)) : "memory");
            mma_16816<DT>(c[j], a0, a1, a2, a3, b0, b1);
        }
        __syncwarp();                                                   // the slot has been read by every lane
        c_slot = (c_slot + 1) & (kNmDepth - 1);
        issue();
        if (++c_ks == nk) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int64_t n = strip * kNmCols + j * 16 + g + (i >> 1) * 8;
                    const int m = 2 * t + (i & 1);
                    if (n < a.N && m < M) store_result<DT>(a, batch, split, m, M, n, c[j][i]);
                    c[j][i] = 0.f;
                }
            }
            c_ks = 0;
            ++strip;
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// ------------------------------------------------------------------------------------------------
// N-major weights: grid = (column blocks, nsplit, batch); a CTA covers 32*V columns
// ------------------------------------------------------------------------------------------------
template <int DT, int M>
__global__ void __launch_bounds__(kThreads) skinny_nm_kernel(const SkinnyArgs a) {
    using E = Elem<DT>;
    constexpr int V = E::vec;
    constexpr int CB = 32 * V;
    extern __shared__ __align__(16) unsigned char smem[];
    float *xs = reinterpret_cast<float *>(smem);   // [M][kch] activations as fp32
    float *red = xs + (int64_t)M * a.kch;          // [M][CB] cross-warp sums

    const int split = blockIdx.y;
    const int64_t batch = blockIdx.z;
    const int64_t k0 = (int64_t)split * a.kch;
    const int64_t kc = min(a.kch, a.K - k0);
    int64_t offA, offB;
    batch_offsets(a, batch, offA, offB);

    for (int m = 0; m < M; ++m)
        for (int64_t k = threadIdx.x; k < kc; k += kThreads)
            xs[m * a.kch + k] = load_as_f32<DT>(a.A, offA + m * a.sAm + (k0 + k) * a.sAk);
    for (int idx = threadIdx.x; idx < M * CB; idx += kThreads) red[idx] = 0.f;
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t col = (int64_t)blockIdx.x * CB + (int64_t)lane * V;
    float acc[M][V];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int j = 0; j < V; ++j) acc[m][j] = 0.f;

    if (col < a.N) {  // N is a multiple of V, so a thread's V columns are all in range or all out
        // contiguous K slice per warp
        const int64_t per = (kc + kWarps - 1) / kWarps;
        const int64_t kb = warp * per, ke = min(kc, kb + per);
        const typename E::bits *Bp = reinterpret_cast<const typename E::bits *>(a.B) + offB + k0 * a.ldb + col;
        int64_t k = kb;
        for (; k + 4 <= ke; k += 4) {
            uint4 w[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) w[u] = ldg_stream(reinterpret_cast<const uint4 *>(Bp + (k + u) * a.ldb));
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                float wf[V];
                unpack<DT>(w[u], wf);
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    float x = xs[m * a.kch + k + u];
#pragma unroll
                    for (int j = 0; j < V; ++j) acc[m][j] = fmaf(x, wf[j], acc[m][j]);
                }
            }
        }
        for (; k < ke; ++k) {
            float wf[V];
            unpack<DT>(ldg_stream(reinterpret_cast<const uint4 *>(Bp + k * a.ldb)), wf);
#pragma unroll
            for (int m = 0; m < M; ++m) {
                float x = xs[m * a.kch + k];
#pragma unroll
                for (int j = 0; j < V; ++j) acc[m][j] = fmaf(x, wf[j], acc[m][j]);
            }
        }
    }
    // Cross-warp sum in a fixed order (warp 0 first ... warp 7 last) so the result is reproducible.
    for (int w = 0; w < kWarps; ++w) {
        if (warp == w) {
#pragma unroll
            for (int m = 0; m < M; ++m)
#pragma unroll
                for (int j = 0; j < V; ++j) red[m * CB + lane * V + j] += acc[m][j];
        }
        __syncthreads();
    }
    for (int idx = threadIdx.x; idx < M * CB; idx += kThreads) {
        int m = idx / CB, c = idx - m * CB;
        int64_t n = (int64_t)blockIdx.x * CB + c;
        if (n < a.N) store_result<DT>(a, batch, split, m, M, n, red[idx]);
    }
}

// partial[nsplit][total] -> C[total], splits summed in index order, one rounding
template <int DT>
__global__ void __launch_bounds__(kThreads) skinny_finalize_kernel(const float *__restrict__ partial, void *__restrict__ C,
                                                                   int64_t total, int nsplit) {
    pdl_launch_dependents();
    pdl_wait();   // the partial sums come from the kernel before this one
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < total; i += stride) {
        float s = 0.f;
        for (int sp = 0; sp < nsplit; ++sp) s += partial[(int64_t)sp * total + i];
        store_from_f32<DT>(C, i, s);
    }
}

constexpr size_t kSmemBudget = 96 * 1024;  // two CTAs per SM

std::atomic<int> g_nm_mma{1};            // N-major 16-bit weights: 1 mma.sync kernel, 0 the FFMA kernel
std::atomic<int> g_row_streaming{1};     // streaming decode kernel: 1 row-contiguous copies (one CTA per SM), 0 per-lane ring
std::atomic<int> g_cluster_max{4};       // largest cluster the decode planner may use (1: never)
// K values a warp must keep after the extra split. Measured at M = 1 (us, no cluster / 2 / 4 CTAs): o 1024 x 2048 3.46 / 2.94 /
// 3.61, down 1024 x 3072 4.76 / 4.19 / 3.97, q 2048 x 1024 2.39 / 3.49: a cluster launch costs about a microsecond, which a
// slice of 96 or more K values per warp earns back and a shorter one does not.
std::atomic<int> g_cluster_min_k{96};

struct Plan {
    bool km;       // K-major weights
    bool mma;      // K-major 16-bit weights through mma.sync
    bool async;    // ... with the cp.async ring (plenty of tiles)
    bool rows;     // ... in its row-contiguous form (one CTA per SM)
    bool nm_mma;   // N-major 16-bit weights through mma.sync
    int KW;        // warps along K per CTA (mma)
    int CL;        // CTAs of a cluster that split K once more (mma, few tiles)
    int64_t xstride;
    int R;         // rows per warp (km)
    int64_t kch;
    int nsplit;
    size_t smem;
    unsigned gridx;
};

template <int DT>
bool make_plan(const GemmProblem &p, Plan &pl) {
    using E = Elem<DT>;
    const int V = E::vec;
    const int M = (int)p.M;
    const bool km = (p.sBk == 1 && p.K > 1) || (p.sBk == 1 && p.N == 1);
    const bool nm = (p.sBn == 1);
    if (!km && !nm) return false;
    if (((uintptr_t)p.B) & 15u) return false;
    if (p.batch_total > 65535) return false;
    for (int d = 0; d < p.nbatch; ++d)
        if (p.bsB[d] % V) return false;  // every batch slice of B must stay 16-byte aligned
    pl.km = km;
    pl.mma = false;
    pl.async = false;
    pl.rows = false;
    pl.nm_mma = false;
    pl.CL = 1;
    if (km && DT != MAGB200_F32) {
        if (p.K % V || (p.N > 1 && p.sBn % V)) return false;
        // activation rows live in shared memory with a pitch of 64 bytes mod 128 so that the 8 row groups
        // of a warp hit different banks
        int64_t kch_max = (int64_t)(kSmemBudget - 8 * 1024) / ((int64_t)M * 2) - 96;
        kch_max -= kch_max % 256;
        int64_t kch = p.K;
        int nsplit = 1;
        if (kch > kch_max) nsplit = (int)((p.K + kch_max - 1) / kch_max);
        const int64_t tiles = (p.N + 15) / 16;
        const int64_t warps_wanted = (int64_t)num_sms() * 16;
        // few row tiles and a long K: split K across CTAs too (each split keeps at least 2048 K values)
        if (tiles * kWarps * p.batch_total < warps_wanted && p.K >= 8192) {
            int want = (int)((warps_wanted + tiles * kWarps * p.batch_total - 1) / (tiles * kWarps * p.batch_total));
            int cap = (int)(p.K / 2048);
            if (want > cap) want = cap;
            if (want > nsplit) nsplit = want;
        }
        if (nsplit > 1) {
            kch = (p.K + nsplit - 1) / nsplit;
            kch = (kch + 255) / 256 * 256;
            nsplit = (int)((p.K + kch - 1) / kch);
        }
        // Long K with few 16-row tiles (e.g. a down projection, N = 5120, K = 25600): more K splits turn it into
        // enough (tile, split) units for the persistent pipelined kernel; only done when that threshold is reached.
        {
            const int64_t base_units = tiles * p.batch_total;
            int want = (int)((2 * warps_wanted + base_units - 1) / base_units);
            const int cap = (int)(p.K / 1024);
            if (want > cap) want = cap;
            if (base_units * nsplit < warps_wanted / 2 && want > nsplit && base_units * want >= warps_wanted / 2) {
                nsplit = want;
                kch = (p.K + nsplit - 1) / nsplit;
                kch = (kch + 255) / 256 * 256;
                nsplit = (int)((p.K + kch - 1) / kch);
            }
        }
        if (tiles * nsplit * p.batch_total >= warps_wanted / 2) {
            // enough tiles for every warp of a persistent grid to stream several: the cp.async-pipelined kernel.
            // Two CTAs per SM need the ring plus the activation rows within 110 KB: shorten the K chunk if necessary
            // (more splits cost a few MB of partial sums, one CTA per SM costs half the loads in flight).
            int64_t kch_two = ((int64_t)110 * 1024 - (int64_t)kAsyncRingBytes) / ((int64_t)M * 2) - 32;
            kch_two -= kch_two % 256;
            const bool scarce = tiles * p.batch_total < warps_wanted;   // fewer row tiles than warps: K chunks are the only parallelism
            if (scarce && kch > kch_two && kch_two >= 1024) {
                nsplit = (int)((p.K + kch_two - 1) / kch_two);
                kch = (p.K + nsplit - 1) / nsplit;
                kch = (kch + 255) / 256 * 256;
                nsplit = (int)((p.K + kch - 1) / kch);
            }
            // A warp streams whole (tile, K chunk) units; when the units do not divide evenly over the warps, the last
            // part of the launch runs with few warps and little memory parallelism. For a long K try more splits and keep
            // the cheapest by a cost in K steps fitted to measurements: 0.3 x the longest warp + 0.7 x the mean warp,
            // plus what splitting costs (the second kernel, the partial sums).
            if (scarce && p.K >= 4096 && kch_two >= 1024) {
                auto cost_of = [&](int ns, int64_t kc_) {
                    const int64_t gx = ((int64_t)num_sms() * 2 + (int64_t)ns * p.batch_total - 1) / ((int64_t)ns * p.batch_total);
                    const double warps = (double)(gx * kWarps);
                    const double steps = (double)((kc_ + 63) / 64);
                    const double longest = (double)((tiles + (int64_t)warps - 1) / (int64_t)warps) * steps;
                    const double mean = (double)tiles / warps * steps;
                    return 0.3 * longest + 0.7 * mean + (ns > 1 ? 16.0 : 0.0) + 0.5 * ns;
                };
                int best_ns = nsplit;
                int64_t best_kch = kch;
                double best = cost_of(nsplit, kch);
                for (int ns = nsplit + 1; ns <= 64 && p.K / ns >= 1024; ++ns) {
                    int64_t kc_ = (p.K + ns - 1) / ns;
                    kc_ = (kc_ + 255) / 256 * 256;
                    const int ns_eff = (int)((p.K + kc_ - 1) / kc_);
                    if (kc_ > kch_two) continue;
                    const double cost = cost_of(ns_eff, kc_);
                    if (cost < best - 1e-9) { best = cost; best_ns = ns_eff; best_kch = kc_; }
                }
                nsplit = best_ns;
                kch = best_kch;
            }
            pl.mma = true; pl.async = true; pl.KW = 1; pl.CL = 1; pl.kch = kch; pl.nsplit = nsplit; pl.R = 0;
            pl.xstride = (kch + 63) / 64 * 64 + 32;
            pl.smem = kAsyncRingBytes + (size_t)M * pl.xstride * 2;
            const int64_t other = (int64_t)nsplit * p.batch_total;
            int per_sm = pl.smem <= 110 * 1024 ? 2 : 1;
            {
                // the row-contiguous form whenever its ring and the activation rows fit one CTA's shared memory (measured at
                // M = 1: 151936 x 1024 5.43 -> 5.92 TB/s, 65536 x 4096 5.56 -> 6.19, 51200 x 5120 5.15 -> 6.51; M = 8 gains 2-4 %)
                const size_t rows_smem = kRowsRingBytes + (size_t)M * pl.xstride * 2;
                // ... and every one of its 8 warps per SM gets whole tiles to stream: with few row tiles and K split over CTAs the
                // per-lane-ring kernel, with twice the warps, balances better (5120 x 5120 at M = 1: 13.0 us against 19.9;
                // 12288 x 4096, 768 tiles: 21.7 against 19.2 the other way)
                const bool enough_tiles = tiles * p.batch_total >= (int64_t)num_sms() * 5;
                if (g_row_streaming.load() && enough_tiles && rows_smem <= (size_t)224 * 1024) { pl.rows = true; pl.smem = rows_smem; per_sm = 1; }
            }
            int64_t want = ((int64_t)num_sms() * per_sm + other - 1) / other;
            if (want < 1) want = 1;
            pl.gridx = (unsigned)want;
            return pl.nsplit <= 65535;
        }
        int KW = 1;
        // more warps along K while the GPU has room for them: past its resident capacity (16 warps per SM) the extra CTAs
        // would only queue behind the first wave (384 tiles x 8 warps: 6.0 us, x 4 warps in one wave: see the measurements
        // beside g_cluster_min_k)
        while (KW < kWarps && tiles * KW * 2 * nsplit * p.batch_total <= warps_wanted && kch / (KW * 2) >= 128) KW *= 2;
        pl.mma = true; pl.KW = KW; pl.kch = kch; pl.nsplit = nsplit; pl.R = 0;
        pl.xstride = (kch + 63) / 64 * 64 + 32;

        const int RW = kWarps / KW;
        const int64_t blocks = (tiles + RW - 1) / RW;
        const int64_t other = (int64_t)nsplit * p.batch_total;
        // fewer CTAs than SMs although every warp already has its own K slice: clusters split K once more
        int CL = 1;
        if (KW == kWarps)
            while (CL < 4 && blocks * other * CL * 2 <= (int64_t)num_sms() * 2 && kch / (KW * CL * 2) >= g_cluster_min_k.load()) CL *= 2;
        if (g_cluster_max.load() < CL) CL = g_cluster_max.load() < 1 ? 1 : g_cluster_max.load();
        pl.CL = CL;
        pl.smem = (size_t)M * pl.xstride * 2 + (KW > 1 ? (size_t)kWarps * 128 * 4 : 0) + (CL > 1 ? (size_t)2 * (CL - 1) * RW * 128 * 4 : 0);
        // many short CTAs (one or two tiles per warp) let the hardware scheduler even out the SMs
        int64_t want = (int64_t)num_sms() * 32;
        want = (want + other - 1) / other;
        if (want < 1) want = 1;
        pl.gridx = (unsigned)(blocks < want ? blocks : want) * (unsigned)CL;
        return pl.nsplit <= 65535;
    }
    if (km) {
        if (p.K % V || (p.N > 1 && p.sBn % V)) return false;
        const int64_t warps_wanted = (int64_t)num_sms() * 2 * kWarps;
        pl.R = (p.N >= 4 * warps_wanted) ? 4 : (p.N >= 2 * warps_wanted ? 2 : 1);
        if (M > 4 && pl.R > 2) pl.R = 2;  // keep R*M accumulators + unpacked operands in registers
        int64_t kch_max = (int64_t)(kSmemBudget / ((size_t)M * E::size));
        kch_max -= kch_max % (V * 32);
        int64_t kch = p.K;
        int nsplit = 1;
        if (kch > kch_max) { nsplit = (int)((p.K + kch_max - 1) / kch_max); }
        // too few row groups to occupy the GPU and a long K: split K as well
        const int64_t groups = (p.N + pl.R - 1) / pl.R * p.batch_total;
        if (groups < warps_wanted / 2 && p.K >= 4096) {
            int want = (int)((warps_wanted / 2 + groups - 1) / groups);
            int cap = (int)(p.K / 1024);
            if (want > cap) want = cap;
            if (want > nsplit) nsplit = want;
        }
        if (nsplit > 1) {
            kch = (p.K + nsplit - 1) / nsplit;
            kch = (kch + V * 32 - 1) / (V * 32) * (V * 32);
            nsplit = (int)((p.K + kch - 1) / kch);
        }
        pl.kch = kch; pl.nsplit = nsplit;
        pl.smem = (size_t)M * kch * E::size;
        int64_t blocks = (p.N + (int64_t)kWarps * pl.R - 1) / ((int64_t)kWarps * pl.R);
        int64_t cap = ((int64_t)num_sms() * 2 * 4) / ((int64_t)nsplit * p.batch_total) ;
        if (cap < 1) cap = 1;
        pl.gridx = (unsigned)(blocks < cap ? blocks : cap);
    } else {
        if (p.N % V || p.sBk % V) return false;
        if (DT != MAGB200_F32 && g_nm_mma.load()) {
            // Strips of 128 columns, each with a K chunk, are the units dealt out to 16 warps per SM. The number of K chunks is
            // searched: a warp's share is whole units, so the launch lasts ceil(units / warps) units (151936 columns on 1184 warps
            // were 1187 units: three warps ran a second strip alone, 4.9 TB/s); more chunks cost partial sums and a second kernel.
            const int64_t strips = (p.N + kNmCols - 1) / kNmCols * p.batch_total;
            const int64_t warps = (int64_t)num_sms() * 2 * kWarps;
            int64_t kch_max = ((int64_t)110 * 1024 - (int64_t)kNmRingBytes) / ((int64_t)M * 2) - 48;
            kch_max -= kch_max % 16;
            const int ns_min = (int)((p.K + kch_max - 1) / kch_max);
            int ns_cap = (int)(p.K / 128);
            if (ns_cap < ns_min) ns_cap = ns_min;
            if (ns_cap > 64) ns_cap = 64 > ns_min ? 64 : ns_min;
            int best_ns = ns_min;
            double best_cost = 1e300;
            for (int ns = ns_min; ns <= ns_cap; ++ns) {
                const int64_t units = strips * ns;
                const int64_t per = (units + warps - 1) / warps;
                const double eff = (double)units / (double)(per * warps);
                const double busy = units < warps ? (double)units / (double)warps : 1.0;   // idle warps cost nothing while enough bytes are in flight
                const double fill = busy < 0.4 ? busy / 0.4 : 1.0;
                const double cost = 1.0 / (units < warps ? fill : eff) * (ns > 1 ? 1.05 + 4.0 * ns * M / (double)p.K : 1.0);
                if (cost < best_cost - 1e-9) { best_cost = cost; best_ns = ns; }
            }
            int nsplit = best_ns;
            int64_t kch = (p.K + nsplit - 1) / nsplit;
            kch = (kch + 15) / 16 * 16;
            nsplit = (int)((p.K + kch - 1) / kch);
            pl.nm_mma = true; pl.kch = kch; pl.nsplit = nsplit; pl.R = 0;
            pl.xstride = (kch + 15) / 16 * 16 + 40;                  // 80 bytes mod 128: the 8 activation rows of a fragment read spread over the banks
            pl.smem = kNmRingBytes + (size_t)M * pl.xstride * 2;
            int64_t gx = ((int64_t)num_sms() * 2 + (int64_t)nsplit * p.batch_total - 1) / ((int64_t)nsplit * p.batch_total);
            if (gx < 1) gx = 1;
            const int64_t strips_one = (p.N + kNmCols - 1) / kNmCols;
            if (gx * kWarps > strips_one) gx = (strips_one + kWarps - 1) / kWarps;
            pl.gridx = (unsigned)gx;
            return pl.nsplit <= 65535;
        }
        const int CB = 32 * V;
        int64_t kch_max = (int64_t)((kSmemBudget - (size_t)M * CB * 4) / ((size_t)M * 4));
        kch_max -= kch_max % 32;
        int64_t kch = p.K;
        int nsplit = 1;
        if (kch > kch_max) nsplit = (int)((p.K + kch_max - 1) / kch_max);
        const int64_t blocks = (p.N + CB - 1) / CB;
        if (blocks * p.batch_total < num_sms() && p.K >= 2048) {
            int want = (int)((num_sms() * 2 + blocks * p.batch_total - 1) / (blocks * p.batch_total));
            int cap = (int)(p.K / 512);
            if (want > cap) want = cap;
            if (want > nsplit) nsplit = want;
        }
        if (nsplit > 1) {
            kch = (p.K + nsplit - 1) / nsplit;
            kch = (kch + 31) / 32 * 32;
            nsplit = (int)((p.K + kch - 1) / kch);
        }
        pl.kch = kch; pl.nsplit = nsplit; pl.R = 0;
        pl.smem = (size_t)M * kch * 4 + (size_t)M * CB * 4;
        pl.gridx = (unsigned)blocks;
    }
    return pl.nsplit <= 65535;
}

// Opt-in to more than 48 KB of dynamic shared memory: once per (kernel, device) with the largest size any plan asks for,
// not on every launch (the attribute call costs more host time than a small decode kernel runs). The kernels share a few
// function signatures, so the record is a small table keyed by the kernel's address.
constexpr size_t kSmemOptIn = 128 * 1024;
struct OptInEntry { std::atomic<uintptr_t> kernel{0}; std::atomic<uint32_t> devices{0}; };
OptInEntry g_optin[128];

template <typename K>
int set_smem(K kernel, size_t bytes) {
    if (bytes <= 48 * 1024) return MAGB200_OK;
    int dev = 0;
    MAGB200_CUDA_TRY(cudaGetDevice(&dev));
    const uint32_t bit = 1u << (dev & 31);
    const uintptr_t me = (uintptr_t)kernel;
    OptInEntry *e = nullptr;
    for (unsigned probe = 0; probe < 128 && !e; ++probe) {
        OptInEntry &c = g_optin[((me >> 4) + probe) & 127u];
        uintptr_t cur = c.kernel.load(std::memory_order_acquire);
        if (cur == 0 && c.kernel.compare_exchange_strong(cur, me)) cur = me;
        if (cur == me) e = &c;
    }
    if (e && bytes <= kSmemOptIn && (e->devices.load(std::memory_order_acquire) & bit)) return MAGB200_OK;
    MAGB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes > kSmemOptIn ? bytes : kSmemOptIn)));
    if (e && bytes <= kSmemOptIn) e->devices.fetch_or(bit, std::memory_order_release);
    return MAGB200_OK;
}

template <int DT, int M>
int launch_m(const GemmProblem &p, const Plan &pl, const SkinnyArgs &a, cudaStream_t st) {
    dim3 grid(pl.gridx, pl.nsplit, (unsigned)p.batch_total);
    int rc = MAGB200_OK;
    if (pl.async) {
        if constexpr (DT != MAGB200_F32) {
            if (pl.rows) {
                static std::atomic<uint32_t> optin{0};
                int dev = 0;
                MAGB200_CUDA_TRY(cudaGetDevice(&dev));
                if (!(optin.load() & (1u << (dev & 31)))) {
                    MAGB200_CUDA_TRY(cudaFuncSetAttribute(skinny_km_rows_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024));
                    optin.fetch_or(1u << (dev & 31));
                }
                if ((rc = launch_pdl(skinny_km_rows_kernel<DT>, grid, dim3(kThreads), pl.smem, st, a, M, (int)pl.xstride))) return rc;
            } else {
            if ((rc = set_smem(skinny_km_async_kernel<DT>, pl.smem))) return rc;
            if ((rc = launch_pdl(skinny_km_async_kernel<DT>, grid, dim3(kThreads), pl.smem, st, a, M, (int)pl.xstride))) return rc;
            }
        }
    } else if (pl.mma) {
        if constexpr (DT != MAGB200_F32) {
#define LAUNCH_KW(KWV)                                                                                   \
    case KWV:                                                                                            \
        if ((rc = set_smem(skinny_km_mma_kernel<DT, KWV, 1>, pl.smem))) return rc;                       \
        if ((rc = launch_pdl(skinny_km_mma_kernel<DT, KWV, 1>, grid, dim3(kThreads), pl.smem, st, a, M, (int)pl.xstride))) return rc; \
        break;
            if (pl.CL == 2) {
                if ((rc = set_smem(skinny_km_mma_kernel<DT, kWarps, 2>, pl.smem))) return rc;
                if ((rc = launch_pdl_cluster(skinny_km_mma_kernel<DT, kWarps, 2>, grid, dim3(kThreads), pl.smem, st, 2, a, M, (int)pl.xstride))) return rc;
            } else if (pl.CL == 4) {
                if ((rc = set_smem(skinny_km_mma_kernel<DT, kWarps, 4>, pl.smem))) return rc;
                if ((rc = launch_pdl_cluster(skinny_km_mma_kernel<DT, kWarps, 4>, grid, dim3(kThreads), pl.smem, st, 4, a, M, (int)pl.xstride))) return rc;
            } else
            switch (pl.KW) { LAUNCH_KW(1) LAUNCH_KW(2) LAUNCH_KW(4) LAUNCH_KW(8) }
#undef LAUNCH_KW
        }
    } else if (pl.km) {
        if (pl.R == 4) {
            if constexpr (M <= 4) {
                if ((rc = set_smem(skinny_km_kernel<DT, M, 4>, pl.smem))) return rc;
                skinny_km_kernel<DT, M, 4><<<grid, kThreads, pl.smem, st>>>(a);
            }
        } else if (pl.R == 2) {
            if ((rc = set_smem(skinny_km_kernel<DT, M, 2>, pl.smem))) return rc;
            skinny_km_kernel<DT, M, 2><<<grid, kThreads, pl.smem, st>>>(a);
        } else {
            if ((rc = set_smem(skinny_km_kernel<DT, M, 1>, pl.smem))) return rc;
            skinny_km_kernel<DT, M, 1><<<grid, kThreads, pl.smem, st>>>(a);
        }
    } else if (pl.nm_mma) {
        if constexpr (DT != MAGB200_F32) {
            static std::atomic<uint32_t> optin{0};
            int dev = 0;
            MAGB200_CUDA_TRY(cudaGetDevice(&dev));
            if (!(optin.load() & (1u << (dev & 31)))) {
                MAGB200_CUDA_TRY(cudaFuncSetAttribute(skinny_nm_mma_kernel<DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024));
                optin.fetch_or(1u << (dev & 31));
            }
            if ((rc = launch_pdl(skinny_nm_mma_kernel<DT>, grid, dim3(kThreads), pl.smem, st, a, M, (int)pl.xstride))) return rc;
        }
    } else {
        if ((rc = set_smem(skinny_nm_kernel<DT, M>, pl.smem))) return rc;
        skinny_nm_kernel<DT, M><<<grid, kThreads, pl.smem, st>>>(a);
    }
    count_launch();
    MAGB200_CUDA_TRY(cudaGetLastError());
    return MAGB200_OK;
}

template <int DT>
int launch_dt(const GemmProblem &p, cudaStream_t st, float *scratch, size_t scratch_bytes, int *used_splitk, bool weights_settled) {
    Plan pl;
    if (!make_plan<DT>(p, pl)) { set_error("skinny: layout not supported"); return MAGB200_ERR_INVALID_ARG; }
    const int64_t total = p.batch_total * p.M * p.N;
    if (pl.nsplit > 1 && (size_t)pl.nsplit * total * sizeof(float) > scratch_bytes) {
        set_error("skinny: split-K scratch of %zu bytes exceeds the %zu available", (size_t)pl.nsplit * total * 4, scratch_bytes);
        return MAGB200_ERR_TOO_LARGE;
    }
    SkinnyArgs a;
    a.A = p.A; a.B = p.B; a.C = p.C; a.partial = scratch;
    a.N = p.N; a.K = p.K; a.sAm = p.sAm; a.sAk = p.sAk;
    a.ldb = pl.km ? p.sBn : p.sBk;
    a.kch = pl.kch; a.nsplit = pl.nsplit; a.nbatch = p.nbatch; a.batch_total = p.batch_total;
    a.early_weights = weights_settled ? 1 : 0;
    a.ngroups = 0;
    for (int d = 0; d < kMaxBatchDims; ++d) { a.bshape[d] = p.bshape[d]; a.bsA[d] = p.bsA[d]; a.bsB[d] = p.bsB[d]; }
    int rc;
    switch (p.M) {
#define CASE(MM) case MM: rc = launch_m<DT, MM>(p, pl, a, st); break;
        CASE(1) CASE(2) CASE(3) CASE(4) CASE(5) CASE(6) CASE(7) CASE(8)
#undef CASE
        default: set_error("skinny: M=%lld out of range", (long long)p.M); return MAGB200_ERR_INVALID_ARG;
    }
    if (rc) return rc;
    if (pl.nsplit > 1) {
        int64_t blocks = (total + kThreads - 1) / kThreads;
        if (blocks > num_sms() * 8) blocks = num_sms() * 8;
        if (int rc2 = launch_pdl(skinny_finalize_kernel<DT>, dim3((unsigned)blocks), dim3(kThreads), 0, st, (const float *)scratch, p.C, total, pl.nsplit)) return rc2;
        count_launch();
        MAGB200_CUDA_TRY(cudaGetLastError());
    }
    if (used_splitk) *used_splitk = pl.nsplit > 1;
    return MAGB200_OK;
}

}  // namespace

namespace {
template <int DT>
int launch_grouped_dt(const GemmProblem *ps, int count, cudaStream_t st, bool weights_settled) {
    // plan for one problem with all the groups' 16-row tiles; only the register-load kernel without a K split is grouped
    GemmProblem pc = ps[0];
    SkinnyArgs a;
    memset(&a, 0, sizeof(a));
    int64_t tiles = 0;
    for (int i = 0; i < count; ++i) {
        a.gB[i] = ps[i].B; a.gC[i] = ps[i].C; a.gN[i] = ps[i].N; a.gldb[i] = ps[i].sBn;
        a.gtile0[i] = tiles;
        tiles += (ps[i].N + 15) / 16;
    }
    a.gtile0[count] = tiles;
    pc.N = tiles * 16;
    Plan pl;
    if (!make_plan<DT>(pc, pl) || !pl.mma || pl.async || pl.nsplit != 1) return 1;   // not applicable: the caller launches one by one
    // (a member launched alone may cut K into a different number of slices than the group does: same products, another
    // order of the fp32 sums)
    a.A = pc.A; a.B = nullptr; a.C = nullptr; a.partial = nullptr;
    a.N = pc.N; a.K = pc.K; a.sAm = pc.sAm; a.sAk = pc.sAk; a.ldb = 0;
    a.kch = pl.kch; a.nsplit = 1; a.nbatch = 0; a.batch_total = 1;
    a.early_weights = weights_settled ? 1 : 0;
    a.ngroups = count;
    const int M = (int)pc.M;
    dim3 grid(pl.gridx, 1, 1);
    int rc = MAGB200_OK;
#define LAUNCH_KW(KWV)                                                                                   \
    case KWV:                                                                                            \
        if ((rc = set_smem(skinny_km_mma_kernel<DT, KWV, 1>, pl.smem))) return rc;                       \
        if ((rc = launch_pdl(skinny_km_mma_kernel<DT, KWV, 1>, grid, dim3(kThreads), pl.smem, st, a, M, (int)pl.xstride))) return rc; \
        break;
    if (pl.CL == 2) {
        if ((rc = set_smem(skinny_km_mma_kernel<DT, kWarps, 2>, pl.smem))) return rc;
        if ((rc = launch_pdl_cluster(skinny_km_mma_kernel<DT, kWarps, 2>, grid, dim3(kThreads), pl.smem, st, 2, a, M, (int)pl.xstride))) return rc;
    } else if (pl.CL == 4) {
        if ((rc = set_smem(skinny_km_mma_kernel<DT, kWarps, 4>, pl.smem))) return rc;
        if ((rc = launch_pdl_cluster(skinny_km_mma_kernel<DT, kWarps, 4>, grid, dim3(kThreads), pl.smem, st, 4, a, M, (int)pl.xstride))) return rc;
    } else
    switch (pl.KW) { LAUNCH_KW(1) LAUNCH_KW(2) LAUNCH_KW(4) LAUNCH_KW(8) }
#undef LAUNCH_KW
    count_launch();
    MAGB200_CUDA_TRY(cudaGetLastError());
    return MAGB200_OK;
}
}  // namespace

void set_decode_row_streaming(int on) { g_row_streaming.store(on ? 1 : 0); g_nm_mma.store(on ? 1 : 0); }
void set_decode_cluster_max(int max_cluster) { g_cluster_max.store(max_cluster < 1 ? 1 : (max_cluster > 4 ? 4 : max_cluster)); }

// Several decode-shaped products with the same activation rows in one launch: r_i = x . y_i. Returns 1 when the group cannot
// run as one launch (mixed layouts, a K split, too many tiles: those shapes are better off alone anyway).
int launch_skinny_grouped(const GemmProblem *ps, int count, cudaStream_t st, bool weights_settled) {
    if (count < 2 || count > kMaxGroups) return 1;
    const GemmProblem &p0 = ps[0];
    if (p0.dtype == MAGB200_F32 || p0.M < 1 || p0.M > 8) return 1;
    for (int i = 0; i < count; ++i) {
        const GemmProblem &p = ps[i];
        if (p.dtype != p0.dtype || p.M != p0.M || p.K != p0.K || p.A != p0.A || p.sAm != p0.sAm || p.sAk != p0.sAk) return 1;
        if (p.batch_total != 1 || p.nbatch != 0 || p.sBk != 1 || p.K < 2 || p.K % 8 || p.sBn % 8 || ((uintptr_t)p.B & 15u)) return 1;
    }
    return p0.dtype == MAGB200_BF16 ? launch_grouped_dt<MAGB200_BF16>(ps, count, st, weights_settled)
                                    : launch_grouped_dt<MAGB200_F16>(ps, count, st, weights_settled);
}

// What the planner would do with a decode-shaped product, without launching anything (host logic only: tests pin the decisions).
// kind: 0 not a decode-shaped product the kernels take, 1 small projections (register loads), 2 per-lane-ring streaming,
// 3 row-contiguous streaming, 4 N-major mma.sync, 5 FFMA kernels.
int describe_skinny_plan(const GemmProblem &p, int *kind, int *nsplit, int *gridx, int *warps_along_k, int *cluster, int64_t *kch) {
    Plan pl;
    bool ok = false;
    if (p.M >= 1 && p.M <= 8) {
        switch (p.dtype) {
            case MAGB200_F32:  ok = make_plan<MAGB200_F32>(p, pl); break;
            case MAGB200_F16:  ok = make_plan<MAGB200_F16>(p, pl); break;
            case MAGB200_BF16: ok = make_plan<MAGB200_BF16>(p, pl); break;
        }
    }
    *kind = !ok ? 0 : pl.nm_mma ? 4 : (pl.mma && pl.async) ? (pl.rows ? 3 : 2) : pl.mma ? 1 : 5;
    *nsplit = ok ? pl.nsplit : 0;
    *gridx = ok ? (int)pl.gridx : 0;
    *warps_along_k = ok && pl.mma && !pl.async ? pl.KW : 0;
    *cluster = ok && pl.mma && !pl.async ? pl.CL : 0;
    *kch = ok ? pl.kch : 0;
    return MAGB200_OK;
}

bool skinny_supported(const GemmProblem &p) {
    if (p.M < 1 || p.M > 8) return false;
    Plan pl;
    switch (p.dtype) {
        case MAGB200_F32:  return make_plan<MAGB200_F32>(p, pl);
        case MAGB200_F16:  return make_plan<MAGB200_F16>(p, pl);
        case MAGB200_BF16: return make_plan<MAGB200_BF16>(p, pl);
    }
    return false;
}

// Scratch needed by launch_skinny for this problem (0 when K is not split).
size_t skinny_scratch_bytes(const GemmProblem &p) {
    Plan pl;
    bool ok = false;
    switch (p.dtype) {
        case MAGB200_F32:  ok = make_plan<MAGB200_F32>(p, pl); break;
        case MAGB200_F16:  ok = make_plan<MAGB200_F16>(p, pl); break;
        case MAGB200_BF16: ok = make_plan<MAGB200_BF16>(p, pl); break;
    }
    if (!ok || pl.nsplit <= 1) return 0;
    return (size_t)pl.nsplit * p.batch_total * p.M * p.N * sizeof(float);
}

// `weights_settled`: the caller knows that no kernel which may still be running writes the weight operand, so the kernels
// may fetch weights before they wait for their predecessors (see pdl_wait above). Pass false when in doubt.
int launch_skinny(const GemmProblem &p, cudaStream_t st, float *scratch, size_t scratch_bytes, int *used_splitk, bool weights_settled) {
    switch (p.dtype) {
        case MAGB200_F32:  return launch_dt<MAGB200_F32>(p, st, scratch, scratch_bytes, used_splitk, weights_settled);
        case MAGB200_F16:  return launch_dt<MAGB200_F16>(p, st, scratch, scratch_bytes, used_splitk, weights_settled);
        case MAGB200_BF16: return launch_dt<MAGB200_BF16>(p, st, scratch, scratch_bytes, used_splitk, weights_settled);
    }
    set_error("skinny: unsupported dtype %d", p.dtype);
    return MAGB200_ERR_INVALID_ARG;
}

}  // namespace magb200
