// Exact-fp32 tiled FFMA matmul for arbitrary element strides.
//
// Role on the path: (1) the float32 matmul -- tensor cores only offer TF32 inputs (10-bit mantissa),
// which cannot hold the reference's fp32 accuracy, so fp32 products run on the FP32 pipes and are
// bounded by the FFMA roofline, not the tensor roofline; (2) 16-bit operands whose layout TMA cannot
// describe (an inner stride that is not 1 on either of the last two dims, a row pitch that is not a
// multiple of 16 bytes, a misaligned base). Operands are gathered through their strides straight into
// shared memory as fp32, so no packed copy of a strided view is ever made in HBM.
//
// Tile: 128x128x16 per 256-thread CTA, 8x8 accumulators per thread (two 4-wide groups of rows and of
// columns, 64 apart): four 128-bit shared-memory reads feed 64 FMAs. A warp covers 4 row groups x 8
// column groups, so its reads are broadcasts or one contiguous 128-byte line. The next K tile is fetched
// from global memory into registers while the current one is multiplied, and shared memory is double
// buffered: one barrier per K tile. One CTA per SM owns the whole register file (up to 255 per thread).
//
// fp32 accuracy: a single fp32 accumulator that walks the whole K loses several units in the last place
// at K in the thousands, more than the reference's blocked CPU kernel does. For float32 the kernel
// therefore sums 64 products at a time in a fresh accumulator and folds it into the running total with an
// error-free TwoSum, carrying the lost low part along; what remains is the rounding inside one 64-term
// group. The running totals stay in registers; the low parts, touched only once per fold, live in shared
// memory (64 KB), which is what keeps the kernel free of register spills. The 16-bit dtypes skip all of
// this: their error is set by the final rounding of the result.
//
// Few tiles (an output smaller than the GPU): K is split over several CTAs per tile; each writes its
// (total, low) pair as fp32 and a second kernel adds the pairs in split order, again with TwoSum, and
// rounds once.
#include "common.cuh"

#include <atomic>
#include <cstring>

namespace magb200 {

namespace {

constexpr int BM = 128, BN = 128, BK = 16, THREADS = 256, PAD = 4;
constexpr int kLoads = (BM * BK) / THREADS;   // elements of each operand tile a thread fetches: 8
constexpr int kFoldTiles = 4;                 // float32: K tiles summed in one fresh accumulator between folds (64 products)
constexpr size_t kTileBytes = 2 * (size_t)BK * (BM + PAD) * sizeof(float);   // one operand, both buffers
constexpr size_t kLowBytes = (size_t)64 * THREADS * sizeof(float);           // low parts of the compensated totals
template <int DT> constexpr size_t simt_smem_bytes() { return 2 * kTileBytes + (DT == MAGB200_F32 ? kLowBytes : 0); }

// s + e == a + b exactly (s may alias a)
__device__ __forceinline__ void two_sum(float a, float b, float &s, float &e) {
    const float sum = __fadd_rn(a, b);
    const float bp = __fsub_rn(sum, a);
    e = __fadd_rn(__fsub_rn(a, __fsub_rn(sum, bp)), __fsub_rn(b, bp));
    s = sum;
}

// total + low, except that an infinite total stays infinite: TwoSum of an infinity leaves NaN in the low part
// (inf - inf), which must not turn a legitimately infinite product sum into NaN.
__device__ __forceinline__ float fold_low(float total, float low) {
    return (fabsf(total) == __int_as_float(0x7F800000)) ? total : __fadd_rn(total, low);
}

// AKF: the A tile is fetched walking k fastest (else m fastest); BNF: the B tile walking n fastest (else k fastest).
// Compile-time modes make every shared-memory offset of the fetch a constant.
template <int DT, bool AKF, bool BNF>
__global__ void __launch_bounds__(THREADS, 1)
gemm_simt_kernel(const GemmProblem p, int64_t tiles_m, int64_t tiles_n, int nsplit, int64_t kchunk, float *__restrict__ partial,
                 int *run_if_set) {
    // Stand-by launch behind the split-operand tensor-core kernel: runs only when the split pass raised the word. The word
    // is lowered again by the last CTA of this launch to finish (run_if_set[1] counts them), by which time every CTA of
    // both kernels has read it, so the next call finds it clear without a memset of its own.
    if (run_if_set) {
        asm volatile("griddepcontrol.wait;" ::: "memory");          // launched as a programmatic dependent of the tensor-core kernel
        if (*reinterpret_cast<volatile int *>(run_if_set) == 0) return;
    }
    extern __shared__ __align__(16) unsigned char simt_smem[];
    typedef float Tile[BK][BM + PAD];
    Tile *As = reinterpret_cast<Tile *>(simt_smem);                   // As[2][BK][BM + PAD]
    Tile *Bs = reinterpret_cast<Tile *>(simt_smem + kTileBytes);      // Bs[2][BK][BN + PAD]
    float4 *low_s = reinterpret_cast<float4 *>(simt_smem + 2 * kTileBytes) + threadIdx.x;   // slot g of this thread: low_s[g * THREADS]

    const int64_t tiles_per_batch = tiles_m * tiles_n;
    const int64_t tiles_total = tiles_per_batch * p.batch_total;
    const int split = (int)((int64_t)blockIdx.x / tiles_total);
    const int64_t tile = (int64_t)blockIdx.x - (int64_t)split * tiles_total;
    const int64_t batch = tile / tiles_per_batch;
    const int64_t trem = tile - batch * tiles_per_batch;
    const int64_t tm = trem / tiles_n, tn = trem - tm * tiles_n;
    const int64_t m0 = tm * BM, n0 = tn * BN;
    const int64_t kbeg = (int64_t)split * kchunk;
    const int64_t kend = (kbeg + kchunk < p.K) ? kbeg + kchunk : p.K;

    // batch index -> operand offsets; broadcast dims carry stride 0
    int64_t offA = 0, offB = 0;
    {
        int64_t rem = batch;
        for (int d = p.nbatch - 1; d >= 0; --d) {
            int64_t q = rem / p.bshape[d];
            int64_t idx = rem - q * p.bshape[d];
            offA += idx * p.bsA[d];
            offB += idx * p.bsB[d];
            rem = q;
        }
    }
    const int t = threadIdx.x;
    const int lane = t & 31, warp = t >> 5;
    const int tx = (warp & 1) * 8 + (lane & 7);    // column group: columns tx*4 .. +3 and 64 + tx*4 .. +3
    const int ty = (warp >> 1) * 4 + (lane >> 3);  // row group: rows ty*4 .. +3 and 64 + ty*4 .. +3

    // ---- what this thread fetches of every K tile: kLoads elements of A and of B. One coordinate is fixed per thread,
    // the other advances by a constant, so the elements sit at pointer + i * step, a K tile later adds BK * stride, and
    // the row/column bounds are tested once (a bit per element); only the last K tile tests k.
    constexpr int a_dk = AKF ? 0 : THREADS / 128, a_dm = AKF ? THREADS / 16 : 0;
    constexpr int b_dk = BNF ? THREADS / 128 : 0, b_dn = BNF ? 0 : THREADS / 16;
    const int a_kk = AKF ? (t & 15) : (t >> 7), a_mm = AKF ? (t >> 4) : (t & 127);
    const int b_kk = BNF ? (t >> 7) : (t & 15), b_nn = BNF ? (t & 127) : (t >> 4);
    constexpr int64_t es = (DT == MAGB200_F32) ? 4 : 2;
    const char *pa = (const char *)p.A + (offA + (m0 + a_mm) * p.sAm + (kbeg + a_kk) * p.sAk) * es;
    const char *pb = (const char *)p.B + (offB + (kbeg + b_kk) * p.sBk + (n0 + b_nn) * p.sBn) * es;
    const int64_t a_step = ((int64_t)a_dm * p.sAm + (int64_t)a_dk * p.sAk) * es;
    const int64_t b_step = ((int64_t)b_dk * p.sBk + (int64_t)b_dn * p.sBn) * es;
    const int64_t a_tile = (int64_t)BK * p.sAk * es, b_tile = (int64_t)BK * p.sBk * es;
    unsigned in_a = 0, in_b = 0;
#pragma unroll
    for (int i = 0; i < kLoads; ++i) {
        if (m0 + a_mm + i * a_dm < p.M) in_a |= 1u << i;
        if (n0 + b_nn + i * b_dn < p.N) in_b |= 1u << i;
    }

    float ra[kLoads], rb[kLoads];
    auto fetch = [&](int64_t k0, bool tail) {
        const char *qa = pa, *qb = pb;
#pragma unroll
        for (int i = 0; i < kLoads; ++i) {
            bool okA = (in_a >> i) & 1u, okB = (in_b >> i) & 1u;
            if (tail) {
                okA = okA && (k0 + a_kk + i * a_dk < kend);
                okB = okB && (k0 + b_kk + i * b_dk < kend);
            }
            ra[i] = okA ? load_as_f32<DT>(qa, 0) : 0.f;
            rb[i] = okB ? load_as_f32<DT>(qb, 0) : 0.f;
            qa += a_step;
            qb += b_step;
        }
        pa += a_tile;
        pb += b_tile;
    };
    float *const sa = &As[0][a_kk][a_mm];
    float *const sb = &Bs[0][b_kk][b_nn];
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < kLoads; ++i) {
            sa[buf * (BK * (BM + PAD)) + i * (a_dk * (BM + PAD) + a_dm)] = ra[i];
            sb[buf * (BK * (BN + PAD)) + i * (b_dk * (BN + PAD) + b_dn)] = rb[i];
        }
    };

    constexpr bool kCompensated = (DT == MAGB200_F32);
    float acc[8][8];                                   // sum of the current group of K tiles (fp32) or of all of K (16-bit)
    float total[kCompensated ? 8 : 1][8];              // fp32: running totals; their lost low parts sit in low_s
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            acc[i][j] = 0.f;
            if constexpr (kCompensated) total[i][j] = 0.f;
        }
    if constexpr (kCompensated) {
#pragma unroll
        for (int g = 0; g < 16; ++g) low_s[g * THREADS] = make_float4(0.f, 0.f, 0.f, 0.f);
    }

    int buf = 0;
    int since_fold = 0;
    if (kbeg < kend) {
        fetch(kbeg, true);
        stash(0);
    }
    __syncthreads();
    for (int64_t k0 = kbeg; k0 < kend; k0 += BK) {
        const bool more = k0 + BK < kend;
        if (more) fetch(k0 + BK, k0 + 2 * BK > kend);   // global loads in flight under the multiply below
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[8], b[8];
            *reinterpret_cast<float4 *>(&a[0]) = *reinterpret_cast<const float4 *>(&As[buf][kk][ty * 4]);
            *reinterpret_cast<float4 *>(&a[4]) = *reinterpret_cast<const float4 *>(&As[buf][kk][64 + ty * 4]);
            *reinterpret_cast<float4 *>(&b[0]) = *reinterpret_cast<const float4 *>(&Bs[buf][kk][tx * 4]);
            *reinterpret_cast<float4 *>(&b[4]) = *reinterpret_cast<const float4 *>(&Bs[buf][kk][64 + tx * 4]);
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if constexpr (kCompensated) {
            if (++since_fold == kFoldTiles || !more) {
                since_fold = 0;
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float4 lo = low_s[(i * 2 + h) * THREADS];
                        float e0, e1, e2, e3;
                        two_sum(total[i][h * 4 + 0], acc[i][h * 4 + 0], total[i][h * 4 + 0], e0);
                        two_sum(total[i][h * 4 + 1], acc[i][h * 4 + 1], total[i][h * 4 + 1], e1);
                        two_sum(total[i][h * 4 + 2], acc[i][h * 4 + 2], total[i][h * 4 + 2], e2);
                        two_sum(total[i][h * 4 + 3], acc[i][h * 4 + 3], total[i][h * 4 + 3], e3);
                        lo.x = __fadd_rn(lo.x, e0);
                        lo.y = __fadd_rn(lo.y, e1);
                        lo.z = __fadd_rn(lo.z, e2);
                        lo.w = __fadd_rn(lo.w, e3);
                        low_s[(i * 2 + h) * THREADS] = lo;
                        acc[i][h * 4 + 0] = acc[i][h * 4 + 1] = acc[i][h * 4 + 2] = acc[i][h * 4 + 3] = 0.f;
                    }
            }
        }
        if (more) stash(buf ^ 1);                      // the other buffer: nobody reads it during this tile
        __syncthreads();
        buf ^= 1;
    }

    // ---- epilogue: row-major C with ldc = N; one rounding to the result dtype, or the (total, low) pair of this K split
    char *C = (char *)p.C;
    const int64_t cbase = batch * p.M * p.N;
    const int64_t elems = p.batch_total * p.M * p.N;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int64_t gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (gm >= p.M) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float lo4[4] = {0.f, 0.f, 0.f, 0.f};
            if constexpr (kCompensated) *reinterpret_cast<float4 *>(lo4) = low_s[(i * 2 + h) * THREADS];
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const int j = h * 4 + jj;
                const int64_t gn = n0 + h * 64 + tx * 4 + jj;
                if (gn >= p.N) continue;
                const int64_t idx = cbase + gm * p.N + gn;
                float hi = acc[i][j];
                if constexpr (kCompensated) hi = total[i][j];
                if (nsplit == 1) {
                    store_from_f32<DT>(C, idx, kCompensated ? fold_low(hi, lo4[jj]) : hi);
                } else {
                    partial[((int64_t)split * 2 + 0) * elems + idx] = hi;
                    partial[((int64_t)split * 2 + 1) * elems + idx] = lo4[jj];
                }
            }
        }
    }
    if (run_if_set) {
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(run_if_set + 1, 1) == (int)gridDim.x - 1) {
                run_if_set[1] = 0;
                run_if_set[0] = 0;
                __threadfence();
            }
        }
    }
}

// partial[nsplit][2][elems] -> C[elems]: the splits' (total, low) pairs added in split order without losing the low parts
template <int DT>
__global__ void __launch_bounds__(256) simt_finalize_kernel(const float *__restrict__ partial, void *__restrict__ C, int64_t elems, int nsplit) {
    const int64_t stride = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < elems; i += stride) {
        float total = partial[i], low = partial[elems + i];
        for (int s = 1; s < nsplit; ++s) {
            float sum, e;
            two_sum(total, partial[((int64_t)s * 2) * elems + i], sum, e);
            total = sum;
            low = __fadd_rn(low, __fadd_rn(e, partial[((int64_t)s * 2 + 1) * elems + i]));
        }
        store_from_f32<DT>(C, i, fold_low(total, low));
    }
}

// More than 48 KB of dynamic shared memory needs an opt-in per (kernel, device): bit d of `done` is set once device d has it.
template <typename K>
int simt_smem_optin(K kernel, size_t bytes, std::atomic<uint32_t> &done) {
    if (bytes <= 48 * 1024) return MAGB200_OK;
    int dev = 0;
    MAGB200_CUDA_TRY(cudaGetDevice(&dev));
    const uint32_t bit = 1u << (dev & 31);
    if (!(done.load(std::memory_order_acquire) & bit)) {
        MAGB200_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        done.fetch_or(bit, std::memory_order_release);
    }
    return MAGB200_OK;
}

struct SimtPlan { int64_t tiles_m, tiles_n, tiles; int nsplit; int64_t kchunk; };

SimtPlan plan_simt(const GemmProblem &p) {
    SimtPlan pl;
    pl.tiles_m = (p.M + BM - 1) / BM;
    pl.tiles_n = (p.N + BN - 1) / BN;
    pl.tiles = pl.tiles_m * pl.tiles_n * p.batch_total;
    pl.nsplit = 1;
    // an output smaller than the GPU: cut K so that about one CTA per SM is busy, never below 256 K values per CTA
    if (pl.tiles > 0 && pl.tiles * 2 <= num_sms() && p.K >= 512) {
        int64_t s = num_sms() / pl.tiles;
        if (s > p.K / 256) s = p.K / 256;
        if (s > 16) s = 16;
        if (s > 1) pl.nsplit = (int)s;
    }
    const int64_t kb = (p.K + BK - 1) / BK;
    pl.kchunk = ((kb + pl.nsplit - 1) / pl.nsplit) * BK;
    if (pl.kchunk < BK) pl.kchunk = BK;
    while (pl.nsplit > 1 && (int64_t)(pl.nsplit - 1) * pl.kchunk >= p.K) --pl.nsplit;   // no empty split
    return pl;
}

}  // namespace

size_t simt_scratch_bytes(const GemmProblem &p) {
    const SimtPlan pl = plan_simt(p);
    return pl.nsplit > 1 ? (size_t)pl.nsplit * 2 * (size_t)(p.batch_total * p.M * p.N) * sizeof(float) : 0;
}

int launch_gemm_simt(const GemmProblem &p, cudaStream_t stream, float *scratch, size_t scratch_bytes, int *run_if_set) {
    SimtPlan pl = plan_simt(p);
    if (pl.tiles <= 0) return MAGB200_OK;
    if (run_if_set) scratch = nullptr;                // the stand-by form never splits K: its finalize pass would be unconditional
    if (pl.nsplit > 1 && (!scratch || scratch_bytes < simt_scratch_bytes(p))) {   // no workspace: one CTA walks all of K
        pl.nsplit = 1;
        pl.kchunk = ((p.K + BK - 1) / BK) * BK;
        if (pl.kchunk < BK) pl.kchunk = BK;
    }
    const int64_t grid = pl.tiles * pl.nsplit;
    if (grid > 0x7FFFFFFFLL) {
        set_error("matmul: %lld tiles exceed the grid limit", (long long)grid);
        return MAGB200_ERR_TOO_LARGE;
    }
    const int64_t elems = p.batch_total * p.M * p.N;
    int64_t fin_blocks = (elems + 255) / 256;
    if (fin_blocks > num_sms() * 8) fin_blocks = num_sms() * 8;
    const bool akf = (p.sAk == 1) || (p.sAm != 1);   // walk k fastest unless m is the unit-stride dim
    const bool bnf = (p.sBn == 1) || (p.sBk != 1);
#define MAGB200_SIMT_GO(DT, AKF, BNF)                                                                        \
    do {                                                                                                     \
        static std::atomic<uint32_t> optin{0};                                                               \
        if (int rc = simt_smem_optin(gemm_simt_kernel<DT, AKF, BNF>, simt_smem_bytes<DT>(), optin)) return rc; \
        cudaLaunchConfig_t cfg;                                                                              \
        memset(&cfg, 0, sizeof(cfg));                                                                        \
        cfg.gridDim = dim3((unsigned)grid, 1, 1); cfg.blockDim = dim3(THREADS, 1, 1);                        \
        cfg.dynamicSmemBytes = simt_smem_bytes<DT>(); cfg.stream = stream;                                   \
        cudaLaunchAttribute attr[1];                                                                         \
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                                     \
        attr[0].val.programmaticStreamSerializationAllowed = 1;                                              \
        cfg.attrs = attr; cfg.numAttrs = run_if_set ? 1 : 0;                                                 \
        MAGB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_simt_kernel<DT, AKF, BNF>, p, pl.tiles_m, pl.tiles_n, pl.nsplit, pl.kchunk, \
                                            scratch, run_if_set));                                           \
    } while (0)
#define MAGB200_SIMT_LAUNCH(DT)                                                                              \
    if (akf) { if (bnf) MAGB200_SIMT_GO(DT, true, true); else MAGB200_SIMT_GO(DT, true, false); }            \
    else     { if (bnf) MAGB200_SIMT_GO(DT, false, true); else MAGB200_SIMT_GO(DT, false, false); }          \
    if (pl.nsplit > 1) {                                                                                     \
        count_launch();                                                                                      \
        simt_finalize_kernel<DT><<<(unsigned)fin_blocks, 256, 0, stream>>>(scratch, p.C, elems, pl.nsplit);  \
    }
    switch (p.dtype) {
        case MAGB200_F32:  MAGB200_SIMT_LAUNCH(MAGB200_F32) break;
        case MAGB200_F16:  MAGB200_SIMT_LAUNCH(MAGB200_F16) break;
        case MAGB200_BF16: MAGB200_SIMT_LAUNCH(MAGB200_BF16) break;
        default: set_error("matmul: unsupported dtype %d", p.dtype); return MAGB200_ERR_INVALID_ARG;
    }
#undef MAGB200_SIMT_GO
#undef MAGB200_SIMT_LAUNCH
    count_launch();
    MAGB200_CUDA_TRY(cudaGetLastError());
    return MAGB200_OK;
}

}  // namespace magb200
