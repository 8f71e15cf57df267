// Exact-fp32 tiled FFMA matmul for arbitrary element strides.
//
// Role on the path: (1) the float32 matmul -- tensor cores only offer TF32 inputs (10-bit mantissa),
// which cannot hold the reference's fp32 accuracy, so fp32 products run on the FP32 pipes and are
// bounded by the FFMA roofline, not the tensor roofline; (2) 16-bit operands whose layout TMA cannot
// describe (an inner stride that is not 1 on either of the last two dims, a row pitch that is not a
// multiple of 16 bytes, a misaligned base). Operands are gathered through their strides straight into
// shared memory as fp32, so no packed copy of a strided view is ever made in HBM.
//
// Tile: 128x128x16 per 256-thread CTA, 8x8 accumulators per thread held as 2x2 blocks of 4x4 so the
// shared-memory reads are conflict-free 128-bit loads.
//
// fp32 accuracy: a single fp32 accumulator that walks the whole K loses several units in the last place
// at K in the thousands, more than the reference's blocked CPU kernel does. For float32 the kernel
// therefore sums each 16-wide K tile in a fresh accumulator and folds it into the running total with an
// error-free TwoSum, carrying the lost low part along; what remains is the rounding inside one 16-term
// tile. The 16-bit dtypes skip this: their error is set by the final rounding of the result.
#include "common.cuh"

namespace magb200 {

namespace {

constexpr int BM = 128, BN = 128, BK = 16, THREADS = 256, PAD = 4;

template <int DT>
__global__ void __launch_bounds__(THREADS, 1) gemm_simt_kernel(const GemmProblem p, int64_t tiles_m, int64_t tiles_n) {
    __shared__ __align__(16) float As[BK][BM + PAD];
    __shared__ __align__(16) float Bs[BK][BN + PAD];

    const int64_t tile = blockIdx.x;
    const int64_t tiles_per_batch = tiles_m * tiles_n;
    const int64_t batch = tile / tiles_per_batch;
    const int64_t trem = tile - batch * tiles_per_batch;
    const int64_t tm = trem / tiles_n, tn = trem - tm * tiles_n;
    const int64_t m0 = tm * BM, n0 = tn * BN;

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
    const char *A = (const char *)p.A;
    const char *B = (const char *)p.B;
    const int t = threadIdx.x;
    const int tx = t & 15, ty = t >> 4;

    constexpr bool kCompensated = (DT == MAGB200_F32);
    float acc[8][8];                                   // sum of the current K tile (fp32) or of all of K (16-bit)
    float total[kCompensated ? 8 : 1][8], low[kCompensated ? 8 : 1][8];  // running total and its lost low part
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            acc[i][j] = 0.f;
            if constexpr (kCompensated) { total[i][j] = 0.f; low[i][j] = 0.f; }
        }

    const bool a_k_fast = (p.sAk == 1) || (p.sAm != 1);  // walk k fastest unless m is the unit-stride dim
    const bool b_n_fast = (p.sBn == 1) || (p.sBk != 1);

    for (int64_t k0 = 0; k0 < p.K; k0 += BK) {
        // ---- gather the A tile (BM x BK) and the B tile (BK x BN) as fp32 ----
#pragma unroll
        for (int i = 0; i < (BM * BK) / THREADS; ++i) {
            int e = t + i * THREADS;
            int kk, mm;
            if (a_k_fast) { kk = e & (BK - 1); mm = e >> 4; } else { mm = e & (BM - 1); kk = e >> 7; }
            int64_t gm = m0 + mm, gk = k0 + kk;
            float v = 0.f;
            if (gm < p.M && gk < p.K) v = load_as_f32<DT>(A, offA + gm * p.sAm + gk * p.sAk);
            As[kk][mm] = v;
        }
#pragma unroll
        for (int i = 0; i < (BN * BK) / THREADS; ++i) {
            int e = t + i * THREADS;
            int kk, nn;
            if (b_n_fast) { nn = e & (BN - 1); kk = e >> 7; } else { kk = e & (BK - 1); nn = e >> 4; }
            int64_t gn = n0 + nn, gk = k0 + kk;
            float v = 0.f;
            if (gn < p.N && gk < p.K) v = load_as_f32<DT>(B, offB + gk * p.sBk + gn * p.sBn);
            Bs[kk][nn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[8], b[8];
            *reinterpret_cast<float4 *>(&a[0]) = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
            *reinterpret_cast<float4 *>(&a[4]) = *reinterpret_cast<const float4 *>(&As[kk][64 + ty * 4]);
            *reinterpret_cast<float4 *>(&b[0]) = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
            *reinterpret_cast<float4 *>(&b[4]) = *reinterpret_cast<const float4 *>(&Bs[kk][64 + tx * 4]);
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if constexpr (kCompensated) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    // TwoSum: s + e == total + acc exactly
                    const float s = __fadd_rn(total[i][j], acc[i][j]);
                    const float bp = __fsub_rn(s, total[i][j]);
                    const float e = __fadd_rn(__fsub_rn(total[i][j], __fsub_rn(s, bp)), __fsub_rn(acc[i][j], bp));
                    total[i][j] = s;
                    low[i][j] = __fadd_rn(low[i][j], e);
                    acc[i][j] = 0.f;
                }
        }
        __syncthreads();
    }
    if constexpr (kCompensated) {
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] = __fadd_rn(total[i][j], low[i][j]);
    }

    // ---- epilogue: one rounding to the result dtype, row-major C with ldc = N ----
    char *C = (char *)p.C;
    const int64_t cbase = batch * p.M * p.N;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        int64_t gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (gm >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            int64_t gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (gn < p.N) store_from_f32<DT>(C, cbase + gm * p.N + gn, acc[i][j]);
        }
    }
}

}  // namespace

int launch_gemm_simt(const GemmProblem &p, cudaStream_t stream) {
    const int64_t tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
    const int64_t total = tiles_m * tiles_n * p.batch_total;
    if (total <= 0) return MAGB200_OK;
    if (total > 0x7FFFFFFFLL) {
        set_error("matmul: %lld tiles exceed the grid limit", (long long)total);
        return MAGB200_ERR_TOO_LARGE;
    }
    switch (p.dtype) {
        case MAGB200_F32:  gemm_simt_kernel<MAGB200_F32><<<(unsigned)total, THREADS, 0, stream>>>(p, tiles_m, tiles_n); break;
        case MAGB200_F16:  gemm_simt_kernel<MAGB200_F16><<<(unsigned)total, THREADS, 0, stream>>>(p, tiles_m, tiles_n); break;
        case MAGB200_BF16: gemm_simt_kernel<MAGB200_BF16><<<(unsigned)total, THREADS, 0, stream>>>(p, tiles_m, tiles_n); break;
        default: set_error("matmul: unsupported dtype %d", p.dtype); return MAGB200_ERR_INVALID_ARG;
    }
    count_launch();
    MAGB200_CUDA_TRY(cudaGetLastError());
    return MAGB200_OK;
}

}  // namespace magb200
