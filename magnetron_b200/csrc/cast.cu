// Streaming dtype conversion kernels for {f32, f16, bf16} (MAG_OP_CAST, MAG_OP_CLONE, MAG_OP_FILL).
//
// HBM-bound: a contiguous cast moves sizeof(src)+sizeof(dst) bytes per element and does a handful of
// integer ops. Each thread converts 8 elements per step with 128-bit loads and stores that bypass L1
// (ld.global.cs / st.global.cs: streaming, evict-first), the grid is a multiple of the SM count, and
// the conversions are the integer formulas of common.cuh so every NaN pattern matches the reference.
#include "common.cuh"

namespace magb200 {

namespace {

constexpr int kThreads = 256;
constexpr int kVec = 8;  // elements per thread per step

template <int S, int D> __device__ __forceinline__ uint32_t convert_bits(uint32_t v);
template <> __device__ __forceinline__ uint32_t convert_bits<MAGB200_F32, MAGB200_F32>(uint32_t v) { return v; }
template <> __device__ __forceinline__ uint32_t convert_bits<MAGB200_F16, MAGB200_F16>(uint32_t v) { return v; }
template <> __device__ __forceinline__ uint32_t convert_bits<MAGB200_BF16, MAGB200_BF16>(uint32_t v) { return v; }
template <> __device__ __forceinline__ uint32_t convert_bits<MAGB200_F32, MAGB200_BF16>(uint32_t v) { return f32_bits_to_bf16_bits(v); }
template <> __device__ __forceinline__ uint32_t convert_bits<MAGB200_F32, MAGB200_F16>(uint32_t v) { return f32_bits_to_f16_bits(v); }
template <> __device__ __forceinline__ uint32_t convert_bits<MAGB200_BF16, MAGB200_F32>(uint32_t v) { return bf16_bits_to_f32_bits(v); }
template <> __device__ __forceinline__ uint32_t convert_bits<MAGB200_F16, MAGB200_F32>(uint32_t v) { return f16_bits_to_f32_bits(v); }
// 16-bit <-> 16-bit pairs go through fp32 exactly like the reference's cast table.
template <> __device__ __forceinline__ uint32_t convert_bits<MAGB200_F16, MAGB200_BF16>(uint32_t v) {
    return f32_bits_to_bf16_bits(f16_bits_to_f32_bits(v));
}
template <> __device__ __forceinline__ uint32_t convert_bits<MAGB200_BF16, MAGB200_F16>(uint32_t v) {
    return f32_bits_to_f16_bits(bf16_bits_to_f32_bits(v));
}

template <int DT> struct Bits { using type = uint16_t; };
template <> struct Bits<MAGB200_F32> { using type = uint32_t; };

// Loads 8 source elements as raw bit patterns into v[8].
template <int S> __device__ __forceinline__ void load8(const void *src, int64_t i, uint32_t (&v)[kVec]) {
    if constexpr (S == MAGB200_F32) {
        const uint4 *p = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint32_t *>(src) + i);
        uint4 a = __ldcs(p), b = __ldcs(p + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
        uint4 a = __ldcs(reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(src) + i));
        v[0] = a.x & 0xFFFFu; v[1] = a.x >> 16; v[2] = a.y & 0xFFFFu; v[3] = a.y >> 16;
        v[4] = a.z & 0xFFFFu; v[5] = a.z >> 16; v[6] = a.w & 0xFFFFu; v[7] = a.w >> 16;
    }
}
template <int D> __device__ __forceinline__ void store8(void *dst, int64_t i, const uint32_t (&v)[kVec]) {
    if constexpr (D == MAGB200_F32) {
        uint4 *p = reinterpret_cast<uint4 *>(reinterpret_cast<uint32_t *>(dst) + i);
        __stcs(p, make_uint4(v[0], v[1], v[2], v[3]));
        __stcs(p + 1, make_uint4(v[4], v[5], v[6], v[7]));
    } else {
        uint4 o = make_uint4(v[0] | (v[1] << 16), v[2] | (v[3] << 16), v[4] | (v[5] << 16), v[6] | (v[7] << 16));
        __stcs(reinterpret_cast<uint4 *>(reinterpret_cast<uint16_t *>(dst) + i), o);
    }
}

// Contiguous source and destination, both 16-byte aligned. n8 = number of full 8-element groups.
template <int S, int D>
__global__ void __launch_bounds__(kThreads) cast_contig_kernel(const void *__restrict__ src, void *__restrict__ dst, int64_t n) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // an independent kernel behind this one may start as SMs come free
    const int64_t n8 = n / kVec;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    // kUnroll groups per thread and step, all loads issued before the first store: a 16-bit source brings only 16 bytes per
    // group, so one group per step left too few bytes in flight to cover the DRAM latency (bf16 -> fp32 ran at 0.74 of the
    // copy bandwidth against 0.82 for fp32 -> bf16)
    constexpr int kUnroll = 4;
    int64_t g = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    for (; g + (kUnroll - 1) * stride < n8; g += kUnroll * stride) {
        uint32_t v[kUnroll][kVec];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) load8<S>(src, (g + u * stride) * kVec, v[u]);
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
#pragma unroll
            for (int j = 0; j < kVec; ++j) v[u][j] = convert_bits<S, D>(v[u][j]);
            store8<D>(dst, (g + u * stride) * kVec, v[u]);
        }
    }
    for (; g < n8; g += stride) {
        uint32_t v[kVec];
        load8<S>(src, g * kVec, v);
#pragma unroll
        for (int j = 0; j < kVec; ++j) v[j] = convert_bits<S, D>(v[j]);
        store8<D>(dst, g * kVec, v);
    }
    // ragged tail (< 8 elements): first threads of block 0
    if (blockIdx.x == 0) {
        int64_t i = n8 * kVec + threadIdx.x;
        if (i < n) {
            uint32_t v = reinterpret_cast<const typename Bits<S>::type *>(src)[i];
            reinterpret_cast<typename Bits<D>::type *>(dst)[i] = (typename Bits<D>::type)convert_bits<S, D>(v);
        }
    }
}

// 16-bit -> fp32, contiguous and aligned: four elements per thread and group (one 8-byte load, one 16-byte store), so
// that the lanes of a warp write 512 contiguous bytes per store instruction instead of 16 bytes every 32; eight groups in
// flight per thread. This direction writes two bytes for every byte it reads and is bound by the write stream.
template <int S>
__global__ void __launch_bounds__(kThreads) cast_widen_kernel(const void *__restrict__ src, void *__restrict__ dst, int64_t n) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int kU = 8;
    const int64_t n4 = n / 4;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const uint2 *in = reinterpret_cast<const uint2 *>(src);
    uint4 *out = reinterpret_cast<uint4 *>(dst);
    int64_t g = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    for (; g + (kU - 1) * stride < n4; g += kU * stride) {
        uint2 v[kU];
#pragma unroll
        for (int u = 0; u < kU; ++u) v[u] = __ldcs(in + g + u * stride);
#pragma unroll
        for (int u = 0; u < kU; ++u)
            __stcs(out + g + u * stride, make_uint4(convert_bits<S, MAGB200_F32>(v[u].x & 0xFFFFu), convert_bits<S, MAGB200_F32>(v[u].x >> 16),
                                                    convert_bits<S, MAGB200_F32>(v[u].y & 0xFFFFu), convert_bits<S, MAGB200_F32>(v[u].y >> 16)));
    }
    for (; g < n4; g += stride) {
        const uint2 v = __ldcs(in + g);
        __stcs(out + g, make_uint4(convert_bits<S, MAGB200_F32>(v.x & 0xFFFFu), convert_bits<S, MAGB200_F32>(v.x >> 16),
                                   convert_bits<S, MAGB200_F32>(v.y & 0xFFFFu), convert_bits<S, MAGB200_F32>(v.y >> 16)));
    }
    if (blockIdx.x == 0) {                       // ragged tail (< 4 elements)
        const int64_t i = n4 * 4 + threadIdx.x;
        if (i < n) reinterpret_cast<uint32_t *>(dst)[i] = convert_bits<S, MAGB200_F32>(reinterpret_cast<const uint16_t *>(src)[i]);
    }
}

// Arbitrary strided source (collapsed dims), contiguous destination. One element per thread-step;
// consecutive threads take consecutive destination elements, so stores stay coalesced and loads are
// coalesced whenever the innermost collapsed stride is 1.
template <int S, int D>
__global__ void __launch_bounds__(kThreads) cast_strided_kernel(const void *__restrict__ src, void *__restrict__ dst,
                                                                int64_t n, CollapsedDims dims) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
        int64_t rem = i, off = 0;
#pragma unroll 1
        for (int d = dims.rank - 1; d >= 0; --d) {
            int64_t q = rem / dims.shape[d];
            off += (rem - q * dims.shape[d]) * dims.strides[d];
            rem = q;
        }
        uint32_t v = reinterpret_cast<const typename Bits<S>::type *>(src)[off];
        reinterpret_cast<typename Bits<D>::type *>(dst)[i] = (typename Bits<D>::type)convert_bits<S, D>(v);
    }
}

template <int DT>
__global__ void __launch_bounds__(kThreads) fill_kernel(void *__restrict__ dst, int64_t n, uint32_t bits) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride)
        reinterpret_cast<typename Bits<DT>::type *>(dst)[i] = (typename Bits<DT>::type)bits;
}

// Copy of one 16-bit matmul operand into rows of unit K stride and a pitch of `kpad` elements (a multiple of 8: 16 bytes), for
// operands whose own layout TMA cannot describe (odd pitch, inner stride 2, misaligned slice). One CTA per (batch, row) pair,
// threads along K, so the writes are coalesced whatever the source strides are. Broadcast batch dims (stride 0) are not
// replicated: the packed operand keeps stride 0 there.
struct PackArgs {
    const uint16_t *src;
    uint16_t *dst;
    int64_t rows, K, kpad;
    int64_t s_row, s_k;                  // source strides of the row and K dims (elements)
    int nbatch;
    int64_t bshape[kMaxBatchDims], bsrc[kMaxBatchDims], bdst[kMaxBatchDims];   // packed batch extents (1 where broadcast) and strides
    int64_t total_rows;                  // rows * product of packed batch extents
};
__global__ void __launch_bounds__(kThreads) pack_operand_kernel(const PackArgs a) {
    for (int64_t id = blockIdx.x; id < a.total_rows; id += gridDim.x) {
        const int64_t row = id % a.rows;
        int64_t rem = id / a.rows, so = row * a.s_row, dof = row * a.kpad;
        for (int d = a.nbatch - 1; d >= 0; --d) {
            const int64_t q = rem / a.bshape[d], idx = rem - q * a.bshape[d];
            so += idx * a.bsrc[d];
            dof += idx * a.bdst[d];
            rem = q;
        }
        // eight K values per thread: eight 2-byte loads (the source may be anything), one 16-byte store (the packed row is aligned)
        for (int64_t k0 = (int64_t)threadIdx.x * 8; k0 < a.kpad; k0 += (int64_t)kThreads * 8) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int64_t ka = k0 + 2 * j, kb = ka + 1;
                const uint32_t lo = ka < a.K ? a.src[so + ka * a.s_k] : 0u, hi = kb < a.K ? a.src[so + kb * a.s_k] : 0u;
                w[j] = lo | (hi << 16);
            }
            *reinterpret_cast<uint4 *>(a.dst + dof + k0) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

// ---- fp32 operand -> three bf16 planes (hi, mid, lo with hi + mid + lo == value to 24 bits) -------------------------------
// An operand whose K stride is 1 is read four K values per thread (one 16-byte load where the alignment allows) and written
// as three 8-byte stores, four such groups in flight per thread. An operand whose rows have the unit stride (a [K, N] weight)
// goes through shared memory in tiles of 32 rows x 64 K values, so the reads walk the rows and the writes walk K. Both
// operands of a product are split by one launch; a work unit is 1024 groups of four or one tile.
struct SplitOperand {
    const float *src;
    uint16_t *dst;
    int64_t rows, K, kpad;
    int64_t s_row, s_k;                  // source strides (elements)
    int nbatch;
    int64_t bshape[kMaxBatchDims], bsrc[kMaxBatchDims], bdst[kMaxBatchDims];   // packed batch extents (1 where broadcast) and strides
    int64_t row_tiles, k_tiles, units;
    int64_t quads_per_row, quads;        // groups of four K values per row (kpad / 4) and in the whole operand
    int k_fast;                          // 1: K has the unit stride (direct path), 0: tiles through shared memory
    int vec4;                            // direct path: rows start 16-byte aligned and K % 4 == 0
};
struct SplitArgs {
    SplitOperand op[2];
    int *unsafe;
};
__device__ __forceinline__ void split3(float v, uint32_t &hi, uint32_t &mid, uint32_t &lo) {
    hi = f32_bits_to_bf16_bits(__float_as_uint(v));
    const float r1 = __fsub_rn(v, __uint_as_float(hi << 16));          // exact: the difference fits in 24 bits
    mid = f32_bits_to_bf16_bits(__float_as_uint(r1));
    const float r2 = __fsub_rn(r1, __uint_as_float(mid << 16));
    lo = f32_bits_to_bf16_bits(__float_as_uint(r2));
}
__device__ __forceinline__ bool unsafe_to_split(float v) {
    const uint32_t a = __float_as_uint(v) & 0x7FFFFFFFu;
    // not finite or rounds to a bf16 infinity; or non-zero below 2^-100, where the lower planes leave the normal range
    return a >= 0x7F7F8000u || (a != 0u && a < (27u << 23));
}
__device__ __forceinline__ void batch_offsets(const SplitOperand &o, int64_t rem, int64_t &so, int64_t &dof) {
    so = 0; dof = 0;
    for (int d = o.nbatch - 1; d >= 0; --d) {
        const int64_t q = rem / o.bshape[d], idx = rem - q * o.bshape[d];
        so += idx * o.bsrc[d];
        dof += idx * o.bdst[d];
        rem = q;
    }
}
__global__ void __launch_bounds__(kThreads) split3_kernel(const SplitArgs a) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // the GEMM behind this pass may set itself up meanwhile (it waits before it reads)
    __shared__ float tile[32][65];
    const int t = threadIdx.x;
    bool bad = false;
    const int64_t total = a.op[0].units + a.op[1].units;
    for (int64_t id = blockIdx.x; id < total; id += gridDim.x) {
        const SplitOperand &o = a.op[id >= a.op[0].units ? 1 : 0];
        const int64_t local = id >= a.op[0].units ? id - a.op[0].units : id;
        if (o.k_fast) {
            float4 v[4];
            uint16_t *q[4];
            const int64_t plane = o.rows * o.kpad;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int64_t g = local * 1024 + i * 256 + t;
                q[i] = nullptr;
                v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (g < o.quads) {
                    const int64_t rl = g / o.quads_per_row, kq = g - rl * o.quads_per_row;
                    const int64_t bi = rl / o.rows, row = rl - bi * o.rows;
                    int64_t so, dof;
                    batch_offsets(o, bi, so, dof);
                    const float *src = o.src + so + row * o.s_row + kq * 4;
                    q[i] = o.dst + dof + row * o.kpad + kq * 4;
                    if (o.vec4) {
                        if (kq * 4 < o.K) v[i] = *reinterpret_cast<const float4 *>(src);   // K % 4 == 0: a group is inside the row or past it
                    } else {
                        const int64_t k = kq * 4;
                        if (k < o.K) v[i].x = src[0];
                        if (k + 1 < o.K) v[i].y = src[1];
                        if (k + 2 < o.K) v[i].z = src[2];
                        if (k + 3 < o.K) v[i].w = src[3];
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (!q[i]) continue;
                bad = bad || unsafe_to_split(v[i].x) || unsafe_to_split(v[i].y) || unsafe_to_split(v[i].z) || unsafe_to_split(v[i].w);
                uint32_t h[4], m[4], l[4];
                split3(v[i].x, h[0], m[0], l[0]);
                split3(v[i].y, h[1], m[1], l[1]);
                split3(v[i].z, h[2], m[2], l[2]);
                split3(v[i].w, h[3], m[3], l[3]);
                *reinterpret_cast<uint2 *>(q[i]) = make_uint2(h[0] | (h[1] << 16), h[2] | (h[3] << 16));
                *reinterpret_cast<uint2 *>(q[i] + plane) = make_uint2(m[0] | (m[1] << 16), m[2] | (m[3] << 16));
                *reinterpret_cast<uint2 *>(q[i] + 2 * plane) = make_uint2(l[0] | (l[1] << 16), l[2] | (l[3] << 16));
            }
            continue;
        }
        const int64_t kt = local % o.k_tiles;
        int64_t rem = local / o.k_tiles;
        const int64_t rt = rem % o.row_tiles;
        rem /= o.row_tiles;
        int64_t so, dof;
        batch_offsets(o, rem, so, dof);
        const int64_t r0 = rt * 32, k0 = kt * 64;
        {
            const int rx = t & 31, ky = t >> 5;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int k = ky + 8 * i;
                float v = 0.f;
                if (r0 + rx < o.rows && k0 + k < o.K) v = o.src[so + (r0 + rx) * o.s_row + (k0 + k) * o.s_k];
                bad = bad || unsafe_to_split(v);
                tile[rx][k] = v;
            }
        }
        __syncthreads();
        const int kp = (t & 31) * 2, ry = t >> 5;
        if (k0 + kp < o.kpad) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int r = ry + 8 * i;
                if (r0 + r >= o.rows) continue;
                uint32_t h0, m0, l0, h1, m1, l1;
                split3(tile[r][kp], h0, m0, l0);
                split3(tile[r][kp + 1], h1, m1, l1);
                uint16_t *q = o.dst + dof + (r0 + r) * o.kpad + k0 + kp;
                const int64_t plane = o.rows * o.kpad;
                *reinterpret_cast<uint32_t *>(q) = h0 | (h1 << 16);
                *reinterpret_cast<uint32_t *>(q + plane) = m0 | (m1 << 16);
                *reinterpret_cast<uint32_t *>(q + 2 * plane) = l0 | (l1 << 16);
            }
        }
        __syncthreads();
    }
    if (bad) *a.unsafe = 1;
}

int grid_for(int64_t work_items) {
    int64_t blocks = (work_items + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)num_sms() * 16;  // 16 resident 256-thread blocks cover every SM several times
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

// Grid for a kernel whose threads take `unroll` groups per step with all loads ahead of the stores: as many blocks as give
// every thread one whole step (a thread with fewer groups than `unroll` would fall to the one-at-a-time loop: 16 Mi elements
// on 2368 blocks left each thread 3.5 groups, none of them unrolled), capped at 16 resident blocks per SM.
int grid_for_unrolled(int64_t groups, int unroll) {
    int64_t blocks = (groups + (int64_t)kThreads * unroll - 1) / ((int64_t)kThreads * unroll);
    const int64_t cap = (int64_t)num_sms() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

template <int S, int D>
int launch_pair(const void *src, void *dst, int64_t n, const CollapsedDims &dims, bool contig, cudaStream_t stream, bool overlapped) {
    const bool aligned = (((uintptr_t)src | (uintptr_t)dst) & 15u) == 0;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlapped ? 1 : 0;      // the caller has checked that this cast touches nothing the kernels before it use
    if (contig && aligned && D == MAGB200_F32 && S != MAGB200_F32) {
        if constexpr (D == MAGB200_F32 && S != MAGB200_F32) {
            cfg.gridDim = dim3((unsigned)grid_for_unrolled((n + 3) / 4, 8), 1, 1);
            MAGB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, cast_widen_kernel<S>, src, dst, n));
        }
    } else if (contig && aligned) {
        cfg.gridDim = dim3((unsigned)grid_for_unrolled((n + kVec - 1) / kVec, 4), 1, 1);
        MAGB200_CUDA_TRY(cudaLaunchKernelEx(&cfg, cast_contig_kernel<S, D>, (const void *)src, dst, n));
    } else {
        CollapsedDims d = dims;
        if (contig) { d.rank = 1; d.shape[0] = n; d.strides[0] = 1; }
        cast_strided_kernel<S, D><<<grid_for(n), kThreads, 0, stream>>>(src, dst, n, d);
    }
    count_launch();
    MAGB200_CUDA_TRY(cudaGetLastError());
    return MAGB200_OK;
}

}  // namespace

int launch_cast(int s, int d, const void *src, void *dst, int64_t n, const CollapsedDims &dims, bool contig, cudaStream_t st, bool overlapped) {
    if (n <= 0) return MAGB200_OK;
#define PAIR(SS, DD) if (s == SS && d == DD) return launch_pair<SS, DD>(src, dst, n, dims, contig, st, overlapped);
    PAIR(MAGB200_F32, MAGB200_F32) PAIR(MAGB200_F32, MAGB200_F16) PAIR(MAGB200_F32, MAGB200_BF16)
    PAIR(MAGB200_F16, MAGB200_F32) PAIR(MAGB200_F16, MAGB200_F16) PAIR(MAGB200_F16, MAGB200_BF16)
    PAIR(MAGB200_BF16, MAGB200_F32) PAIR(MAGB200_BF16, MAGB200_F16) PAIR(MAGB200_BF16, MAGB200_BF16)
#undef PAIR
    set_error("cast: unsupported dtype pair %d -> %d", s, d);
    return MAGB200_ERR_INVALID_ARG;
}

size_t packed_operand_bytes(const GemmProblem &p, bool is_a) {
    const int64_t rows = is_a ? p.M : p.N, kpad = (p.K + 7) / 8 * 8;
    int64_t batches = 1;
    for (int d = 0; d < p.nbatch; ++d)
        if ((is_a ? p.bsA[d] : p.bsB[d]) != 0) batches *= p.bshape[d];
    return (size_t)(batches * rows * kpad) * 2;
}

// Packs operand A (x) or B (y) of `p` into `dst` and rewrites `p` to read the packed copy.
int launch_pack_operand(GemmProblem &p, bool is_a, void *dst, cudaStream_t stream) {
    PackArgs a;
    memset(&a, 0, sizeof(a));
    a.src = reinterpret_cast<const uint16_t *>(is_a ? p.A : p.B);
    a.dst = reinterpret_cast<uint16_t *>(dst);
    a.rows = is_a ? p.M : p.N; a.K = p.K; a.kpad = (p.K + 7) / 8 * 8;
    a.s_row = is_a ? p.sAm : p.sBn; a.s_k = is_a ? p.sAk : p.sBk;
    a.nbatch = p.nbatch;
    int64_t pitch = a.rows * a.kpad, batches = 1;
    int64_t new_stride[kMaxBatchDims] = {0, 0, 0};
    for (int d = p.nbatch - 1; d >= 0; --d) {
        const int64_t st = is_a ? p.bsA[d] : p.bsB[d];
        a.bshape[d] = st != 0 ? p.bshape[d] : 1;
        a.bsrc[d] = st;
        a.bdst[d] = st != 0 ? pitch : 0;
        new_stride[d] = a.bdst[d];
        if (st != 0) { pitch *= p.bshape[d]; batches *= p.bshape[d]; }
    }
    a.total_rows = a.rows * batches;
    int64_t blocks = a.total_rows < (int64_t)num_sms() * 32 ? a.total_rows : (int64_t)num_sms() * 32;
    if (blocks < 1) return MAGB200_OK;
    pack_operand_kernel<<<(unsigned)blocks, kThreads, 0, stream>>>(a);
    count_launch();
    MAGB200_CUDA_TRY(cudaGetLastError());
    if (is_a) { p.A = dst; p.sAm = a.kpad; p.sAk = 1; for (int d = 0; d < p.nbatch; ++d) p.bsA[d] = new_stride[d]; }
    else { p.B = dst; p.sBn = a.kpad; p.sBk = 1; for (int d = 0; d < p.nbatch; ++d) p.bsB[d] = new_stride[d]; }
    return MAGB200_OK;
}

namespace {
template <int DT>
__global__ void __launch_bounds__(kThreads) swiglu_kernel(const uint32_t *__restrict__ g, const uint32_t *__restrict__ u,
                                                          uint32_t *__restrict__ out, int64_t pairs) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < pairs; i += stride) out[i] = swiglu_pack2<DT>(g[i], u[i]);
}
}  // namespace

int launch_swiglu(int dtype, const void *g, const void *u, void *out, int64_t n, cudaStream_t stream) {
    if (n <= 0) return MAGB200_OK;
    if ((n & 1) || (((uintptr_t)g | (uintptr_t)u | (uintptr_t)out) & 3u)) {
        set_error("swiglu: needs an even element count and 4-byte aligned tensors");
        return MAGB200_ERR_INVALID_ARG;
    }
    const int64_t pairs = n / 2;
    if (dtype == MAGB200_BF16)
        swiglu_kernel<MAGB200_BF16><<<grid_for(pairs), kThreads, 0, stream>>>((const uint32_t *)g, (const uint32_t *)u, (uint32_t *)out, pairs);
    else if (dtype == MAGB200_F16)
        swiglu_kernel<MAGB200_F16><<<grid_for(pairs), kThreads, 0, stream>>>((const uint32_t *)g, (const uint32_t *)u, (uint32_t *)out, pairs);
    else { set_error("swiglu: 16-bit dtypes only"); return MAGB200_ERR_INVALID_ARG; }
    count_launch();
    MAGB200_CUDA_TRY(cudaGetLastError());
    return MAGB200_OK;
}

int launch_split3(const GemmProblem &p, void *planes_a, void *planes_b, int *unsafe, cudaStream_t stream) {
    SplitArgs a;
    memset(&a, 0, sizeof(a));
    a.unsafe = unsafe;
    for (int which = 0; which < 2; ++which) {
        const bool is_a = which == 0;
        SplitOperand &o = a.op[which];
        const PlaneLayout l = plane_layout(p, is_a);
        o.src = reinterpret_cast<const float *>(is_a ? p.A : p.B);
        o.dst = reinterpret_cast<uint16_t *>(is_a ? planes_a : planes_b);
        o.rows = l.rows; o.K = p.K; o.kpad = l.kpad;
        o.s_row = is_a ? p.sAm : p.sBn; o.s_k = is_a ? p.sAk : p.sBk;
        o.nbatch = p.nbatch;
        for (int d = 0; d < p.nbatch; ++d) {
            const int64_t st = is_a ? p.bsA[d] : p.bsB[d];
            const bool kept = st != 0 && p.bshape[d] > 1;
            o.bshape[d] = kept ? p.bshape[d] : 1;
            o.bsrc[d] = st;
            o.bdst[d] = l.bstride[d];
        }
        o.row_tiles = (o.rows + 31) / 32;
        o.k_tiles = (o.kpad + 63) / 64;
        o.quads_per_row = o.kpad / 4;
        o.quads = o.quads_per_row * o.rows * l.batches;
        o.k_fast = (o.s_k == 1 || p.K == 1) ? 1 : 0;
        o.units = o.k_fast ? (o.quads + 1023) / 1024 : o.row_tiles * o.k_tiles * l.batches;
        bool aligned = (((uintptr_t)o.src) & 15u) == 0 && p.K % 4 == 0 && o.s_row % 4 == 0;
        for (int d = 0; d < p.nbatch; ++d)
            if (o.bsrc[d] % 4) aligned = false;
        o.vec4 = aligned ? 1 : 0;
    }
    int64_t blocks = a.op[0].units + a.op[1].units;
    if (blocks < 1) return MAGB200_OK;
    if (blocks > (int64_t)num_sms() * 16) blocks = (int64_t)num_sms() * 16;
    split3_kernel<<<(unsigned)blocks, kThreads, 0, stream>>>(a);
    count_launch();
    MAGB200_CUDA_TRY(cudaGetLastError());
    return MAGB200_OK;
}

int launch_fill(int dt, void *dst, int64_t n, double value, cudaStream_t stream) {
    if (n <= 0) return MAGB200_OK;
    // Host-side conversion with the same formulas as the device path (bf16: integer RNE; fp16: RNE).
    float f = (float)value;
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t bits = u;
    if (dt == MAGB200_BF16) {
        bits = ((u & 0x7FFFFFFFu) > 0x7F800000u) ? 0x7FC0u : ((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
        fill_kernel<MAGB200_BF16><<<grid_for(n), kThreads, 0, stream>>>(dst, n, bits);
    } else if (dt == MAGB200_F16) {
        uint32_t a = u & 0x7FFFFFFFu;
        if (a > 0x7F800000u) bits = ((u >> 16) & 0x8000u) | 0x7E00u | ((a >> 13) & 0x3FFu);
        else bits = (uint32_t)__half_as_ushort(__float2half_rn(f));
        fill_kernel<MAGB200_F16><<<grid_for(n), kThreads, 0, stream>>>(dst, n, bits);
    } else if (dt == MAGB200_F32) {
        fill_kernel<MAGB200_F32><<<grid_for(n), kThreads, 0, stream>>>(dst, n, bits);
    } else {
        set_error("fill: unsupported dtype %d", dt);
        return MAGB200_ERR_INVALID_ARG;
    }
    count_launch();
    MAGB200_CUDA_TRY(cudaGetLastError());
    return MAGB200_OK;
}

}  // namespace magb200
