// Second half of the fused row-sharded linear: sum the partial row blocks that the peers' GEMM epilogues pushed into this
// rank's staging buffer, round once, and write the finished rows into every rank's output (ordinary 128-bit stores through
// peer mappings: an all-gather without a separate collective).
//
// Staging layout on every rank: [ranks][rows_per_rank * N] elements; slot s holds rank s's partial product for the row
// block this rank owns. Partials arrive already rounded to the 16-bit storage type; they are summed in fp32 in slot order
// (reproducible) and rounded once more -- fewer roundings than a ring all-reduce, which rounds at every hop.
#include "common.cuh"

namespace magb200 {

namespace {

constexpr int kThreads = 256;
constexpr int kMaxRanks = 8;

struct PeerOut { void *p[kMaxRanks]; };

template <int DT>
__global__ void __launch_bounds__(kThreads) reduce_broadcast_kernel(const uint4 *__restrict__ stage, PeerOut out, int ranks, int rank,
                                                                   int64_t block_vecs) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < block_vecs; i += stride) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.f;
        for (int s = 0; s < ranks; ++s) {
            const uint4 v = __ldcs(stage + (int64_t)s * block_vecs + i);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if constexpr (DT == MAGB200_BF16) {
                    acc[2 * j] += __uint_as_float(w[j] << 16);
                    acc[2 * j + 1] += __uint_as_float(w[j] & 0xFFFF0000u);
                } else {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[j]));
                    acc[2 * j] += f.x;
                    acc[2 * j + 1] += f.y;
                }
            }
        }
        uint4 o;
        o.x = pack2_rn<DT>(acc[0], acc[1]);
        o.y = pack2_rn<DT>(acc[2], acc[3]);
        o.z = pack2_rn<DT>(acc[4], acc[5]);
        o.w = pack2_rn<DT>(acc[6], acc[7]);
        for (int d = 0; d < ranks; ++d)
            reinterpret_cast<uint4 *>(out.p[d])[(int64_t)rank * block_vecs + i] = o;
    }
}

// The same exchange through the NVSwitch: `mc_partial` and `mc_out` are multicast addresses of buffers that every rank
// allocated symmetrically (each rank's partial product [M,N] in its own memory, each rank's output [M,N]). One
// multimem.ld_reduce makes the switch fetch the 16 bytes at that offset from every rank's partial and add them (fp32
// accumulation), so a rank receives its row block once instead of once per peer; one multimem.st writes the finished 16
// bytes into every rank's output, so it leaves the rank once. Per GEMM a rank moves (p-1)/p + 1/p of the tensor in each
// direction instead of twice (p-1)/p, and the GEMM keeps its plain local epilogue.
template <int DT>
__global__ void __launch_bounds__(kThreads) multimem_reduce_broadcast_kernel(const uint4 *mc_partial, uint4 *mc_out, int64_t first_vec,
                                                                            int64_t block_vecs) {
    // A reduction through the switch takes microseconds to come back, so every thread keeps kInFlight of them in flight
    // (issued back to back, stored afterwards): 16 bytes x 8 x 256 threads x the grid is what covers the link's latency.
    constexpr int kInFlight = 8;
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t i0 = (int64_t)blockIdx.x * kThreads + threadIdx.x; i0 < block_vecs; i0 += stride * kInFlight) {
        uint32_t v[kInFlight][4];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const int64_t i = i0 + u * stride;
            if (i < block_vecs) {
                const uint4 *src = mc_partial + first_vec + i;
                if constexpr (DT == MAGB200_BF16)
                    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(v[u][0]), "=r"(v[u][1]), "=r"(v[u][2]), "=r"(v[u][3]) : "l"(src) : "memory");
                else
                    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                                 : "=r"(v[u][0]), "=r"(v[u][1]), "=r"(v[u][2]), "=r"(v[u][3]) : "l"(src) : "memory");
            }
        }
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const int64_t i = i0 + u * stride;
            if (i < block_vecs)
                asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
                             ::"l"(mc_out + first_vec + i), "r"(v[u][0]), "r"(v[u][1]), "r"(v[u][2]), "r"(v[u][3]) : "memory");
        }
    }
}

}  // namespace

int launch_multimem_reduce_broadcast(int dtype, const void *mc_partial, void *mc_out, int ranks, int rank, int64_t block_elems,
                                     int max_ctas, cudaStream_t stream) {
    if (ranks < 1 || ranks > kMaxRanks || rank < 0 || rank >= ranks) { set_error("multimem_reduce_broadcast: bad rank %d of %d", rank, ranks); return MAGB200_ERR_INVALID_ARG; }
    if (!mc_partial || !mc_out || block_elems % 8 || (((uintptr_t)mc_partial | (uintptr_t)mc_out) & 15u)) {
        set_error("multimem_reduce_broadcast: multicast addresses must be non-null and 16-byte aligned, the row block a multiple of 8 elements");
        return MAGB200_ERR_INVALID_ARG;
    }
    const int64_t vecs = block_elems / 8;
    int64_t blocks = (vecs + kThreads * 8 - 1) / (kThreads * 8);
    const int64_t cap = max_ctas > 0 ? max_ctas : num_sms() * 2;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) return MAGB200_OK;
    if (dtype == MAGB200_BF16)
        multimem_reduce_broadcast_kernel<MAGB200_BF16><<<(unsigned)blocks, kThreads, 0, stream>>>((const uint4 *)mc_partial, (uint4 *)mc_out, (int64_t)rank * vecs, vecs);
    else if (dtype == MAGB200_F16)
        multimem_reduce_broadcast_kernel<MAGB200_F16><<<(unsigned)blocks, kThreads, 0, stream>>>((const uint4 *)mc_partial, (uint4 *)mc_out, (int64_t)rank * vecs, vecs);
    else { set_error("multimem_reduce_broadcast: 16-bit dtypes only"); return MAGB200_ERR_INVALID_ARG; }
    count_launch();
    MAGB200_CUDA_TRY(cudaGetLastError());
    return MAGB200_OK;
}

int launch_reduce_broadcast(int dtype, const void *stage, void *const *peer_out, int ranks, int rank, int64_t block_elems,
                            cudaStream_t stream) {
    if (ranks < 1 || ranks > kMaxRanks || rank < 0 || rank >= ranks) { set_error("reduce_broadcast: bad rank %d of %d", rank, ranks); return MAGB200_ERR_INVALID_ARG; }
    if (block_elems % 8 || ((uintptr_t)stage & 15u)) { set_error("reduce_broadcast: the row block must be a multiple of 8 elements and 16-byte aligned"); return MAGB200_ERR_INVALID_ARG; }
    PeerOut out;
    for (int i = 0; i < kMaxRanks; ++i) out.p[i] = i < ranks ? peer_out[i] : nullptr;
    for (int i = 0; i < ranks; ++i)
        if (!out.p[i] || ((uintptr_t)out.p[i] & 15u)) { set_error("reduce_broadcast: output pointer of rank %d is null or misaligned", i); return MAGB200_ERR_INVALID_ARG; }
    const int64_t vecs = block_elems / 8;
    int64_t blocks = (vecs + kThreads - 1) / kThreads;
    if (blocks > num_sms() * 8) blocks = num_sms() * 8;
    if (blocks < 1) return MAGB200_OK;
    if (dtype == MAGB200_BF16)
        reduce_broadcast_kernel<MAGB200_BF16><<<(unsigned)blocks, kThreads, 0, stream>>>((const uint4 *)stage, out, ranks, rank, vecs);
    else if (dtype == MAGB200_F16)
        reduce_broadcast_kernel<MAGB200_F16><<<(unsigned)blocks, kThreads, 0, stream>>>((const uint4 *)stage, out, ranks, rank, vecs);
    else { set_error("reduce_broadcast: 16-bit dtypes only"); return MAGB200_ERR_INVALID_ARG; }
    count_launch();
    MAGB200_CUDA_TRY(cudaGetLastError());
    return MAGB200_OK;
}

}  // namespace magb200
