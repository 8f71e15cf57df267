// Shared device/host helpers for the B200 matmul + cast path.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/magnetron_b200.h"

namespace magb200 {

constexpr int kMaxDims = MAGB200_MAX_DIMS;
constexpr int kDefaultSMs = 148;   // a B200; used only until the current device has been asked
int num_sms();                     // multiprocessor count of the current device (cached per device)

// ---- error plumbing (thread-local message, never an exception across the C ABI) -----------------
void set_error(const char *fmt, ...);
int  cuda_fail(cudaError_t e, const char *what, const char *file, int line);
void count_launch(int n = 1);
// run-time knobs of the tensor-core kernels (gemm_tcgen05.cu)
void set_wait_limit_ns(uint64_t ns);
uint64_t get_wait_limit_ns();
void set_skip_kb_once(int kb);

#define MAGB200_CUDA_TRY(expr)                                                        \
    do {                                                                              \
        cudaError_t _e = (expr);                                                      \
        if (_e != cudaSuccess) return ::magb200::cuda_fail(_e, #expr, __FILE__, __LINE__); \
    } while (0)

static inline size_t dtype_size(int dt) { return dt == MAGB200_F32 ? 4 : 2; }
static inline bool dtype_ok(int dt) { return dt == MAGB200_F32 || dt == MAGB200_F16 || dt == MAGB200_BF16; }

// ---- a view with its dimensions collapsed, passed to kernels by value ---------------------------
// Adjacent dims d, d+1 are merged when stride[d] == stride[d+1]*shape[d+1]; size-1 dims vanish.
struct CollapsedDims {
    int     rank;               // 0..kMaxDims (0: a single element)
    int64_t shape[kMaxDims];
    int64_t strides[kMaxDims];
};
CollapsedDims collapse_dims(int rank, const int64_t *shape, const int64_t *strides);
bool    view_is_contiguous(const magb200_view_t *v);
int64_t view_numel(const magb200_view_t *v);

// ---- bit-exact scalar conversions (device) ------------------------------------------------------
// fp32 -> bf16: every NaN becomes 0x7FC0; otherwise round-to-nearest-even on the integer pattern
// (magnetron/core/mag_bfloat16.h:47-58). cvt.rn.bf16.f32 is not used because it maps NaN to 0x7FFF.
__device__ __forceinline__ uint32_t f32_bits_to_bf16_bits(uint32_t u) {
    uint32_t r = (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
    return ((u & 0x7FFFFFFFu) > 0x7F800000u) ? 0x7FC0u : r;
}
__device__ __forceinline__ uint32_t bf16_bits_to_f32_bits(uint32_t h) { return h << 16; }

// fp32 -> fp16 with the semantics of x86 F16C `vcvtps2ph` (magnetron/cpu/mag_cpu_impl_cast.inl:12-28):
// RNE with gradual underflow; NaN keeps sign + top 10 payload bits and gets the quiet bit.
__device__ __forceinline__ uint32_t f32_bits_to_f16_bits(uint32_t u) {
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return ((u >> 16) & 0x8000u) | 0x7E00u | ((a >> 13) & 0x3FFu);
    return (uint32_t)__half_as_ushort(__float2half_rn(__uint_as_float(u)));
}
// fp16 -> fp32 with the semantics of `vcvtph2ps` (magnetron/cpu/mag_cpu_impl_cast.inl:30-46):
// exact; a signalling NaN is quieted, payload shifted up.
__device__ __forceinline__ uint32_t f16_bits_to_f32_bits(uint32_t h) {
    h &= 0xFFFFu;
    if ((h & 0x7FFFu) > 0x7C00u) return ((h & 0x8000u) << 16) | 0x7FC00000u | ((h & 0x3FFu) << 13);
    return __float_as_uint(__half2float(__ushort_as_half((unsigned short)h)));
}

template <int DT> __device__ __forceinline__ float load_as_f32(const void *p, int64_t i);
template <> __device__ __forceinline__ float load_as_f32<MAGB200_F32>(const void *p, int64_t i) { return ((const float *)p)[i]; }
template <> __device__ __forceinline__ float load_as_f32<MAGB200_F16>(const void *p, int64_t i) {
    return __uint_as_float(f16_bits_to_f32_bits(((const uint16_t *)p)[i]));
}
template <> __device__ __forceinline__ float load_as_f32<MAGB200_BF16>(const void *p, int64_t i) {
    return __uint_as_float(((uint32_t)((const uint16_t *)p)[i]) << 16);
}
template <int DT> __device__ __forceinline__ void store_from_f32(void *p, int64_t i, float v);
template <> __device__ __forceinline__ void store_from_f32<MAGB200_F32>(void *p, int64_t i, float v) { ((float *)p)[i] = v; }
template <> __device__ __forceinline__ void store_from_f32<MAGB200_F16>(void *p, int64_t i, float v) {
    ((uint16_t *)p)[i] = (uint16_t)f32_bits_to_f16_bits(__float_as_uint(v));
}
template <> __device__ __forceinline__ void store_from_f32<MAGB200_BF16>(void *p, int64_t i, float v) {
    ((uint16_t *)p)[i] = (uint16_t)f32_bits_to_bf16_bits(__float_as_uint(v));
}

// two fp32 accumulators -> one packed 32-bit word of two 16-bit results (element 0 in the low half)
template <int DT> __device__ __forceinline__ uint32_t pack2_from_f32(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2_from_f32<MAGB200_BF16>(float lo, float hi) {
    return f32_bits_to_bf16_bits(__float_as_uint(lo)) | (f32_bits_to_bf16_bits(__float_as_uint(hi)) << 16);
}
template <> __device__ __forceinline__ uint32_t pack2_from_f32<MAGB200_F16>(float lo, float hi) {
    return f32_bits_to_f16_bits(__float_as_uint(lo)) | (f32_bits_to_f16_bits(__float_as_uint(hi)) << 16);
}

// Matmul epilogues round with the hardware converters (one instruction per pair). They differ from the integer formulas above
// only in the bit pattern of a NaN result (0x7FFF instead of 0x7FC0 / a payload): a matmul produces NaN only from NaN or
// infinite inputs, and the reference's own NaN encoding there depends on which CPU specialisation stored the tile
// (magnetron/cpu/mag_cpu_impl_ops_matmul.inl:655-662 vs :772-778), so there is no single pattern to match. Casts keep the
// integer formulas and stay bit-exact.
template <int DT> __device__ __forceinline__ uint32_t pack2_rn(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2_rn<MAGB200_BF16>(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}
template <> __device__ __forceinline__ uint32_t pack2_rn<MAGB200_F16>(float lo, float hi) {
    uint32_t d;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
    return d;
}

// silu(g) * u as the unfused operator sequence of a gated MLP computes it (examples/qwen3/model.py:48-49: two matmuls, SILU,
// MUL, each rounding its result to the tensor dtype): `packed_g` and `packed_u` hold two matmul results each, already rounded
// to DT; silu is rounded once more, then the product. Shared by the fused GEMM epilogue and the elementwise kernel, so both
// give the same bits.
template <int DT> __device__ __forceinline__ void unpack2(uint32_t w, float &lo, float &hi);
template <> __device__ __forceinline__ void unpack2<MAGB200_BF16>(uint32_t w, float &lo, float &hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xFFFF0000u);
}
template <> __device__ __forceinline__ void unpack2<MAGB200_F16>(uint32_t w, float &lo, float &hi) {
    asm("{\n\t.reg .b16 l, h;\n\tmov.b32 {l, h}, %2;\n\tcvt.f32.f16 %0, l;\n\tcvt.f32.f16 %1, h;\n\t}" : "=f"(lo), "=f"(hi) : "r"(w));
}
__device__ __forceinline__ float silu_f32(float g) { return g / (1.0f + expf(-g)); }
template <int DT> __device__ __forceinline__ uint32_t swiglu_pack2(uint32_t packed_g, uint32_t packed_u) {
    float g0, g1, u0, u1, s0, s1;
    unpack2<DT>(packed_g, g0, g1);
    unpack2<DT>(packed_u, u0, u1);
    unpack2<DT>(pack2_rn<DT>(silu_f32(g0), silu_f32(g1)), s0, s1);
    return pack2_rn<DT>(s0 * u0, s1 * u1);
}

// ---- canonical description of one matmul, produced by the front-end in cabi.cu -----------------
constexpr int kMaxBatchDims = 3;
struct GemmProblem {
    int     dtype;                 // operand and result dtype
    int64_t M, N, K;
    const void *A;                 // x data (base + offset applied)
    const void *B;                 // y data
    void       *C;                 // result, row-major [batch..., M, N], ldc = N
    int64_t sAm, sAk;              // element strides of x's last two dims
    int64_t sBk, sBn;              // element strides of y's last two dims
    int     nbatch;                // collapsed batch dims, 0..kMaxBatchDims
    int64_t bshape[kMaxBatchDims]; // result batch extents (outermost first)
    int64_t bsA[kMaxBatchDims];    // x batch strides in elements (0 = broadcast)
    int64_t bsB[kMaxBatchDims];    // y batch strides
    int64_t batch_total;           // product of bshape
};

// kernel launchers (each returns a magb200_status_t); `stream` is the device's launch stream
// `run_if_set` (optional): two device words. The launch does nothing when word 0 is zero; when it ran, its last CTA clears
// word 0 again (word 1 counts the finished CTAs).
int launch_gemm_simt(const GemmProblem &p, cudaStream_t stream, float *splitk_scratch, size_t scratch_bytes, int *run_if_set = nullptr);
size_t simt_scratch_bytes(const GemmProblem &p);
bool skinny_supported(const GemmProblem &p);
int launch_skinny(const GemmProblem &p, cudaStream_t stream, float *splitk_scratch, size_t scratch_bytes, int *used_splitk, bool weights_settled);
void set_split_small(int on);   // one-CTA tensor-core kernel: CTA pairs split K when the output has at most 74 tiles of 128 x 128
void set_decode_row_streaming(int on);   // streaming decode kernel: row-contiguous copies (default) or the per-lane ring
int describe_skinny_plan(const GemmProblem &p, int *kind, int *nsplit, int *gridx, int *warps_along_k, int *cluster, int64_t *kch);
void set_decode_cluster_max(int max_cluster);   // 1, 2 or 4 CTAs per cluster for decode matrices with few row tiles (default 4)
int launch_skinny_grouped(const GemmProblem *ps, int count, cudaStream_t stream, bool weights_settled);   // 1: not applicable
bool tcgen05_supported(const GemmProblem &p);
// Destination of a scatter epilogue: every rank's staging buffer [ranks][rows_per_rank][N] (device or peer-mapped pointers)
struct ScatterTarget {
    int ranks, rank;
    int64_t rows_per_rank;
    void *stage[8];
};
// `overlapped`: launch as a programmatic dependent of the kernel before it on the stream, without a wait inside -- only when the
// caller knows that this product touches nothing that kernel (and those it may itself overlap) reads or writes
int launch_gemm_tcgen05(const GemmProblem &p, cudaStream_t stream, int cta_limit, int *status_word_dev, const ScatterTarget *scatter = nullptr,
                        bool overlapped = false);
bool tcgen05_2sm_supported(const GemmProblem &p);
bool tcgen05_2sm_preferred(const GemmProblem &p);
// Workspace for the shared-out last wave of the two-SM kernel: fp32 partial tiles and per-tile counters (zero between launches).
struct SplitWorkspace {
    float *partial;
    size_t partial_bytes;
    int *counters;        // 2 ints per tile
    int max_tiles;
};
int launch_gemm_tcgen05_2sm(const GemmProblem &p, cudaStream_t stream, int cta_limit, int *status_word_dev, const ScatterTarget *scatter = nullptr,
                            const SplitWorkspace *ws = nullptr, bool overlapped = false);
void set_balance_tail(int enabled);
int launch_reduce_broadcast(int dtype, const void *stage, void *const *peer_out, int ranks, int rank, int64_t block_elems, cudaStream_t stream);

int launch_multimem_reduce_broadcast(int dtype, const void *mc_partial, void *mc_out, int ranks, int rank, int64_t block_elems, int max_ctas,
                                     cudaStream_t stream);

int launch_cast(int src_dt, int dst_dt, const void *src, void *dst, int64_t n,
                const CollapsedDims &src_dims, bool src_contig, cudaStream_t stream, bool overlapped = false);
int launch_fill(int dt, void *dst, int64_t n, double value, cudaStream_t stream);
// device-side repack of a 16-bit operand that TMA cannot describe (see cast.cu)
bool tcgen05_operand_ok(const GemmProblem &p, bool is_a);
size_t packed_operand_bytes(const GemmProblem &p, bool is_a);
int launch_pack_operand(GemmProblem &p, bool is_a, void *dst, cudaStream_t stream);

// ---- gated MLP: out = silu(x @ Wg) * (x @ Wu) --------------------------------------------------------------------------
// Fused form: one two-SM GEMM whose 256 accumulator columns are 128 gate and 128 up columns of the same outputs, combined on
// the TMEM drain (`p` describes x @ Wg with C = out; `b_up` is Wu with Wg's strides). False / non-zero when the shapes or
// layouts do not allow it; the caller then runs two matmuls and launch_swiglu.
bool swiglu_fused_supported(const GemmProblem &p, const void *b_up);
int launch_gemm_swiglu(const GemmProblem &p, const void *b_up, cudaStream_t st, int cta_limit, int *status_word_dev);
// out[i] = silu(g[i]) * u[i], contiguous, n elements of a 16-bit dtype (n even, 4-byte aligned pointers)
int launch_swiglu(int dtype, const void *g, const void *u, void *out, int64_t n, cudaStream_t stream);

// ---- float32 on the tensor cores: every fp32 operand element is written as the sum of three bf16 values (8 + 8 + 8
// significant bits) and the product is assembled from six bf16 MMAs; see gemm_tcgen05.cu. The three planes of one operand
// batch are stacked along the row dim: element (plane, row, k) sits at [plane * rows + row][k] of a [3 * rows][kpad] matrix
// with unit K stride, so one tensor map with the usual batch dims describes all of it. Broadcast batch dims are not replicated.
struct PlaneLayout {
    int64_t rows, kpad;                    // rows of one plane (M or N); row pitch in elements (K rounded up to 8)
    int64_t bstride[kMaxBatchDims];        // element stride of each batch dim in the packed operand (0: broadcast)
    int64_t batches;                       // product of the non-broadcast batch extents
};
inline PlaneLayout plane_layout(const GemmProblem &p, bool is_a) {
    PlaneLayout l;
    l.rows = is_a ? p.M : p.N;
    l.kpad = (p.K + 7) / 8 * 8;
    l.batches = 1;
    int64_t pitch = 3 * l.rows * l.kpad;
    for (int d = 0; d < kMaxBatchDims; ++d) l.bstride[d] = 0;
    for (int d = p.nbatch - 1; d >= 0; --d) {
        const int64_t st = is_a ? p.bsA[d] : p.bsB[d];
        if (st != 0 && p.bshape[d] > 1) { l.bstride[d] = pitch; pitch *= p.bshape[d]; l.batches *= p.bshape[d]; }
    }
    return l;
}
inline size_t plane_bytes(const PlaneLayout &l) { return (size_t)(l.batches * 3 * l.rows * l.kpad) * 2; }
// Splits both fp32 operands of `p` into their planes (one launch). `*unsafe` is raised when an element is not finite, would
// overflow bf16, or is so small that its lower planes would be subnormal: the split product is then not to be used.
int launch_split3(const GemmProblem &p, void *planes_a, void *planes_b, int *unsafe, cudaStream_t stream);
bool f32x3_supported(const GemmProblem &p);
// C = A @ B from the planes; the launch does nothing when `*skip_if_set` is non-zero.
int launch_gemm_f32x3(const GemmProblem &p, const void *planes_a, const void *planes_b, const int *skip_if_set, int *status_word_dev, cudaStream_t stream);

}  // namespace magb200
