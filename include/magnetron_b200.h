/*
 * magnetron_b200.h -- C ABI of the B200 (sm_100a) device implementation of magnetron's MATMUL and
 * fp32<->bf16/fp16 CAST operators.
 *
 * Plain C: pointers, sizes and POD structs only. Every function returns MAGB200_OK (0) or a negative
 * error code; the text of the last error of the calling thread is available from
 * magb200_last_error(). Nothing here falls back to the CPU: if no sm_100 device is present the calls
 * fail with MAGB200_ERR_NO_DEVICE.
 *
 * The entry points are what a magnetron backend module binds for this path. A magnetron backend
 * receives `mag_command_t {op, in[], out[]}` (magnetron/core/mag_backend.h:80-87) whose tensors are
 * described by (storage base, storage_offset in elements, dtype, rank, shape[16], strides[16])
 * (magnetron/core/mag_tensor.h:52-68, magnetron/core/mag_coords.h:21-25). `magb200_view_t` carries
 * exactly those fields.
 */
#ifndef MAGNETRON_B200_H
#define MAGNETRON_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default) /* the library is built with hidden visibility; these are its exports */
#endif

#define MAGB200_MAX_DIMS 16 /* MAG_MAX_DIMS, include/magnetron/magnetron.h */

/* Same numeric values as mag_dtype_t (include/magnetron/magnetron.h:171-174). */
typedef enum magb200_dtype_t {
    MAGB200_F32  = 0,
    MAGB200_F16  = 1,
    MAGB200_BF16 = 2
} magb200_dtype_t;

typedef enum magb200_status_t {
    MAGB200_OK                = 0,
    MAGB200_ERR_NO_DEVICE     = -1,  /* no CUDA device / not sm_100 */
    MAGB200_ERR_INVALID_ARG   = -2,  /* null pointer, bad rank, dtype outside {f32,f16,bf16}, misaligned base */
    MAGB200_ERR_SHAPE         = -3,  /* shapes do not form a matmul / cast pair (MAG_STATUS_ERR_OPERATOR_IMPOSSIBLE) */
    MAGB200_ERR_CUDA          = -4,  /* a CUDA runtime / driver call failed; text in magb200_last_error() */
    MAGB200_ERR_OOM           = -5,  /* device allocation failed (MAG_STATUS_ERR_MEMORY_ALLOCATION_FAILED) */
    MAGB200_ERR_TIMEOUT       = -6,  /* a bounded device-side wait ran out; the context stays usable */
    MAGB200_ERR_TOO_LARGE     = -7   /* a fixed-capacity entry point was given a problem beyond its limit */
} magb200_status_t;

/* One tensor operand as a backend sees it: mag_tensor_t without the runtime bookkeeping. */
typedef struct magb200_view_t {
    void   *base;                          /* device address of the storage buffer (storage->base)     */
    int64_t offset;                        /* storage_offset, in ELEMENTS                               */
    int32_t dtype;                         /* magb200_dtype_t                                           */
    int32_t rank;                          /* 0..16 (0: a scalar, one element)                          */
    int64_t shape[MAGB200_MAX_DIMS];
    int64_t strides[MAGB200_MAX_DIMS];     /* in elements; 0 is legal on size-1 (broadcast) dims        */
} magb200_view_t;

/* Which device kernel a matmul was routed to (for tests, profiles and the bench's launch count). */
typedef enum magb200_kernel_t {
    MAGB200_KERNEL_NONE     = 0,
    MAGB200_KERNEL_TCGEN05  = 1,  /* TMA-fed tcgen05.mma tiles, fp32 accumulators in TMEM               */
    MAGB200_KERNEL_SKINNY   = 2,  /* M <= 8 weight-streaming kernel (HBM bound)                          */
    MAGB200_KERNEL_SIMT     = 3,  /* exact-fp32 / arbitrary-stride tiled FFMA kernel                     */
    MAGB200_KERNEL_SKINNY_SPLITK = 4, /* M <= 8, K split across CTAs with an fp32 scratch reduction      */
    MAGB200_KERNEL_TCGEN05_2SM = 5,  /* 256 x 256 tiles on CTA pairs (tcgen05.mma.cta_group::2)           */
    MAGB200_KERNEL_TCGEN05_F32X3 = 6 /* float32 as three bf16 planes per operand: six tcgen05 MMAs per product,
                                        per-K-block accumulators folded with compensated fp32 sums        */
} magb200_kernel_t;

/* ---- library / device ------------------------------------------------------------------------ */
const char *magb200_last_error(void);
int  magb200_device_count(void);                          /* visible sm_100 devices (0 if none)        */
int  magb200_device_name(int device, char *buf, size_t cap);
int  magb200_device_init(int device);                     /* creates the per-device stream + workspace; idempotent */
int  magb200_device_shutdown(int device);
int  magb200_synchronize(int device);
/* Use an external CUDA stream (a cudaStream_t, e.g. the caller's current stream) for all launches
 * on `device`; NULL restores the library's own stream. */
int  magb200_set_stream(int device, void *cuda_stream);
void *magb200_get_stream(int device);
/* Cap the number of CTAs the tensor-core matmuls launch on `device` (0 = all 148 SMs). A tensor-parallel caller leaves a
 * few SMs free this way so that a collective running on another stream makes progress beside the persistent GEMM. */
int  magb200_set_cta_limit(int device, int max_ctas);

/* ---- failure handling ---------------------------------------------------------------------------
 * Every wait inside a kernel (on an mbarrier of the TMA / tensor-core pipeline) is bounded: when it runs out the kernel
 * raises a status word, stops issuing work, lets copies in flight land, frees its tensor memory and returns; the next
 * magb200_synchronize / magb200_download reports MAGB200_ERR_TIMEOUT and the device stays usable. The reference has no
 * counterpart (its CPU workers block on a condition variable, magnetron/cpu/mag_cpu_threadpool.c). The limit is one
 * second unless changed here (1 ms .. 60 s, process wide). */
int      magb200_set_wait_limit_ns(uint64_t ns);
uint64_t magb200_get_wait_limit_ns(void);
/* Test hooks, host side only -- nothing traps, faults or spins without a limit.
 * test_leave_stage_unarmed: in the NEXT tensor-core matmul, the loads of K block `k_block` of each CTA's first tile are
 *   never issued and their barrier is never armed, so the consumer's bounded wait runs out and the launch takes the
 *   time-out path described above. -1 disarms.
 * test_inject_fault: the next call that passes `site` fails with the given cudaError_t as if the CUDA runtime had
 *   returned it (before any device is touched, so the error mapping can be tested without a GPU). */
typedef enum magb200_fault_site_t {
    MAGB200_FAULT_SITE_MALLOC = 1,   /* magb200_malloc */
    MAGB200_FAULT_SITE_LAUNCH = 2    /* magb200_matmul */
} magb200_fault_site_t;
int  magb200_test_leave_stage_unarmed(int k_block);
int  magb200_test_inject_fault(int site, int cuda_error);

/* ---- storage: counterpart of mag_device_t::alloc_storage (magnetron/core/mag_backend.h:96) and of
 * the transfers the reference performs with memcpy on CPU storage (mag_copy_raw_,
 * magnetron/core/mag_op_stubs.c:1360-1375; mag_tensor_copy_data, magnetron/core/mag_tensor.c:232-250). */
int  magb200_malloc(int device, void **out, size_t bytes);          /* 256-byte aligned device memory */
int  magb200_free(int device, void *ptr);
/* malloc / free go through a per-device pool: a freed block is kept (size classes, at most 12.5 % slack) and handed out
 * again without a CUDA call or a synchronisation -- legal because every operator and copy of this library runs on the
 * device's one launch stream, so the next user of a block is ordered after its last one. The reference frees with the
 * storage's reference count (magnetron/cpu/mag_cpu.c:100-130); doing that with cudaFree would stall the stream per tensor.
 * pool_stats: bytes handed out, bytes cached, and how many allocations were served from the cache / by cudaMalloc.
 * pool_trim: waits for the device and returns every cached block to the driver. */
int  magb200_pool_stats(int device, uint64_t *live_bytes, uint64_t *cached_bytes, uint64_t *hits, uint64_t *misses);
int  magb200_pool_trim(int device);
/* Free and total device memory as the driver reports them (cudaMemGetInfo); blocks cached by the pool count as used. */
int  magb200_mem_info(int device, uint64_t *free_bytes, uint64_t *total_bytes);
int  magb200_upload(int device, void *dst_device, const void *src_host, size_t bytes);   /* stream-ordered, then synchronised */
int  magb200_download(int device, void *dst_host, const void *src_device, size_t bytes); /* stream-ordered, then synchronised */
int  magb200_upload_async(int device, void *dst_device, const void *src_pinned_host, size_t bytes);
/* `rows` rows of `width_bytes` each from a pitched host matrix into a pitched device matrix, then synchronised: one rank's
 * slice of a weight that sits whole in a memory-mapped snapshot file (magnetron/core/mag_snapshot.c:566-640 hands out such
 * tensors on the CPU only) goes to the device without an intermediate copy of the slice. */
int  magb200_upload_2d(int device, void *dst_device, size_t dst_pitch, const void *src_host, size_t src_pitch, size_t width_bytes, size_t rows);
int  magb200_download_async(int device, void *dst_pinned_host, const void *src_device, size_t bytes);
/* Transfers on the library's two copy streams, so host<->device traffic of one operator runs beside the kernels of
 * others and uploads run beside downloads (the link is full duplex). No reference counterpart: magnetron's module ABI
 * has no transfer entry at all (magnetron/core/mag_backend.h:80-115).
 * upload_overlapped: starts after the operators submitted so far (they may still read dst); operators submitted later
 *   wait for it. download_overlapped: starts after the operators submitted so far; later operators do NOT wait for it,
 *   so the caller must leave src_device untouched until magb200_synchronize, which also waits for both copy streams. */
int  magb200_upload_overlapped(int device, void *dst_device, const void *src_pinned_host, size_t bytes);
int  magb200_download_overlapped(int device, void *dst_pinned_host, const void *src_device, size_t bytes);
int  magb200_host_alloc_pinned(void **out, size_t bytes);
int  magb200_host_free_pinned(void *ptr);

/* ---- operators --------------------------------------------------------------------------------
 * All three are stream-ordered on the device's stream and return without synchronising. */

/* MAG_OP_CAST: replaces mag_cast_generic + mag_vcast_* (magnetron/cpu/mag_cpu_impl_cast.inl:482-523)
 * for dtype pairs within {f32, f16, bf16}. Bit-exact with the reference conversions
 * (magnetron/core/mag_bfloat16.h:47-65; F16C semantics of magnetron/cpu/mag_cpu_impl_cast.inl:12-46).
 * `dst` must be contiguous with the same shape as `src`; `src` may be any strided view. */
int  magb200_cast(int device, const magb200_view_t *src, const magb200_view_t *dst);

/* MAG_OP_CLONE for the same dtypes (strided gather into a contiguous result); what
 * mag_contiguous / mag_reshape of a strided view dispatch (magnetron/core/mag_op_stubs.c:424-470). */
int  magb200_clone(int device, const magb200_view_t *src, const magb200_view_t *dst);

/* MAG_OP_CAT (mag_cat, magnetron/core/mag_op_stubs.c:996-1030; CPU kernels magnetron/cpu/mag_cpu_impl.inl:692-701):
 * `count` contiguous inputs of one dtype and rank, equal on every axis but `dim`, copied one after the other along `dim`
 * into the contiguous `dst` (stream-ordered device-to-device copies; the KV-cache append of the Qwen3 example). */
int  magb200_cat(int device, const magb200_view_t *const *parts, int count, int dim, const magb200_view_t *dst);

/* MAG_OP_FILL with a floating point value (magnetron/cpu/mag_cpu_impl_ops_fill.inl), contiguous dst. */
int  magb200_fill(int device, const magb200_view_t *dst, double value);

/* MAG_OP_MATMUL: replaces mag_matmul_float32 / _bfloat16 / _float16
 * (magnetron/cpu/mag_cpu_impl_ops_matmul.inl:2821-2919, :2921-3019, :3062-3116) including the
 * batch/broadcast index mapping (:2971-2989, :2798-2819) and the rank-1 operand rules of the
 * operator stub (magnetron/core/mag_op_stubs.c:1249-1310). x and y share one dtype; `r` is the
 * pre-allocated contiguous result of the shape the stub infers. fp32 accumulation over the whole K,
 * one rounding to the result dtype. */
int  magb200_matmul(int device, const magb200_view_t *x, const magb200_view_t *y, const magb200_view_t *r);

/* Gated MLP, r = silu(x @ w_gate) * (x @ w_up): the operator sequence MATMUL, MATMUL, SILU, MUL of a SwiGLU block
 * (examples/qwen3/model.py:48-49) as one call, with the roundings of that sequence (both matmul results, silu and the
 * product are each rounded to the tensor dtype), so the result is what the four operators give. bf16 and fp16. When
 * M >= 256, N >= 128 and TMA can describe the operands, one two-SM GEMM computes gate and up columns of the same outputs
 * side by side in TMEM and combines them on the drain: the two [M, N] intermediates never reach memory. Other shapes run two
 * matmuls into pooled temporaries and an elementwise pass (not during graph capture). w_gate and w_up are y operands of
 * magb200_matmul (e.g. W.T views) of equal shape and strides; r is contiguous. */
int  magb200_matmul_swiglu(int device, const magb200_view_t *x, const magb200_view_t *w_gate, const magb200_view_t *w_up,
                           const magb200_view_t *r);

/* `count` (1..4) matmuls that share their first operand: r_i = x @ y_i, e.g. the q, k and v projections or gate and up of a
 * decode step, which magnetron dispatches as consecutive MAG_OP_MATMULs with the same in[0] (examples/qwen3/model.py:109-111,
 * :48-49). Decode-shaped groups (M <= 8, 16-bit K-major weights, no K split) run as ONE launch whose 16-row weight tiles
 * span all the y_i; anything else is executed product by product. Each result is the fp32-accumulated product rounded once,
 * as from magb200_matmul; it has the same bits as a separate call whenever the group and the separate call cut K into the same
 * number of slices (always for fewer than 297 row tiles in total, e.g. q/k/v of a small model), otherwise the fp32 sums are
 * taken in another order. */
int  magb200_matmul_grouped(int device, const magb200_view_t *x, int count, const magb200_view_t *const *ys,
                            const magb200_view_t *const *rs);

/* Shape inference of the operator stub (magnetron/core/mag_op_stubs.c:1249-1310) for callers that
 * allocate `r` themselves. Returns MAGB200_ERR_SHAPE with the reference's message on a mismatch. */
int  magb200_matmul_result_shape(const magb200_view_t *x, const magb200_view_t *y, int32_t *out_rank, int64_t *out_shape);

/* Kernel that the most recent magb200_matmul on this thread was routed to, and the number of
 * device kernels launched by this library since magb200_launch_count_reset(). */
int      magb200_last_kernel(void);
uint64_t magb200_launch_count(void);
void     magb200_launch_count_reset(void);
/* Restrict routing (testing / profiling): 0 = automatic, otherwise a magb200_kernel_t that must be
 * able to run the problem, else the call fails with MAGB200_ERR_INVALID_ARG. */
int  magb200_force_kernel(int kernel);
/* Tensor-core matmuls submitted back to back (consecutive magb200_matmul calls on a device with nothing but pool
 * allocations and releases in between, on the library's own stream): one that reads nothing the ones before it write and
 * writes nothing they read or write is launched as a programmatic dependent without a wait, so its first CTAs run on the SMs
 * that the partial last wave of the matmul before it leaves idle (q, k, v of one input; gate and up). Any overlap of the
 * address ranges, any other operation in between, or a stream installed by the caller gives the ordinary, fully ordered
 * launch. Default on; 0 orders every launch. The counter says how many launches overlapped (tests). */
int      magb200_set_gemm_overlap(int on);
uint64_t magb200_overlapped_launch_count(void);

/* 16-bit products with K >= 1024 whose output has at most 74 tiles of 128 x 128 (e.g. 512 x 2048 x 2048) run as clusters of
 * two CTAs that split K and exchange halves of their fp32 accumulators through distributed shared memory, so twice as many
 * SMs work (default on; 0 keeps one CTA per tile: tests compare the two). */
int  magb200_set_small_output_split(int on);

/* Which kernel x @ y would be routed to (magb200_kernel_t), decided on the host from dtype, shapes, strides and alignment
 * alone; nothing is launched and no device is needed. `repacked` = 1: a 16-bit operand that TMA cannot describe (row pitch not
 * a multiple of 16 bytes, inner stride 2, misaligned slice) would first be copied into a legal layout on the device. */
int  magb200_matmul_route(const magb200_view_t *x, const magb200_view_t *y, int *kernel, int *repacked);

/* What the library would do with the decode-shaped product x @ y (M <= 8 after folding), decided on the host from shapes,
 * strides and alignment alone; nothing is launched and no device is needed (the data pointers must be the real ones only as
 * far as their alignment goes). kind: 0 not taken by the decode kernels, 1 small projection (register loads; `warps_along_k`
 * warps of a CTA and `cluster` CTAs split K), 2 streaming with a ring per lane, 3 streaming with row-contiguous copies,
 * 4 N-major weights through mma.sync, 5 FFMA kernels (float32). `k_splits` > 1: K is cut into chunks of `k_chunk` across CTAs
 * and a second kernel sums the partial results; `ctas`: grid size along the tile dimension. */
int  magb200_decode_plan(const magb200_view_t *x, const magb200_view_t *y, int *kind, int *k_splits, int *ctas, int *warps_along_k,
                         int *cluster, int64_t *k_chunk);

/* Decode-shaped products with plenty of weight rows (lm_head, the projections of a large model) stream their weights with
 * copies of 512 contiguous bytes of one row per warp instruction (default); 0 selects the older kernel in which every lane
 * keeps to its own two rows (64 bytes from each of 8 rows per instruction). Same arithmetic, another order of the fp32 sums. */
int  magb200_set_decode_row_streaming(int on);

/* Decode-shaped products whose weight matrix has few 16-row tiles (the 1024-row o and down projections of a small model) run
 * as clusters of up to `max_cluster` CTAs (1, 2 or 4; default 4) that split K once more and meet through distributed shared
 * memory, so that more SMs stream weights. 1 switches the clusters off (tests compare the two). */
int  magb200_set_decode_cluster(int max_cluster);

/* The two-SM kernel can share the tiles of a partial last wave out among all CTA pairs along K (fp32 partial tiles in the
 * library's workspace, summed in a fixed order, so results are reproducible). mode 1 (default): only where it pays (few
 * left-over tiles, K >= 4096); 0: never; 2: whenever the shape allows (tests). */
int  magb200_set_balanced_last_wave(int mode);

/* ---- tensor-parallel row-sharded linear, fused with its exchange ---------------------------------
 * No counterpart in the reference (it has no multi-device code). A row-sharded (K-sharded) linear needs the sum of
 * every rank's partial [M,N] product. Instead of a GEMM followed by an all-reduce, the GEMM's epilogue pushes each
 * finished tile straight into the staging buffer of the rank that owns those rows (ordinary stores through peer
 * mappings, under the main loop), and after a cross-rank barrier (the caller's, e.g. a symmetric-memory barrier)
 * magb200_reduce_broadcast sums the `nranks` partial blocks in fp32, rounds once and writes the finished rows into
 * every rank's output. `peer_stage[i]` / `peer_out[i]` are device addresses valid on THIS device for rank i's
 * buffers (peer-mapped; [nranks][M/nranks][N] and [M][N] elements). M must be divisible by nranks. */
int  magb200_matmul_scatter(int device, const magb200_view_t *x, const magb200_view_t *y, void *const *peer_stage, int nranks, int rank);
int  magb200_reduce_broadcast(int device, void *cuda_stream, const void *stage, void *const *peer_out, int nranks, int rank,
                              int64_t rows_per_rank, int64_t n, int dtype);   /* cuda_stream NULL = the device's stream; another
                              stream lets the exchange of one token chunk run beside the next chunk's GEMMs */

/* Planner of a tensor-parallel linear y[M,N] = x[M,K] @ W[N,K]^T over `ranks` GPUs: how to shard it, which exchange to use,
 * and whether sharding pays. `kind` says how the layer pairs the operator (column: shard N, no exchange; row: shard K, sum of
 * partial results). The answer may be REPLICATE when the sharded form would be slower than one GPU alone (tiny operators,
 * whose collective costs more than the work it saves); `pays` is set when the predicted speed-up is at least half of linear. */
typedef enum magb200_tp_mode_t { MAGB200_TP_REPLICATE = 0, MAGB200_TP_COLUMN = 1, MAGB200_TP_ROW = 2 } magb200_tp_mode_t;
typedef enum magb200_tp_exchange_t {
    MAGB200_TP_EXCHANGE_NONE = 0,
    MAGB200_TP_EXCHANGE_NCCL = 1,      /* local GEMM, then an NCCL all-reduce */
    MAGB200_TP_EXCHANGE_SCATTER = 2,   /* magb200_matmul_scatter + magb200_reduce_broadcast over peer memory */
    MAGB200_TP_EXCHANGE_SWITCH = 3     /* local GEMM + magb200_multimem_reduce_broadcast (in-switch reduction) */
} magb200_tp_exchange_t;
typedef struct magb200_tp_plan_t {
    int32_t mode;          /* magb200_tp_mode_t */
    int32_t exchange;      /* magb200_tp_exchange_t */
    int32_t chunks;        /* token chunks to pipeline through the layer (1: none) */
    int32_t pays;          /* predicted speed-up >= ranks / 2 */
    double  single_us;     /* predicted time on one GPU */
    double  sharded_us;    /* predicted time per rank, exchange included */
    double  speedup;
} magb200_tp_plan_t;
int  magb200_tp_plan(int64_t M, int64_t N, int64_t K, int ranks, int kind, int dtype, int has_peer_access, int has_multicast,
                     magb200_tp_plan_t *out);

/* The exchange of a row-sharded linear through the NVSwitch (NVLS), for buffers that all ranks allocated symmetrically and bound
 * to a multicast object: every rank's GEMM writes its partial [M,N] into its own `partial` buffer (plain magb200_matmul), the
 * ranks meet at a barrier, then each rank calls this for its row block: multimem.ld_reduce on `mc_partial` (the multicast
 * address of the partial buffers) makes the switch sum the block over all ranks, multimem.st on `mc_out` writes the sum into
 * every rank's output. A rank then receives and sends each byte of the result once instead of once per peer. No counterpart
 * in the reference. `max_ctas` bounds the grid (0 = default) so the kernel can run beside a GEMM on a side stream. */
int  magb200_multimem_reduce_broadcast(int device, void *cuda_stream, const void *mc_partial, void *mc_out, int nranks, int rank,
                                       int64_t rows_per_rank, int64_t n, int dtype, int max_ctas);

/* Decode-shaped matmul (M <= 8) that allocates nothing, for callers that are not allowed to call
 * cudaMalloc (a plug-in inside another framework's stream-ordered region, a serving loop that must not touch
 * the allocator once warm). No counterpart in the reference: its CPU backend takes split buffers from a
 * thread-local arena. Same operands and result as magb200_matmul; launches on `cuda_stream` (a
 * cudaStream_t; NULL = the default stream) and returns without synchronising. The split-K partial sums go
 * to a 4 MiB array built into the library (held by every GPU that loads it): problems whose partials
 * (splits x batch x M x N floats) exceed it fail with MAGB200_ERR_TOO_LARGE. The first call on a device
 * resolves the array's address and should be made before any stream capture. All calls share the array;
 * calls whose kernels overlap on the GPU race, so keep them on one stream. The call leaves `device` as the
 * calling thread's current CUDA device; a device that is absent or not sm_100 gives MAGB200_ERR_NO_DEVICE. */
int  magb200_matmul_skinny_noalloc(int device, void *cuda_stream, const magb200_view_t *x, const magb200_view_t *y,
                                   const magb200_view_t *r);

/* ---- host-buffer convenience: one call = upload operands, matmul, download result ------------
 * This is the call a CPU-side user of the reference makes (operands and result in host memory,
 * magnetron/core/mag_op_stubs.c:1249); the views' `base` fields are HOST addresses here. Synchronous. */
int  magb200_matmul_host(int device, const magb200_view_t *x, size_t x_storage_bytes,
                         const magb200_view_t *y, size_t y_storage_bytes,
                         const magb200_view_t *r);
int  magb200_cast_host(int device, const magb200_view_t *src, size_t src_storage_bytes, const magb200_view_t *dst);

/* ---- CUDA graphs for launch-bound sequences -----------------------------------------------------
 * A decode step is hundreds of microsecond-sized matmuls; replaying them as one graph removes the
 * per-call host cost. Between begin and end, operator calls on `device` are recorded instead of run.
 * Calls that allocate or synchronise (malloc/free/upload/download/synchronize, the *_host entry points,
 * a matmul whose split-K workspace would have to grow) are not allowed while capturing: run the sequence
 * once un-captured first. The reference has no counterpart (its CPU backend runs each operator
 * synchronously, magnetron/cpu/mag_cpu.c:70-89). */
int  magb200_graph_begin_capture(int device);
int  magb200_graph_end_capture(int device, void **out_graph);
int  magb200_graph_launch(int device, void *graph);     /* stream-ordered replay of the recorded launches */
int  magb200_graph_destroy(void *graph);

/* ---- timing on the library's stream (CUDA events recorded on the launch stream) --------------- */
int  magb200_event_create(void **out_event);
int  magb200_event_destroy(void *event);
int  magb200_event_record(int device, void *event);
int  magb200_event_elapsed_ms(void *start, void *stop, float *out_ms); /* synchronises on `stop` */

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* MAGNETRON_B200_H */
