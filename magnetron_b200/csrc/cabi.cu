// C ABI of the B200 matmul / cast path: device state, operand canonicalisation, kernel routing.
#include "common.cuh"

#include <mutex>
#include <stdarg.h>
#include <stdlib.h>
#include <atomic>
#include <unordered_map>
#include <vector>

namespace magb200 {

size_t skinny_scratch_bytes(const GemmProblem &p);  // gemv.cu

// ---- errors / counters --------------------------------------------------------------------------
static thread_local char g_err[768] = "";
static thread_local int g_last_kernel = MAGB200_KERNEL_NONE;
static std::atomic<uint64_t> g_launches{0};
static std::atomic<int> g_force{0};

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
int cuda_fail(cudaError_t e, const char *what, const char *file, int line) {
    set_error("%s failed: %s (%s:%d)", what, cudaGetErrorString(e), file, line);
    return e == cudaErrorMemoryAllocation ? MAGB200_ERR_OOM : MAGB200_ERR_CUDA;
}
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

int num_sms() {
    static std::atomic<int> cached[32];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 32) { (void)cudaGetLastError(); return kDefaultSMs; }
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n > 0) return n;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) { (void)cudaGetLastError(); return kDefaultSMs; }
    cached[dev].store(n, std::memory_order_relaxed);
    return n;
}

// ---- host-side fault injection (tests of the error paths; nothing on the device is made to fail) -------------------
// One pending fault per site: the next call that passes the site returns the given CUDA error as if the runtime had.
static std::atomic<int> g_inject[3] = {{0}, {0}, {0}};   // index = magb200_fault_site_t
static cudaError_t take_injected(int site) { return (cudaError_t)g_inject[site].exchange(0); }

// ---- device memory pool ------------------------------------------------------------------------------------------------
// magnetron allocates a storage buffer per tensor and frees it when the last reference goes
// (magnetron/core/mag_tensor.c:88-93, magnetron/cpu/mag_cpu.c:100-130); with cudaMalloc / cudaFree behind that, every
// intermediate of a layer costs a device synchronisation. Freed blocks are therefore kept in size classes (eight per power
// of two, at most 12.5 % slack) and handed out again without any CUDA call. Reuse needs no synchronisation because every
// operator and copy of this library runs on the device's one launch stream: whatever still reads a freed block was
// submitted before whatever will write it next. The one exception are downloads on the copy stream: a block freed while
// such a download may still read it is parked with an event recorded on that stream and rejoins the free lists once the
// event has completed. Blocks go back to the driver at shutdown or when cudaMalloc runs dry.
struct MemPool {
    std::mutex mu;
    std::unordered_map<size_t, std::vector<void *>> free_blocks;   // class size -> blocks
    std::unordered_map<void *, size_t> live;                       // block -> class size
    struct Deferred { void *ptr; size_t cls; cudaEvent_t ev; };
    std::vector<Deferred> deferred;                                // freed while a copy-stream download may still read them
    size_t cached_bytes = 0, live_bytes = 0;
    uint64_t hits = 0, misses = 0;
};
static size_t size_class(size_t bytes) {
    if (bytes <= 512) return 512;
    int top = 63 - __builtin_clzll((unsigned long long)(bytes - 1));   // bytes in (2^top, 2^(top+1)]
    const size_t step = (size_t)1 << (top - 2);                         // an eighth of the upper power of two
    return (bytes + step - 1) / step * step;
}

// ---- per-device state ---------------------------------------------------------------------------
constexpr int kMaxDevices = 16;
constexpr size_t kStatusBytes = 4096;
constexpr int kSplitFlagWord = 8;                          // "operands cannot be split" word of the float32 tensor-core path (+ a CTA counter)
constexpr int kCounterWord0 = 64, kCounterTiles = 256;   // counters of the two-SM kernel's shared last wave live in the status buffer
struct AddrRange { uintptr_t lo, hi; };
struct DeviceState {
    std::atomic<bool> ready{false};
    cudaStream_t own_stream = nullptr;
    cudaStream_t stream = nullptr;   // launch stream (own_stream unless the caller installed one)
    float *scratch = nullptr;        // split-K partial sums
    size_t scratch_bytes = 0;
    int *status = nullptr;           // device word raised by a kernel whose bounded wait ran out
    void *staging[3] = {nullptr, nullptr, nullptr};  // device buffers of the host-buffer entry points
    size_t staging_bytes[3] = {0, 0, 0};
    char name[256] = "";
    bool capturing = false;          // between graph_begin_capture and graph_end_capture
    int cta_limit = 0;               // 0: all SMs; else the tensor-core GEMMs launch at most this many CTAs
    cudaStream_t h2d_stream = nullptr;   // copy streams of the overlapped transfers (created on first use)
    cudaStream_t d2h_stream = nullptr;
    bool d2h_pending = false;            // overlapped downloads submitted since the last synchronize
    // Results written by the decode kernels launched since the last fully ordered operation. Those kernels let their
    // successors start early, so they may still be running when a later decode kernel begins: a weight operand inside one
    // of these ranges must not be fetched ahead of the kernel's wait for its predecessors.
    AddrRange in_flight[32];
    int n_in_flight = 0;
    bool in_flight_overflow = false;
    // Tensor-core GEMMs submitted back to back (nothing else put on the stream in between): what they read and write. A GEMM
    // that touches none of it is launched as a programmatic dependent without a wait, so its first CTAs run on the SMs that
    // the partial last wave of the GEMM before it leaves idle.
    AddrRange tc_reads[32], tc_writes[16];
    int n_tc_reads = 0, n_tc_writes = 0;
    bool chain_open = false;            // the last operation this library put on the stream was a tensor-core GEMM
    bool chain_open_at_entry = false;   // ... as of the start of the current entry point (every entry point closes the chain;
                                        // those that put nothing else on the stream restore it)
    MemPool *pool = nullptr;

    void reset() {
        own_stream = stream = nullptr; scratch = nullptr; scratch_bytes = 0; status = nullptr;
        for (int i = 0; i < 3; ++i) { staging[i] = nullptr; staging_bytes[i] = 0; }
        name[0] = 0; capturing = false; cta_limit = 0; h2d_stream = d2h_stream = nullptr; d2h_pending = false;
        n_in_flight = 0; in_flight_overflow = false;
        n_tc_reads = n_tc_writes = 0; chain_open = chain_open_at_entry = false;
        ready.store(false, std::memory_order_release);
    }
};
static DeviceState g_dev[kMaxDevices];
static std::mutex g_mu;

static int check_device(int device) {
    if (device < 0 || device >= kMaxDevices) { set_error("device %d out of range", device); return MAGB200_ERR_INVALID_ARG; }
    return MAGB200_OK;
}

static int ensure_device(int device, DeviceState **out) {
    int rc = check_device(device);
    if (rc) return rc;
    DeviceState &d = g_dev[device];
    if (!d.ready.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_mu);
        if (!d.ready.load(std::memory_order_relaxed)) {
            int n = 0;
            cudaError_t e = cudaGetDeviceCount(&n);
            if (e != cudaSuccess || device >= n) {
                set_error("no CUDA device %d (%s): this library has no CPU fallback", device,
                          e != cudaSuccess ? cudaGetErrorString(e) : "ordinal beyond the visible devices");
                return MAGB200_ERR_NO_DEVICE;
            }
            cudaDeviceProp prop;
            MAGB200_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
            if (prop.major != 10) {
                set_error("device %d (%s) is sm_%d%d; the kernels are built for sm_100a only", device, prop.name, prop.major, prop.minor);
                return MAGB200_ERR_NO_DEVICE;
            }
            snprintf(d.name, sizeof(d.name), "%s", prop.name);
            MAGB200_CUDA_TRY(cudaSetDevice(device));
            MAGB200_CUDA_TRY(cudaStreamCreateWithFlags(&d.own_stream, cudaStreamNonBlocking));
            d.stream = d.own_stream;
            MAGB200_CUDA_TRY(cudaMalloc(&d.status, kStatusBytes));     // word 0: time-out status; from word 64: tile counters
            MAGB200_CUDA_TRY(cudaMemset(d.status, 0, kStatusBytes));
            d.scratch_bytes = 64ull << 20;   // split-K partial sums; the two-SM kernel's shared last wave needs up to ~40 MB
            MAGB200_CUDA_TRY(cudaMalloc(&d.scratch, d.scratch_bytes));
            if (!d.pool) d.pool = new MemPool();
            d.ready.store(true, std::memory_order_release);
        }
    }
    MAGB200_CUDA_TRY(cudaSetDevice(device));
    d.chain_open_at_entry = d.chain_open;
    d.chain_open = false;
    *out = &d;
    return MAGB200_OK;
}
static void keep_chain(DeviceState &d) { d.chain_open = d.chain_open_at_entry; }   // for entry points that put nothing on the stream before a GEMM

static int ensure_scratch(DeviceState &d, size_t bytes) {
    if (bytes <= d.scratch_bytes) return MAGB200_OK;
    if (d.capturing) {
        set_error("the split-K workspace would have to grow to %zu bytes during stream capture; run the same call once before capturing", bytes);
        return MAGB200_ERR_INVALID_ARG;
    }
    // kernels submitted to an earlier launch stream (before magb200_set_stream) may still use the old buffer
    MAGB200_CUDA_TRY(cudaDeviceSynchronize());
    MAGB200_CUDA_TRY(cudaFree(d.scratch));
    d.scratch = nullptr; d.scratch_bytes = 0;
    size_t want = bytes + (bytes >> 2);
    MAGB200_CUDA_TRY(cudaMalloc(&d.scratch, want));
    d.scratch_bytes = want;
    return MAGB200_OK;
}

// ---- which results may still be in flight under programmatic dependent launch -----------------------------------------
static void ordered_point(DeviceState &d) {   // a fully ordered launch or copy
    d.n_in_flight = 0; d.in_flight_overflow = false;
    d.n_tc_reads = d.n_tc_writes = 0; d.chain_open = false;
}

// ---- back-to-back tensor-core GEMMs that may overlap --------------------------------------------------------------------
static std::atomic<int> g_gemm_overlap{1};
static std::atomic<uint64_t> g_overlapped_launches{0};
__global__ void order_kernel() {}
static bool operand_range(const void *base, size_t es, int64_t e0, int64_t s0, int64_t e1, int64_t s1, const GemmProblem &g, const int64_t *bs,
                          AddrRange &r) {
    if (s0 < 0 || s1 < 0) return false;
    int64_t reach = (e0 - 1) * s0 + (e1 - 1) * s1;
    for (int d = 0; d < g.nbatch; ++d) {
        if (bs[d] < 0) return false;
        reach += (g.bshape[d] - 1) * bs[d];
    }
    r.lo = (uintptr_t)base;
    r.hi = r.lo + (size_t)(reach + 1) * es;
    return true;
}
static bool hits(const AddrRange *list, int n, const AddrRange &r) {
    for (int i = 0; i < n; ++i)
        if (r.lo < list[i].hi && list[i].lo < r.hi) return true;
    return false;
}
// Decide how the next kernel of a run (a tensor-core GEMM or a contiguous cast: both let their successor start early) is
// launched, and record what it touches. True: as a programmatic dependent of the kernel before it (they may run side by
// side). False: an ordinary, fully ordered launch. `known`: the ranges below describe everything the kernel touches.
static bool next_kernel_overlaps(DeviceState &d, const AddrRange *reads, int n_reads, const AddrRange &write, bool known) {
    bool overlap = g_gemm_overlap.load() && d.chain_open && known && d.stream == d.own_stream && d.n_in_flight == 0 && !d.in_flight_overflow &&
                   d.n_tc_reads + n_reads <= 32 && d.n_tc_writes + 1 <= 16;
    if (overlap) overlap = !hits(d.tc_reads, d.n_tc_reads, write) && !hits(d.tc_writes, d.n_tc_writes, write);
    for (int i = 0; overlap && i < n_reads; ++i) overlap = !hits(d.tc_writes, d.n_tc_writes, reads[i]);
    if (!overlap) ordered_point(d);               // everything submitted before is complete when this launch starts
    if (known) {
        for (int i = 0; i < n_reads; ++i) d.tc_reads[d.n_tc_reads++] = reads[i];
        d.tc_writes[d.n_tc_writes++] = write;
    }
    d.chain_open = known;
    if (overlap) g_overlapped_launches.fetch_add(1);
    return overlap;
}
static bool next_gemm_overlaps(DeviceState &d, const GemmProblem &g) {
    const size_t es = dtype_size(g.dtype);
    AddrRange r[2], rc;
    const bool known = operand_range(g.A, es, g.M, g.sAm, g.K, g.sAk, g, g.bsA, r[0]) && operand_range(g.B, es, g.K, g.sBk, g.N, g.sBn, g, g.bsB, r[1]);
    rc.lo = (uintptr_t)g.C;
    rc.hi = rc.lo + (size_t)(g.batch_total * g.M * g.N) * es;
    return next_kernel_overlaps(d, r, 2, rc, known);
}
// A decode kernel is itself launched as a programmatic dependent: behind a run of overlapping GEMMs it could start while an
// earlier one of them still runs. An empty, fully ordered launch in between closes the run.
static int close_gemm_chain(DeviceState &d) {
    if (d.chain_open || d.chain_open_at_entry) {
        order_kernel<<<1, 32, 0, d.stream>>>();
        MAGB200_CUDA_TRY(cudaGetLastError());
        d.chain_open_at_entry = false;
    }
    d.n_tc_reads = d.n_tc_writes = 0;
    d.chain_open = false;
    return MAGB200_OK;
}
static void note_early_result(DeviceState &d, const void *ptr, size_t bytes) {
    const uintptr_t lo = (uintptr_t)ptr, hi = lo + bytes;
    for (int i = 0; i < d.n_in_flight; ++i)          // a decode loop writes the same few result buffers over and over
        if (lo >= d.in_flight[i].lo && hi <= d.in_flight[i].hi) return;
    if (d.n_in_flight < 32) { d.in_flight[d.n_in_flight].lo = lo; d.in_flight[d.n_in_flight].hi = hi; ++d.n_in_flight; return; }
    // full: fold everything into one covering range (weights inside it are then read after the wait, which is always safe)
    AddrRange all = {lo, hi};
    for (int i = 0; i < d.n_in_flight; ++i) {
        if (d.in_flight[i].lo < all.lo) all.lo = d.in_flight[i].lo;
        if (d.in_flight[i].hi > all.hi) all.hi = d.in_flight[i].hi;
    }
    d.in_flight[0] = all;
    d.n_in_flight = 1;
}
// Byte range an operand of the canonical problem can touch: base .. last addressed element.
static AddrRange weight_range(const GemmProblem &g) {
    int64_t reach = (g.K - 1) * g.sBk + (g.N - 1) * g.sBn;
    for (int i = 0; i < g.nbatch; ++i) reach += (g.bshape[i] - 1) * g.bsB[i];
    AddrRange r;
    r.lo = (uintptr_t)g.B;
    r.hi = r.lo + (size_t)(reach + 1) * dtype_size(g.dtype);
    return r;
}
static bool weights_settled(const DeviceState &d, const GemmProblem &g) {
    if (d.in_flight_overflow) return false;
    const AddrRange w = weight_range(g);
    for (int i = 0; i < d.n_in_flight; ++i)
        if (w.lo < d.in_flight[i].hi && d.in_flight[i].lo < w.hi) return false;
    return true;
}

static int check_status_word(DeviceState &d) {
    int h = 0;
    MAGB200_CUDA_TRY(cudaMemcpyAsync(&h, d.status, sizeof(int), cudaMemcpyDeviceToHost, d.stream));
    MAGB200_CUDA_TRY(cudaStreamSynchronize(d.stream));
    if (h != 0) {
        MAGB200_CUDA_TRY(cudaMemsetAsync(d.status, 0, kStatusBytes, d.stream));   // an abandoned launch may have left tile counters raised
        set_error("a device-side wait ran out (status %d): the launch was abandoned, results are invalid", h);
        return MAGB200_ERR_TIMEOUT;
    }
    return MAGB200_OK;
}

// ---- views --------------------------------------------------------------------------------------
int64_t view_numel(const magb200_view_t *v) {
    int64_t n = 1;
    for (int i = 0; i < v->rank; ++i) n *= v->shape[i];
    return n;
}
bool view_is_contiguous(const magb200_view_t *v) {
    int64_t expect = 1;
    for (int i = v->rank - 1; i >= 0; --i) {
        if (v->shape[i] != 1 && v->strides[i] != expect) return false;
        expect *= v->shape[i];
    }
    return true;
}
CollapsedDims collapse_dims(int rank, const int64_t *shape, const int64_t *strides) {
    CollapsedDims c;
    c.rank = 0;
    for (int i = 0; i < rank; ++i) {
        if (shape[i] == 1) continue;
        if (c.rank > 0 && c.strides[c.rank - 1] == strides[i] * shape[i]) {
            c.shape[c.rank - 1] *= shape[i];
            c.strides[c.rank - 1] = strides[i];
        } else {
            c.shape[c.rank] = shape[i];
            c.strides[c.rank] = strides[i];
            ++c.rank;
        }
    }
    return c;
}
static int check_view(const magb200_view_t *v, const char *what) {
    if (!v || !v->base) { set_error("%s: null view or base pointer", what); return MAGB200_ERR_INVALID_ARG; }
    if (!dtype_ok(v->dtype)) { set_error("%s: dtype %d is outside {float32, float16, bfloat16}", what, v->dtype); return MAGB200_ERR_INVALID_ARG; }
    if (v->rank < 0 || v->rank > kMaxDims) { set_error("%s: rank %d out of range", what, v->rank); return MAGB200_ERR_INVALID_ARG; }
    for (int i = 0; i < v->rank; ++i)
        if (v->shape[i] < 1 || v->strides[i] < 0) { set_error("%s: dim %d has extent %lld stride %lld", what, i, (long long)v->shape[i], (long long)v->strides[i]); return MAGB200_ERR_INVALID_ARG; }
    if (v->offset < 0) { set_error("%s: negative storage offset", what); return MAGB200_ERR_INVALID_ARG; }
    return MAGB200_OK;
}
// Bytes of storage a view reaches, from the storage base: (offset + sum (shape-1)*stride + 1) elements.
static size_t view_reach_bytes(const magb200_view_t *v) {
    int64_t last = v->offset;
    for (int i = 0; i < v->rank; ++i) last += (v->shape[i] - 1) * v->strides[i];
    return (size_t)(last + 1) * dtype_size(v->dtype);
}
static int check_view_fits(const magb200_view_t *v, size_t storage_bytes, const char *what) {
    const size_t need = view_reach_bytes(v);
    if (need > storage_bytes) {
        set_error("%s: the view reaches %zu bytes into a storage buffer of %zu", what, need, storage_bytes);
        return MAGB200_ERR_INVALID_ARG;
    }
    return MAGB200_OK;
}
static inline char *view_data(const magb200_view_t *v) { return (char *)v->base + v->offset * (int64_t)dtype_size(v->dtype); }

// ---- matmul front-end ---------------------------------------------------------------------------
static int result_shape(const magb200_view_t *x, const magb200_view_t *y, int32_t *out_rank, int64_t *out_shape) {
    const int xr = x->rank, yr = y->rank;
    const int64_t kx = x->shape[xr - 1];
    const int64_t ky = (yr == 1 || (yr == 2 && xr == 1)) ? y->shape[0] : y->shape[yr - 2];
    if (kx != ky) {
        set_error("Cannot perform matmul: last dimension of first tensor (%lld) does not match second tensor (%lld)", (long long)kx, (long long)ky);
        return MAGB200_ERR_SHAPE;
    }
    const int xbd = xr > 2 ? xr - 2 : 0, ybd = yr > 2 ? yr - 2 : 0, rbd = xbd > ybd ? xbd : ybd;
    for (int i = 0; i < rbd; ++i) {
        int64_t xd = i < rbd - xbd ? 1 : x->shape[i - (rbd - xbd)];
        int64_t yd = i < rbd - ybd ? 1 : y->shape[i - (rbd - ybd)];
        if (xd != yd && xd != 1 && yd != 1) {
            set_error("Cannot perform matmul: batch dimensions at index %d do not match (%lld != %lld)", i, (long long)xd, (long long)yd);
            return MAGB200_ERR_SHAPE;
        }
    }
    if (xr == 1 && yr == 1) { *out_rank = 0; out_shape[0] = 1; return MAGB200_OK; }  /* (K)x(K) -> scalar, mag_empty_scalar */
    if (xr == 1 && yr == 2) { *out_rank = 1; out_shape[0] = y->shape[1]; return MAGB200_OK; }
    if (xr == 2 && yr == 1) { *out_rank = 1; out_shape[0] = x->shape[0]; return MAGB200_OK; }
    for (int i = 0; i < rbd; ++i) {
        int64_t xd = i < rbd - xbd ? 1 : x->shape[i - (rbd - xbd)];
        int64_t yd = i < rbd - ybd ? 1 : y->shape[i - (rbd - ybd)];
        out_shape[i] = xd > yd ? xd : yd;
    }
    out_shape[rbd] = xr == 1 ? 1 : x->shape[xr - 2];
    out_shape[rbd + 1] = yr == 1 ? 1 : y->shape[yr - 1];
    *out_rank = rbd + 2;
    return MAGB200_OK;
}

struct FullProblem {
    GemmProblem g;                  // innermost (up to three) batch dims
    int n_outer;                    // further outer batch dims, looped on the host
    int64_t oshape[kMaxDims], osA[kMaxDims], osB[kMaxDims];
};

static int build_problem(const magb200_view_t *x, const magb200_view_t *y, const magb200_view_t *r, FullProblem &fp) {
    int rc;
    if ((rc = check_view(x, "matmul x")) || (rc = check_view(y, "matmul y")) || (rc = check_view(r, "matmul result"))) return rc;
    if (x->rank < 1 || y->rank < 1) { set_error("matmul: both tensors must have rank at least 1"); return MAGB200_ERR_INVALID_ARG; }
    if (x->dtype != y->dtype || x->dtype != r->dtype) {
        set_error("matmul: operands and result must share one dtype (got %d, %d -> %d)", x->dtype, y->dtype, r->dtype);
        return MAGB200_ERR_INVALID_ARG;
    }
    int32_t rr = 0;
    int64_t rs[kMaxDims + 2];
    if ((rc = result_shape(x, y, &rr, rs))) return rc;
    // the result must be the contiguous tensor the operator stub allocates; a leading size-1 difference
    // in rank is not accepted: shapes must match exactly
    bool same = (rr == r->rank);
    for (int i = 0; same && i < rr; ++i) same = (rs[i] == r->shape[i]);
    if (!same) { set_error("matmul: result view does not have the inferred shape"); return MAGB200_ERR_SHAPE; }
    if (!view_is_contiguous(r)) { set_error("matmul: result must be contiguous"); return MAGB200_ERR_INVALID_ARG; }

    GemmProblem &g = fp.g;
    memset(&fp, 0, sizeof(fp));
    const int xr = x->rank, yr = y->rank;
    g.dtype = x->dtype;
    g.M = xr == 1 ? 1 : x->shape[xr - 2];
    g.K = x->shape[xr - 1];
    g.N = yr == 1 ? 1 : y->shape[yr - 1];
    g.A = view_data(x); g.B = view_data(y); g.C = view_data(r);
    g.sAm = xr == 1 ? 0 : x->strides[xr - 2];
    g.sAk = x->strides[xr - 1];
    if (yr == 1) { g.sBk = y->strides[0]; g.sBn = 0; }
    else { g.sBk = y->strides[yr - 2]; g.sBn = y->strides[yr - 1]; }

    // batch dims of the result with per-operand strides (0 where the operand is broadcast)
    const int xbd = xr > 2 ? xr - 2 : 0, ybd = yr > 2 ? yr - 2 : 0, rbd = xbd > ybd ? xbd : ybd;
    int64_t ext[kMaxDims], sa[kMaxDims], sb[kMaxDims];
    int nb = 0;
    for (int i = 0; i < rbd; ++i) {
        const int xi = i - (rbd - xbd), yi = i - (rbd - ybd);
        const int64_t xd = xi < 0 ? 1 : x->shape[xi], yd = yi < 0 ? 1 : y->shape[yi];
        const int64_t e = xd > yd ? xd : yd;
        if (e == 1) continue;
        ext[nb] = e;
        sa[nb] = xd == 1 ? 0 : x->strides[xi];
        sb[nb] = yd == 1 ? 0 : y->strides[yi];
        ++nb;
    }
    // fold the innermost batch dim into M while y is broadcast there and x's rows continue seamlessly:
    // nn.Linear on [B,T,K] and GQA query groups become one taller GEMM instead of many small ones
    while (nb > 0 && sb[nb - 1] == 0 && (g.M == 1 || sa[nb - 1] == g.M * g.sAm)) {
        if (g.M == 1) g.sAm = sa[nb - 1];
        g.M *= ext[nb - 1];
        --nb;
    }
    // merge adjacent batch dims that both operands walk with one stride
    int m = 0;
    for (int i = 0; i < nb; ++i) {
        if (m > 0 && sa[m - 1] == sa[i] * ext[i] && sb[m - 1] == sb[i] * ext[i]) {
            ext[m - 1] *= ext[i]; sa[m - 1] = sa[i]; sb[m - 1] = sb[i];
        } else {
            ext[m] = ext[i]; sa[m] = sa[i]; sb[m] = sb[i]; ++m;
        }
    }
    nb = m;
    const int inner = nb < kMaxBatchDims ? nb : kMaxBatchDims;
    fp.n_outer = nb - inner;
    for (int i = 0; i < fp.n_outer; ++i) { fp.oshape[i] = ext[i]; fp.osA[i] = sa[i]; fp.osB[i] = sb[i]; }
    g.nbatch = inner;
    g.batch_total = 1;
    for (int i = 0; i < kMaxBatchDims; ++i) { g.bshape[i] = 1; g.bsA[i] = 0; g.bsB[i] = 0; }
    for (int i = 0; i < inner; ++i) {
        g.bshape[i] = ext[fp.n_outer + i]; g.bsA[i] = sa[fp.n_outer + i]; g.bsB[i] = sb[fp.n_outer + i];
        g.batch_total *= g.bshape[i];
    }
    return MAGB200_OK;
}

// Host-only canonicalisation for entry points that bring their own stream and scratch: same validation and
// folding as magb200_matmul, no device state touched. Problems that keep more than three batch dims are refused.
int canonicalize_skinny_problem(const magb200_view_t *x, const magb200_view_t *y, const magb200_view_t *r, GemmProblem *out) {
    FullProblem fp;
    int rc = build_problem(x, y, r, fp);
    if (rc) return rc;
    if (fp.n_outer != 0) { set_error("matmul: more than three independent batch dims are not supported by this entry point"); return MAGB200_ERR_INVALID_ARG; }
    *out = fp.g;
    return MAGB200_OK;
}

static int route(const GemmProblem &g, int forced, int *kernel) {
    const bool sk = g.M <= 8 && skinny_supported(g);
    const bool tc = tcgen05_supported(g);
    int k = sk ? MAGB200_KERNEL_SKINNY
               : (tc ? (tcgen05_2sm_preferred(g) ? MAGB200_KERNEL_TCGEN05_2SM : MAGB200_KERNEL_TCGEN05) : MAGB200_KERNEL_SIMT);
    // float32: the split-operand tensor-core kernel once the product is large enough to carry its fixed cost (one pass that
    // splits the operands, a stand-by launch of the FFMA kernel behind it)
    const bool f3 = g.dtype == MAGB200_F32 && f32x3_supported(g);
    if (k == MAGB200_KERNEL_SIMT && f3 && g.K >= 64 &&
        (double)g.M * (double)g.N * (double)g.K * (double)g.batch_total >= (double)(1ll << 28))
        k = MAGB200_KERNEL_TCGEN05_F32X3;
    if (forced) {
        if (forced == MAGB200_KERNEL_SKINNY_SPLITK) forced = MAGB200_KERNEL_SKINNY;
        const bool can = (forced == MAGB200_KERNEL_SKINNY && sk) || (forced == MAGB200_KERNEL_TCGEN05 && tc) ||
                         (forced == MAGB200_KERNEL_TCGEN05_2SM && tcgen05_2sm_supported(g)) || forced == MAGB200_KERNEL_SIMT ||
                         (forced == MAGB200_KERNEL_TCGEN05_F32X3 && f3);
        if (!can) {
            set_error("matmul: forced kernel %d cannot run this problem (M=%lld N=%lld K=%lld)", forced, (long long)g.M, (long long)g.N, (long long)g.K);
            return MAGB200_ERR_INVALID_ARG;
        }
        k = forced;
    }
    *kernel = k;
    return MAGB200_OK;
}

static SplitWorkspace split_workspace(DeviceState &d) {
    SplitWorkspace ws;
    ws.partial = d.scratch; ws.partial_bytes = d.scratch_bytes;
    ws.counters = d.status + kCounterWord0; ws.max_tiles = kCounterTiles;
    return ws;
}

static int run_one(DeviceState &d, int device, const GemmProblem &g, int kernel) {
    switch (kernel) {
        case MAGB200_KERNEL_SKINNY: {
            int rc = ensure_scratch(d, skinny_scratch_bytes(g));
            if (rc) return rc;
            if ((rc = close_gemm_chain(d))) return rc;
            int split = 0;
            rc = launch_skinny(g, d.stream, d.scratch, d.scratch_bytes, &split, weights_settled(d, g));
            g_last_kernel = split ? MAGB200_KERNEL_SKINNY_SPLITK : MAGB200_KERNEL_SKINNY;
            note_early_result(d, g.C, (size_t)(g.batch_total * g.M * g.N) * dtype_size(g.dtype));
            return rc;
        }
        case MAGB200_KERNEL_TCGEN05: {
            g_last_kernel = MAGB200_KERNEL_TCGEN05;
            const bool overlapped = next_gemm_overlaps(d, g);
            return launch_gemm_tcgen05(g, d.stream, d.cta_limit, d.status, nullptr, overlapped);
        }
        case MAGB200_KERNEL_TCGEN05_2SM: {
            g_last_kernel = MAGB200_KERNEL_TCGEN05_2SM;
            const bool overlapped = next_gemm_overlaps(d, g);
            const SplitWorkspace ws = split_workspace(d);
            return launch_gemm_tcgen05_2sm(g, d.stream, d.cta_limit, d.status, nullptr, &ws, overlapped);
        }
        case MAGB200_KERNEL_TCGEN05_F32X3: {
            // planes of both operands in the workspace; the FFMA kernel stands by behind the tensor-core launch and runs
            // instead of it when the split pass meets an element it cannot split (not finite, or out of bf16's normal range)
            const size_t bytes_a = (plane_bytes(plane_layout(g, true)) + 255) & ~(size_t)255;
            const size_t bytes_b = plane_bytes(plane_layout(g, false));
            const bool fits = bytes_a + bytes_b <= ((size_t)8 << 30) && !(d.capturing && bytes_a + bytes_b > d.scratch_bytes);
            if (fits && ensure_scratch(d, bytes_a + bytes_b) == MAGB200_OK) {
                g_last_kernel = MAGB200_KERNEL_TCGEN05_F32X3;
                ordered_point(d);
                int *unsafe = d.status + kSplitFlagWord;
                char *planes = reinterpret_cast<char *>(d.scratch);
                // `unsafe` is clear here: the stand-by launch of the call that raised it has lowered it again
                int rc = launch_split3(g, planes, planes + bytes_a, unsafe, d.stream);
                if (!rc) rc = launch_gemm_f32x3(g, planes, planes + bytes_a, unsafe, d.status, d.stream);
                if (!rc) rc = launch_gemm_simt(g, d.stream, nullptr, 0, unsafe);
                return rc;
            }
            (void)cudaGetLastError();
        }   // no room for the planes: the FFMA kernel takes the product
        // fallthrough
        default:
            g_last_kernel = MAGB200_KERNEL_SIMT;
            if (int rc = ensure_scratch(d, simt_scratch_bytes(g))) return rc;
            ordered_point(d);
            return launch_gemm_simt(g, d.stream, d.scratch, d.scratch_bytes);
    }
}

extern "C" int magb200_malloc(int device, void **out, size_t bytes);
extern "C" int magb200_free(int device, void *ptr);

// A 16-bit problem that fell to the FFMA kernel only because TMA cannot describe an operand (a row pitch that is not a
// multiple of 16 bytes -- any odd K --, an inner stride of 2, a misaligned slice): copy the offending operand(s) into pooled
// scratch with a legal pitch and run the tensor-core kernel on the copy. The reference packs every operand on every call
// (magnetron/cpu/mag_cpu_impl_ops_matmul.inl:1257-2308); here it is the exception. Returns 1 when the detour does not apply.
static int run_packed(DeviceState &d, int device, const GemmProblem &g) {
    if (g.dtype == MAGB200_F32 || g.M <= 8 || (double)g.M * (double)g.N * (double)g.K * (double)g.batch_total < (double)(1 << 24)) return 1;
    const bool pack_a = !tcgen05_operand_ok(g, true), pack_b = !tcgen05_operand_ok(g, false);
    if (!pack_a && !pack_b) return 1;
    if (d.capturing) return 1;                     // the scratch comes from the pool: not while a graph is being recorded
    ordered_point(d);                              // the pack kernels below are ordinary launches: the GEMM behind them must wait for them
    GemmProblem gp = g;
    void *ta = nullptr, *tb = nullptr;
    int rc = MAGB200_OK;
    if (pack_a && !(rc = magb200_malloc(device, &ta, packed_operand_bytes(g, true)))) rc = launch_pack_operand(gp, true, ta, d.stream);
    if (!rc && pack_b && !(rc = magb200_malloc(device, &tb, packed_operand_bytes(g, false)))) rc = launch_pack_operand(gp, false, tb, d.stream);
    if (!rc) {
        if (!tcgen05_supported(gp)) rc = 1;        // something else is in the way (e.g. a misaligned result): the FFMA kernel takes it
        else rc = run_one(d, device, gp, tcgen05_2sm_preferred(gp) ? MAGB200_KERNEL_TCGEN05_2SM : MAGB200_KERNEL_TCGEN05);
    }
    // back to the pool at once: the next owner of the blocks is ordered after this launch on the same stream
    if (ta) magb200_free(device, ta);
    if (tb) magb200_free(device, tb);
    return rc;
}

static int matmul_device(DeviceState &d, int device, const magb200_view_t *x, const magb200_view_t *y, const magb200_view_t *r) {
    FullProblem fp;
    int rc = build_problem(x, y, r, fp);
    if (rc) return rc;
    int kernel = 0;
    if ((rc = route(fp.g, g_force.load(), &kernel))) return rc;
    if (fp.n_outer == 0) {
        if (kernel == MAGB200_KERNEL_SIMT && g_force.load() == 0) {
            rc = run_packed(d, device, fp.g);
            if (rc <= 0) return rc;
        }
        return run_one(d, device, fp.g, kernel);
    }
    // more than three independent batch dims survive merging: walk the outer ones on the host
    int64_t outer_total = 1;
    for (int i = 0; i < fp.n_outer; ++i) outer_total *= fp.oshape[i];
    const int64_t es = (int64_t)dtype_size(fp.g.dtype);
    const int64_t slice = fp.g.batch_total * fp.g.M * fp.g.N;
    for (int64_t o = 0; o < outer_total; ++o) {
        int64_t rem = o, offA = 0, offB = 0;
        for (int i = fp.n_outer - 1; i >= 0; --i) {
            int64_t q = rem / fp.oshape[i], idx = rem - q * fp.oshape[i];
            offA += idx * fp.osA[i]; offB += idx * fp.osB[i];
            rem = q;
        }
        GemmProblem g = fp.g;
        g.A = (const char *)fp.g.A + offA * es;
        g.B = (const char *)fp.g.B + offB * es;
        g.C = (char *)fp.g.C + o * slice * es;
        int k2 = kernel;
        if ((rc = route(g, g_force.load(), &k2)) || (rc = run_one(d, device, g, k2))) return rc;
    }
    return MAGB200_OK;
}

static int cast_device(DeviceState &d, const magb200_view_t *src, const magb200_view_t *dst, bool same_dtype_required) {
    int rc;
    if ((rc = check_view(src, "cast source")) || (rc = check_view(dst, "cast result"))) return rc;
    if (same_dtype_required && src->dtype != dst->dtype) { set_error("clone: dtypes differ"); return MAGB200_ERR_INVALID_ARG; }
    const int64_t n = view_numel(src);
    if (n != view_numel(dst)) { set_error("cast: element counts differ (%lld vs %lld)", (long long)n, (long long)view_numel(dst)); return MAGB200_ERR_SHAPE; }
    if (!view_is_contiguous(dst)) { set_error("cast: result must be contiguous"); return MAGB200_ERR_INVALID_ARG; }
    CollapsedDims cd = collapse_dims(src->rank, src->shape, src->strides);
    // a contiguous cast behind a GEMM or a cast that touches none of its tensors may start on the SMs that kernel has left
    const bool contig = view_is_contiguous(src);
    AddrRange rs, rd;
    rs.lo = (uintptr_t)view_data(src); rs.hi = rs.lo + (size_t)n * dtype_size(src->dtype);
    rd.lo = (uintptr_t)view_data(dst); rd.hi = rd.lo + (size_t)n * dtype_size(dst->dtype);
    const bool overlapped = next_kernel_overlaps(d, &rs, 1, rd, contig && n > 0);
    return launch_cast(src->dtype, dst->dtype, view_data(src), view_data(dst), n, cd, contig, d.stream, overlapped);
}

static int ensure_staging(DeviceState &d, int slot, size_t bytes) {
    if (bytes <= d.staging_bytes[slot]) return MAGB200_OK;
    MAGB200_CUDA_TRY(cudaStreamSynchronize(d.stream));
    if (d.staging[slot]) MAGB200_CUDA_TRY(cudaFree(d.staging[slot]));
    d.staging[slot] = nullptr; d.staging_bytes[slot] = 0;
    MAGB200_CUDA_TRY(cudaMalloc(&d.staging[slot], bytes));
    d.staging_bytes[slot] = bytes;
    return MAGB200_OK;
}

}  // namespace magb200

using namespace magb200;

extern "C" {

const char *magb200_last_error(void) { return g_err; }

int magb200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { (void)cudaGetLastError(); return 0; }
    int ok = 0;
    for (int i = 0; i < n && i < kMaxDevices; ++i) {
        cudaDeviceProp p;
        if (cudaGetDeviceProperties(&p, i) == cudaSuccess && p.major == 10) ++ok; else break;
    }
    return ok;
}

int magb200_device_name(int device, char *buf, size_t cap) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if (buf && cap) snprintf(buf, cap, "%s", d->name);
    return MAGB200_OK;
}

int magb200_device_init(int device) { DeviceState *d; return ensure_device(device, &d); }

int magb200_device_shutdown(int device) {
    int rc = check_device(device);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(g_mu);
    DeviceState &d = g_dev[device];
    if (!d.ready) return MAGB200_OK;
    MAGB200_CUDA_TRY(cudaSetDevice(device));
    MAGB200_CUDA_TRY(cudaStreamSynchronize(d.stream));
    MAGB200_CUDA_TRY(cudaDeviceSynchronize());
    for (int i = 0; i < 3; ++i) if (d.staging[i]) { cudaFree(d.staging[i]); d.staging[i] = nullptr; d.staging_bytes[i] = 0; }
    cudaFree(d.scratch); cudaFree(d.status);
    if (d.h2d_stream) cudaStreamDestroy(d.h2d_stream);
    if (d.d2h_stream) cudaStreamDestroy(d.d2h_stream);
    cudaStreamDestroy(d.own_stream);
    if (d.pool) {   // cached blocks go back to the driver; blocks still held by the caller stay valid and are forgotten
        std::lock_guard<std::mutex> pl(d.pool->mu);
        for (auto &df : d.pool->deferred) { cudaEventDestroy(df.ev); cudaFree(df.ptr); }
        d.pool->deferred.clear();
        for (auto &cls : d.pool->free_blocks) for (void *b : cls.second) cudaFree(b);
        d.pool->free_blocks.clear(); d.pool->live.clear();
        d.pool->cached_bytes = d.pool->live_bytes = 0;
    }
    d.reset();
    return MAGB200_OK;
}

int magb200_synchronize(int device) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    MAGB200_CUDA_TRY(cudaStreamSynchronize(d->stream));
    if (d->d2h_stream) MAGB200_CUDA_TRY(cudaStreamSynchronize(d->d2h_stream));
    if (d->h2d_stream) MAGB200_CUDA_TRY(cudaStreamSynchronize(d->h2d_stream));
    d->d2h_pending = false;
    ordered_point(*d);
    return check_status_word(*d);
}

int magb200_set_cta_limit(int device, int max_ctas) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if (max_ctas < 0 || max_ctas > num_sms()) { set_error("set_cta_limit: %d is outside 0..%d", max_ctas, num_sms()); return MAGB200_ERR_INVALID_ARG; }
    d->cta_limit = max_ctas;
    return MAGB200_OK;
}

int magb200_set_stream(int device, void *cuda_stream) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    MAGB200_CUDA_TRY(cudaStreamSynchronize(d->stream));
    d->stream = cuda_stream ? (cudaStream_t)cuda_stream : d->own_stream;
    return MAGB200_OK;
}
void *magb200_get_stream(int device) {
    DeviceState *d;
    if (ensure_device(device, &d)) return nullptr;
    return (void *)d->stream;
}

static int order_after(cudaStream_t later, cudaStream_t earlier);

// Release every cached block of the pool to the driver (after the device has gone idle). Returns the bytes released.
static size_t pool_trim(DeviceState &d) {
    MemPool &p = *d.pool;
    if (p.cached_bytes == 0 && p.deferred.empty()) return 0;
    cudaDeviceSynchronize();
    for (auto &df : p.deferred) { cudaEventDestroy(df.ev); p.free_blocks[df.cls].push_back(df.ptr); p.cached_bytes += df.cls; }
    p.deferred.clear();
    size_t released = p.cached_bytes;
    for (auto &cls : p.free_blocks) for (void *b : cls.second) cudaFree(b);
    p.free_blocks.clear();
    p.cached_bytes = 0;
    return released;
}

int magb200_malloc(int device, void **out, size_t bytes) {
    if (!out) { set_error("malloc: null out pointer"); return MAGB200_ERR_INVALID_ARG; }
    *out = nullptr;
    if (cudaError_t inj = take_injected(MAGB200_FAULT_SITE_MALLOC)) return cuda_fail(inj, "cudaMalloc (injected)", __FILE__, __LINE__);
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    keep_chain(*d);                        // nothing goes on the launch stream here
    MemPool &p = *d->pool;
    const size_t cls = size_class(bytes ? bytes : 1);
    std::lock_guard<std::mutex> lock(p.mu);
    for (size_t i = 0; i < p.deferred.size();) {       // parked blocks whose download has finished are free again
        if (cudaEventQuery(p.deferred[i].ev) == cudaSuccess) {
            cudaEventDestroy(p.deferred[i].ev);
            p.free_blocks[p.deferred[i].cls].push_back(p.deferred[i].ptr);
            p.cached_bytes += p.deferred[i].cls;
            p.deferred[i] = p.deferred.back();
            p.deferred.pop_back();
        } else {
            (void)cudaGetLastError();                  // cudaErrorNotReady is not an error
            ++i;
        }
    }
    auto it = p.free_blocks.find(cls);
    if (it != p.free_blocks.end() && !it->second.empty()) {
        *out = it->second.back();
        it->second.pop_back();
        p.cached_bytes -= cls;
        ++p.hits;
    } else {
        void *ptr = nullptr;
        cudaError_t e = cudaMalloc(&ptr, cls);   // cudaMalloc returns >= 256-byte aligned memory
        if (e == cudaErrorMemoryAllocation && pool_trim(*d) > 0) { (void)cudaGetLastError(); e = cudaMalloc(&ptr, cls); }
        if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc", __FILE__, __LINE__);
        *out = ptr;
        ++p.misses;
    }
    p.live[*out] = cls;
    p.live_bytes += cls;
    return MAGB200_OK;
}
int magb200_free(int device, void *ptr) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    keep_chain(*d);                        // nothing goes on the launch stream here
    if (!ptr) return MAGB200_OK;
    MemPool &p = *d->pool;
    std::lock_guard<std::mutex> lock(p.mu);
    auto it = p.live.find(ptr);
    if (it == p.live.end()) {   // not from this pool (allocated before a shutdown): plain release
        MAGB200_CUDA_TRY(cudaStreamSynchronize(d->stream));
        MAGB200_CUDA_TRY(cudaFree(ptr));
        return MAGB200_OK;
    }
    const size_t cls = it->second;
    p.live.erase(it);
    p.live_bytes -= cls;
    if (d->d2h_pending && d->d2h_stream && !d->capturing) {
        // a download on the copy stream may still read the block: park it until everything queued there so far is done
        MemPool::Deferred df;
        df.ptr = ptr; df.cls = cls;
        MAGB200_CUDA_TRY(cudaEventCreateWithFlags(&df.ev, cudaEventDisableTiming));
        MAGB200_CUDA_TRY(cudaEventRecord(df.ev, d->d2h_stream));
        p.deferred.push_back(df);
        return MAGB200_OK;
    }
    p.free_blocks[cls].push_back(ptr);
    p.cached_bytes += cls;
    return MAGB200_OK;
}
int magb200_pool_stats(int device, uint64_t *live_bytes, uint64_t *cached_bytes, uint64_t *hits, uint64_t *misses) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(d->pool->mu);
    if (live_bytes) *live_bytes = d->pool->live_bytes;
    if (cached_bytes) *cached_bytes = d->pool->cached_bytes;
    if (hits) *hits = d->pool->hits;
    if (misses) *misses = d->pool->misses;
    return MAGB200_OK;
}
int magb200_mem_info(int device, uint64_t *free_bytes, uint64_t *total_bytes) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    size_t f = 0, t = 0;
    MAGB200_CUDA_TRY(cudaMemGetInfo(&f, &t));
    if (free_bytes) *free_bytes = f;
    if (total_bytes) *total_bytes = t;
    return MAGB200_OK;
}
int magb200_pool_trim(int device) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    std::lock_guard<std::mutex> lock(d->pool->mu);
    pool_trim(*d);
    return MAGB200_OK;
}
int magb200_upload_async(int device, void *dst, const void *src, size_t bytes) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    ordered_point(*d);
    MAGB200_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, d->stream));
    return MAGB200_OK;
}
int magb200_download_async(int device, void *dst, const void *src, size_t bytes) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    MAGB200_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, d->stream));
    return MAGB200_OK;
}
// `later` starts after everything submitted to `earlier` so far
static int order_after(cudaStream_t later, cudaStream_t earlier) {
    cudaEvent_t ev;
    MAGB200_CUDA_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    cudaError_t e = cudaEventRecord(ev, earlier);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(later, ev, 0);
    cudaEventDestroy(ev);   // released by the runtime once the recorded work has completed
    if (e != cudaSuccess) return cuda_fail(e, "event ordering", __FILE__, __LINE__);
    return MAGB200_OK;
}
static int copy_stream(DeviceState &d, cudaStream_t *slot) {
    if (d.capturing) { set_error("overlapped transfers cannot be recorded into a graph"); return MAGB200_ERR_INVALID_ARG; }
    if (!*slot) MAGB200_CUDA_TRY(cudaStreamCreateWithFlags(slot, cudaStreamNonBlocking));
    return MAGB200_OK;
}
int magb200_upload_overlapped(int device, void *dst, const void *src, size_t bytes) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc || (rc = copy_stream(*d, &d->h2d_stream))) return rc;
    if ((rc = order_after(d->h2d_stream, d->stream))) return rc;          // earlier operators may still read dst
    MAGB200_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, d->h2d_stream));
    return order_after(d->stream, d->h2d_stream);                          // later operators see the data
}
int magb200_download_overlapped(int device, void *dst, const void *src, size_t bytes) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc || (rc = copy_stream(*d, &d->d2h_stream))) return rc;
    if ((rc = order_after(d->d2h_stream, d->stream))) return rc;          // the producer of src has been submitted
    MAGB200_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, d->d2h_stream));
    d->d2h_pending = true;
    return MAGB200_OK;
}
int magb200_upload(int device, void *dst, const void *src, size_t bytes) {
    int rc = magb200_upload_async(device, dst, src, bytes);
    if (rc) return rc;
    MAGB200_CUDA_TRY(cudaStreamSynchronize(g_dev[device].stream));
    return MAGB200_OK;
}
int magb200_upload_2d(int device, void *dst, size_t dst_pitch, const void *src, size_t src_pitch, size_t width_bytes, size_t rows) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if (!dst || !src || width_bytes > dst_pitch || width_bytes > src_pitch) { set_error("upload_2d: a row is wider than a pitch"); return MAGB200_ERR_INVALID_ARG; }
    if (width_bytes == 0 || rows == 0) return MAGB200_OK;
    ordered_point(*d);
    MAGB200_CUDA_TRY(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyHostToDevice, d->stream));
    MAGB200_CUDA_TRY(cudaStreamSynchronize(d->stream));
    return MAGB200_OK;
}
int magb200_download(int device, void *dst, const void *src, size_t bytes) {
    int rc = magb200_download_async(device, dst, src, bytes);
    if (rc) return rc;
    return magb200_synchronize(device);
}
int magb200_host_alloc_pinned(void **out, size_t bytes) {
    if (!out) { set_error("host_alloc_pinned: null out pointer"); return MAGB200_ERR_INVALID_ARG; }
    MAGB200_CUDA_TRY(cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault));
    return MAGB200_OK;
}
int magb200_host_free_pinned(void *ptr) {
    if (ptr) MAGB200_CUDA_TRY(cudaFreeHost(ptr));
    return MAGB200_OK;
}

int magb200_cast(int device, const magb200_view_t *src, const magb200_view_t *dst) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    keep_chain(*d);
    return cast_device(*d, src, dst, false);
}
int magb200_clone(int device, const magb200_view_t *src, const magb200_view_t *dst) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    return cast_device(*d, src, dst, true);
}
int magb200_cat(int device, const magb200_view_t *const *parts, int count, int dim, const magb200_view_t *dst) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if (!parts || count < 1) { set_error("cat: no inputs"); return MAGB200_ERR_INVALID_ARG; }
    if ((rc = check_view(dst, "cat result"))) return rc;
    if (!view_is_contiguous(dst)) { set_error("cat: result must be contiguous"); return MAGB200_ERR_INVALID_ARG; }
    if (dim < 0 || dim >= dst->rank) { set_error("cat: dimension %d is outside [0, %d)", dim, dst->rank); return MAGB200_ERR_INVALID_ARG; }
    // contiguous inputs: input i is `outer` runs of inner_i elements, which land in the result at a pitch of sum inner_i
    int64_t outer = 1, tail = 1, along = 0;
    for (int i = 0; i < dim; ++i) outer *= dst->shape[i];
    for (int i = dim + 1; i < dst->rank; ++i) tail *= dst->shape[i];
    for (int p = 0; p < count; ++p) {
        const magb200_view_t *v = parts[p];
        if ((rc = check_view(v, "cat input"))) return rc;
        if (v->dtype != dst->dtype || v->rank != dst->rank) { set_error("cat: input %d differs from the result in dtype or rank", p); return MAGB200_ERR_INVALID_ARG; }
        if (!view_is_contiguous(v)) { set_error("cat: inputs must be contiguous row-major"); return MAGB200_ERR_INVALID_ARG; }
        for (int i = 0; i < dst->rank; ++i)
            if (i != dim && v->shape[i] != dst->shape[i]) { set_error("cat: shapes must match on non-concat dimensions (axis %d)", i); return MAGB200_ERR_SHAPE; }
        along += v->shape[dim];
    }
    if (along != dst->shape[dim]) { set_error("cat: inputs add up to %lld along dim %d, the result has %lld", (long long)along, dim, (long long)dst->shape[dim]); return MAGB200_ERR_SHAPE; }
    const size_t es = dtype_size(dst->dtype);
    const size_t pitch = (size_t)(dst->shape[dim] * tail) * es;
    char *out = view_data(dst);
    ordered_point(*d);
    for (int p = 0; p < count; ++p) {
        const size_t width = (size_t)(parts[p]->shape[dim] * tail) * es;
        MAGB200_CUDA_TRY(cudaMemcpy2DAsync(out, pitch, view_data(parts[p]), width, width, (size_t)outer, cudaMemcpyDeviceToDevice, d->stream));
        out += width;
    }
    return MAGB200_OK;
}
int magb200_fill(int device, const magb200_view_t *dst, double value) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if ((rc = check_view(dst, "fill result"))) return rc;
    if (!view_is_contiguous(dst)) { set_error("fill: result must be contiguous"); return MAGB200_ERR_INVALID_ARG; }
    ordered_point(*d);
    return launch_fill(dst->dtype, view_data(dst), view_numel(dst), value, d->stream);
}

int magb200_matmul_result_shape(const magb200_view_t *x, const magb200_view_t *y, int32_t *out_rank, int64_t *out_shape) {
    int rc;
    if ((rc = check_view(x, "matmul x")) || (rc = check_view(y, "matmul y"))) return rc;
    if (x->rank < 1 || y->rank < 1) { set_error("matmul: both tensors must have rank at least 1"); return MAGB200_ERR_INVALID_ARG; }
    if (!out_rank || !out_shape) { set_error("matmul_result_shape: null output"); return MAGB200_ERR_INVALID_ARG; }
    return result_shape(x, y, out_rank, out_shape);
}

int magb200_matmul(int device, const magb200_view_t *x, const magb200_view_t *y, const magb200_view_t *r) {
    if (cudaError_t inj = take_injected(MAGB200_FAULT_SITE_LAUNCH)) return cuda_fail(inj, "kernel launch (injected)", __FILE__, __LINE__);
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    keep_chain(*d);                        // a GEMM right behind the GEMM of the call before may run beside it
    return matmul_device(*d, device, x, y, r);
}

int magb200_matmul_swiglu(int device, const magb200_view_t *x, const magb200_view_t *w_gate, const magb200_view_t *w_up, const magb200_view_t *r) {
    if (cudaError_t inj = take_injected(MAGB200_FAULT_SITE_LAUNCH)) return cuda_fail(inj, "kernel launch (injected)", __FILE__, __LINE__);
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if (!x || !w_gate || !w_up || !r) { set_error("matmul_swiglu: null operand"); return MAGB200_ERR_INVALID_ARG; }
    FullProblem fg, fu;
    if ((rc = build_problem(x, w_gate, r, fg)) || (rc = build_problem(x, w_up, r, fu))) return rc;
    const GemmProblem &g = fg.g, &u = fu.g;
    if (g.dtype != MAGB200_BF16 && g.dtype != MAGB200_F16) { set_error("matmul_swiglu: 16-bit dtypes only"); return MAGB200_ERR_INVALID_ARG; }
    bool same = fg.n_outer == 0 && fu.n_outer == 0 && g.M == u.M && g.N == u.N && g.K == u.K && g.sBk == u.sBk && g.sBn == u.sBn &&
                g.nbatch == u.nbatch && g.batch_total == u.batch_total;
    for (int i = 0; same && i < g.nbatch; ++i) same = g.bsB[i] == u.bsB[i] && g.bshape[i] == u.bshape[i];
    if (same && g_force.load() == 0 && swiglu_fused_supported(g, u.B)) {
        g_last_kernel = MAGB200_KERNEL_TCGEN05_2SM;
        ordered_point(*d);
        return launch_gemm_swiglu(g, u.B, d->stream, d->cta_limit, d->status);
    }
    // the operator sequence as it is: two matmuls into pooled temporaries, then the elementwise pass
    if (d->capturing) { set_error("matmul_swiglu: this shape needs temporaries from the pool, which a graph capture cannot take"); return MAGB200_ERR_INVALID_ARG; }
    const int64_t n = view_numel(r);
    if (!view_is_contiguous(r) || (n & 1)) { set_error("matmul_swiglu: the result must be contiguous with an even element count"); return MAGB200_ERR_INVALID_ARG; }
    void *tg = nullptr, *tu = nullptr;
    const size_t bytes = (size_t)n * dtype_size(g.dtype);
    if ((rc = magb200_malloc(device, &tg, bytes)) == MAGB200_OK && (rc = magb200_malloc(device, &tu, bytes)) == MAGB200_OK) {
        magb200_view_t vg = *r, vu = *r;
        vg.base = tg; vg.offset = 0;
        vu.base = tu; vu.offset = 0;
        if (!(rc = matmul_device(*d, device, x, w_gate, &vg)) && !(rc = matmul_device(*d, device, x, w_up, &vu))) {
            ordered_point(*d);
            rc = launch_swiglu(g.dtype, tg, tu, view_data(r), n, d->stream);
        }
    }
    if (tg) magb200_free(device, tg);
    if (tu) magb200_free(device, tu);
    return rc;
}

int magb200_matmul_grouped(int device, const magb200_view_t *x, int count, const magb200_view_t *const *ys, const magb200_view_t *const *rs) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if (!x || !ys || !rs || count < 1 || count > 4) { set_error("matmul_grouped: 1..4 products per call"); return MAGB200_ERR_INVALID_ARG; }
    FullProblem fp[4];
    GemmProblem gs[4];
    bool one_launch = count > 1 && g_force.load() == 0;
    bool settled = true;
    for (int i = 0; i < count; ++i) {
        if ((rc = build_problem(x, ys[i], rs[i], fp[i]))) return rc;
        gs[i] = fp[i].g;
        one_launch = one_launch && fp[i].n_outer == 0;
        settled = settled && weights_settled(*d, gs[i]);
    }
    if (one_launch) {
        if ((rc = close_gemm_chain(*d))) return rc;
        rc = launch_skinny_grouped(gs, count, d->stream, settled);
        if (rc == MAGB200_OK) {
            g_last_kernel = MAGB200_KERNEL_SKINNY;
            for (int i = 0; i < count; ++i) note_early_result(*d, gs[i].C, (size_t)(gs[i].M * gs[i].N) * dtype_size(gs[i].dtype));
            return MAGB200_OK;
        }
        if (rc < 0) return rc;
    }
    for (int i = 0; i < count; ++i)
        if ((rc = matmul_device(*d, device, x, ys[i], rs[i]))) return rc;
    return MAGB200_OK;
}

int magb200_matmul_scatter(int device, const magb200_view_t *x, const magb200_view_t *y, void *const *peer_stage, int nranks, int rank) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if (!peer_stage || nranks < 1 || nranks > 8 || rank < 0 || rank >= nranks) { set_error("matmul_scatter: bad rank %d of %d", rank, nranks); return MAGB200_ERR_INVALID_ARG; }
    if ((rc = check_view(x, "matmul x")) || (rc = check_view(y, "matmul y"))) return rc;
    if (x->rank != 2 || y->rank != 2) { set_error("matmul_scatter: 2-D operands only"); return MAGB200_ERR_INVALID_ARG; }
    // the partial product has no home of its own: describe it as an [M,N] view of this rank's staging buffer for validation
    magb200_view_t r;
    memset(&r, 0, sizeof(r));
    r.base = peer_stage[rank]; r.dtype = x->dtype; r.rank = 2;
    r.shape[0] = x->shape[0]; r.shape[1] = y->shape[1]; r.strides[0] = y->shape[1]; r.strides[1] = 1;
    FullProblem fp;
    if ((rc = build_problem(x, y, &r, fp))) return rc;
    const GemmProblem &g = fp.g;
    if (g.nbatch != 0 || fp.n_outer != 0 || !tcgen05_supported(g) || g.M % nranks || g.N % 8) {
        set_error("matmul_scatter: needs a 16-bit, TMA-describable, unbatched problem with M divisible by the rank count and N by 8 "
                  "(M=%lld N=%lld K=%lld ranks=%d)", (long long)g.M, (long long)g.N, (long long)g.K, nranks);
        return MAGB200_ERR_INVALID_ARG;
    }
    ScatterTarget sc;
    sc.ranks = nranks; sc.rank = rank; sc.rows_per_rank = g.M / nranks;
    for (int i = 0; i < 8; ++i) sc.stage[i] = i < nranks ? peer_stage[i] : nullptr;
    for (int i = 0; i < nranks; ++i)
        if (!sc.stage[i] || ((uintptr_t)sc.stage[i] & 15u)) { set_error("matmul_scatter: staging pointer of rank %d is null or misaligned", i); return MAGB200_ERR_INVALID_ARG; }
    if (tcgen05_2sm_preferred(g)) {
        g_last_kernel = MAGB200_KERNEL_TCGEN05_2SM;
        const SplitWorkspace ws = split_workspace(*d);
        return launch_gemm_tcgen05_2sm(g, d->stream, d->cta_limit, d->status, &sc, &ws);
    }
    g_last_kernel = MAGB200_KERNEL_TCGEN05;
    return launch_gemm_tcgen05(g, d->stream, d->cta_limit, d->status, &sc);
}

int magb200_reduce_broadcast(int device, void *cuda_stream, const void *stage, void *const *peer_out, int nranks, int rank,
                             int64_t rows_per_rank, int64_t n, int dtype) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if (!stage || !peer_out || rows_per_rank < 1 || n < 1) { set_error("reduce_broadcast: null pointer or empty block"); return MAGB200_ERR_INVALID_ARG; }
    return launch_reduce_broadcast(dtype, stage, peer_out, nranks, rank, rows_per_rank * n, cuda_stream ? (cudaStream_t)cuda_stream : d->stream);
}

int magb200_set_wait_limit_ns(uint64_t ns) {
    if (ns < 1000ull * 1000ull || ns > 60ull * 1000ull * 1000ull * 1000ull) {
        set_error("set_wait_limit_ns: %llu is outside 1 ms .. 60 s", (unsigned long long)ns);
        return MAGB200_ERR_INVALID_ARG;
    }
    set_wait_limit_ns(ns);
    return MAGB200_OK;
}
uint64_t magb200_get_wait_limit_ns(void) { return get_wait_limit_ns(); }
int magb200_test_leave_stage_unarmed(int k_block) {
    if (k_block < -1) { set_error("test_leave_stage_unarmed: k_block must be >= 0 (or -1 to disarm)"); return MAGB200_ERR_INVALID_ARG; }
    set_skip_kb_once(k_block);
    return MAGB200_OK;
}
int magb200_set_balanced_last_wave(int mode) {
    if (mode < 0 || mode > 2) { set_error("set_balanced_last_wave: mode %d is outside 0..2", mode); return MAGB200_ERR_INVALID_ARG; }
    set_balance_tail(mode);
    return MAGB200_OK;
}
int magb200_test_inject_fault(int site, int cuda_error) {
    if (site < MAGB200_FAULT_SITE_MALLOC || site > MAGB200_FAULT_SITE_LAUNCH || cuda_error < 0) {
        set_error("test_inject_fault: unknown site %d", site);
        return MAGB200_ERR_INVALID_ARG;
    }
    g_inject[site].store(cuda_error);
    return MAGB200_OK;
}

// ---- tensor-parallel planner ---------------------------------------------------------------------------------------------
// Cost model in microseconds, from figures measured on this part: tensor-core GEMMs 1400 TFLOP/s, weight streaming 6000 GB/s,
// NVLink 650 GB/s per direction per GPU, 3 us per launch, an NCCL all-reduce 12 us before its first byte, the fused exchanges
// two cross-rank barriers of 4 us and one kernel.
int magb200_tp_plan(int64_t M, int64_t N, int64_t K, int ranks, int kind, int dtype, int has_peer_access, int has_multicast,
                    magb200_tp_plan_t *out) {
    if (!out || M < 1 || N < 1 || K < 1 || ranks < 1 || ranks > 8 || (kind != MAGB200_TP_COLUMN && kind != MAGB200_TP_ROW) || !dtype_ok(dtype)) {
        set_error("tp_plan: bad argument");
        return MAGB200_ERR_INVALID_ARG;
    }
    const double es = (double)dtype_size(dtype), p = (double)ranks;
    const double kTensor = 1400e6 /*FLOP per us*/, kHbm = 6000e3 /*bytes per us*/, kLink = 650e3, kLaunch = 3.0, kNccl = 12.0, kBarrier = 4.0;
    auto gemm_us = [&](double m, double n, double k) {
        const double flops = 2.0 * m * n * k, bytes = es * (m * k + n * k + m * n);
        const double t = flops / kTensor, b = bytes / kHbm;
        return (t > b ? t : b) + kLaunch;
    };
    memset(out, 0, sizeof(*out));
    out->single_us = gemm_us((double)M, (double)N, (double)K);
    out->chunks = 1;
    if (ranks == 1) { out->mode = kind; out->exchange = MAGB200_TP_EXCHANGE_NONE; out->sharded_us = out->single_us; out->pays = 0; return MAGB200_OK; }
    if (kind == MAGB200_TP_COLUMN) {          // independent GEMMs on N / p columns, no exchange
        out->mode = MAGB200_TP_COLUMN;
        out->exchange = MAGB200_TP_EXCHANGE_NONE;
        out->sharded_us = gemm_us((double)M, (double)N / p, (double)K);
    } else {                                  // partial products over K / p, then the sum of p partial [M,N] results
        const double result_bytes = es * (double)M * (double)N;
        const double wire = result_bytes * (p - 1.0) / p;          // per rank and direction, reduce-scatter + all-gather halves
        double ex;
        const bool fused_ok = has_peer_access && M % ranks == 0 && M >= 256 && N % 8 == 0 && dtype != MAGB200_F32;
        // the in-switch reduction moves fewer bytes per rank only from four ranks up ((p-1)/p + 1/p against 2 (p-1)/p), and at
        // two ranks it ran at a third of the peer-store path's rate
        if (fused_ok && has_multicast && ranks >= 8) { out->exchange = MAGB200_TP_EXCHANGE_SWITCH; ex = 2 * kBarrier + kLaunch + (wire + result_bytes / p) / kLink; }
        else if (fused_ok) { out->exchange = MAGB200_TP_EXCHANGE_SCATTER; ex = 2 * kBarrier + kLaunch + 2.0 * wire / kLink; }
        else { out->exchange = MAGB200_TP_EXCHANGE_NCCL; ex = kNccl + 2.0 * wire / kLink; }
        out->mode = MAGB200_TP_ROW;
        out->sharded_us = gemm_us((double)M, (double)N, (double)K / p) + ex;
        // two token chunks through the layer let the exchange kernels of one chunk fill the gaps between the other chunk's
        // GEMMs; measured on the Qwen3-32B layer at M = 8192: 8 ranks 7695 against 7440 TFLOP/s unchunked, 2 and 4 ranks no gain
        out->chunks = (M >= 4096 && ranks >= 8) ? 2 : 1;
    }
    if (out->sharded_us > out->single_us) {   // sharding would slow this operator down: every rank keeps the whole weight
        out->mode = MAGB200_TP_REPLICATE; out->exchange = MAGB200_TP_EXCHANGE_NONE; out->sharded_us = out->single_us; out->chunks = 1;
    }
    out->speedup = out->single_us / out->sharded_us;
    out->pays = out->speedup >= 0.5 * p ? 1 : 0;   // at least half of linear scaling
    return MAGB200_OK;
}

int magb200_multimem_reduce_broadcast(int device, void *cuda_stream, const void *mc_partial, void *mc_out, int nranks, int rank,
                                      int64_t rows_per_rank, int64_t n, int dtype, int max_ctas) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if (rows_per_rank < 1 || n < 1) { set_error("multimem_reduce_broadcast: empty block"); return MAGB200_ERR_INVALID_ARG; }
    return launch_multimem_reduce_broadcast(dtype, mc_partial, mc_out, nranks, rank, rows_per_rank * n, max_ctas,
                                            cuda_stream ? (cudaStream_t)cuda_stream : d->stream);
}

int magb200_last_kernel(void) { return g_last_kernel; }
uint64_t magb200_launch_count(void) { return g_launches.load(); }
void magb200_launch_count_reset(void) { g_launches.store(0); }
int magb200_set_gemm_overlap(int on) {
    g_gemm_overlap.store(on ? 1 : 0);
    return MAGB200_OK;
}
uint64_t magb200_overlapped_launch_count(void) { return g_overlapped_launches.load(); }
int magb200_set_small_output_split(int on) {
    set_split_small(on);
    return MAGB200_OK;
}
int magb200_matmul_route(const magb200_view_t *x, const magb200_view_t *y, int *kernel, int *repacked) {
    if (!x || !y || !kernel || !repacked) { set_error("matmul_route: null argument"); return MAGB200_ERR_INVALID_ARG; }
    int32_t rank = 0;
    int64_t shape[MAGB200_MAX_DIMS + 2];
    int rc = magb200_matmul_result_shape(x, y, &rank, shape);
    if (rc) return rc;
    magb200_view_t r;
    memset(&r, 0, sizeof(r));
    alignas(16) static char unused[16];
    r.base = unused; r.dtype = x->dtype; r.rank = rank;
    int64_t acc = 1;
    for (int i = rank - 1; i >= 0; --i) { r.shape[i] = shape[i]; r.strides[i] = acc; acc *= shape[i]; }
    FullProblem fp;
    if ((rc = build_problem(x, y, &r, fp))) return rc;
    if ((rc = route(fp.g, 0, kernel))) return rc;
    *repacked = 0;
    const GemmProblem &g = fp.g;
    // the detour of run_packed: a 16-bit product that fell to the FFMA kernel only because TMA cannot describe an operand
    if (*kernel == MAGB200_KERNEL_SIMT && g.dtype != MAGB200_F32 && g.M > 8 &&
        (double)g.M * (double)g.N * (double)g.K * (double)g.batch_total >= (double)(1 << 24) &&
        (!tcgen05_operand_ok(g, true) || !tcgen05_operand_ok(g, false))) {
        *repacked = 1;
        GemmProblem gp = g;
        const int64_t kpad = (g.K + 7) / 8 * 8;
        if (!tcgen05_operand_ok(g, true)) { gp.sAm = kpad; gp.sAk = 1; gp.A = unused; }
        if (!tcgen05_operand_ok(g, false)) { gp.sBn = kpad; gp.sBk = 1; gp.B = unused; }
        *kernel = tcgen05_2sm_preferred(gp) ? MAGB200_KERNEL_TCGEN05_2SM : MAGB200_KERNEL_TCGEN05;
    }
    return MAGB200_OK;
}

int magb200_decode_plan(const magb200_view_t *x, const magb200_view_t *y, int *kind, int *k_splits, int *ctas, int *warps_along_k, int *cluster,
                        int64_t *k_chunk) {
    if (!x || !y || !kind || !k_splits || !ctas || !warps_along_k || !cluster || !k_chunk) { set_error("decode_plan: null argument"); return MAGB200_ERR_INVALID_ARG; }
    int32_t rank = 0;
    int64_t shape[MAGB200_MAX_DIMS + 2];
    int rc = magb200_matmul_result_shape(x, y, &rank, shape);
    if (rc) return rc;
    magb200_view_t r;
    memset(&r, 0, sizeof(r));
    alignas(16) static char unused[16];
    r.base = unused; r.dtype = x->dtype; r.rank = rank;
    int64_t acc = 1;
    for (int i = rank - 1; i >= 0; --i) { r.shape[i] = shape[i]; r.strides[i] = acc; acc *= shape[i]; }
    FullProblem fp;
    if ((rc = build_problem(x, y, &r, fp))) return rc;
    return describe_skinny_plan(fp.g, kind, k_splits, ctas, warps_along_k, cluster, k_chunk);
}
int magb200_set_decode_row_streaming(int on) {
    set_decode_row_streaming(on);
    return MAGB200_OK;
}
int magb200_set_decode_cluster(int max_cluster) {
    if (max_cluster != 1 && max_cluster != 2 && max_cluster != 4) { set_error("set_decode_cluster: 1, 2 or 4"); return MAGB200_ERR_INVALID_ARG; }
    set_decode_cluster_max(max_cluster);
    return MAGB200_OK;
}
int magb200_force_kernel(int kernel) {
    if (kernel < 0 || kernel > MAGB200_KERNEL_TCGEN05_F32X3) { set_error("force_kernel: unknown kernel %d", kernel); return MAGB200_ERR_INVALID_ARG; }
    g_force.store(kernel);
    return MAGB200_OK;
}

int magb200_matmul_host(int device, const magb200_view_t *x, size_t x_bytes, const magb200_view_t *y, size_t y_bytes, const magb200_view_t *r) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if ((rc = check_view(x, "matmul x")) || (rc = check_view(y, "matmul y")) || (rc = check_view(r, "matmul result"))) return rc;
    const size_t r_bytes = (size_t)view_numel(r) * dtype_size(r->dtype);
    if ((rc = check_view_fits(x, x_bytes, "matmul x")) || (rc = check_view_fits(y, y_bytes, "matmul y"))) return rc;
    if (!view_is_contiguous(r)) { set_error("matmul: result must be contiguous"); return MAGB200_ERR_INVALID_ARG; }
    if ((rc = ensure_staging(*d, 0, x_bytes)) || (rc = ensure_staging(*d, 1, y_bytes)) || (rc = ensure_staging(*d, 2, r_bytes))) return rc;
    MAGB200_CUDA_TRY(cudaMemcpyAsync(d->staging[0], x->base, x_bytes, cudaMemcpyHostToDevice, d->stream));
    MAGB200_CUDA_TRY(cudaMemcpyAsync(d->staging[1], y->base, y_bytes, cudaMemcpyHostToDevice, d->stream));
    magb200_view_t dx = *x, dy = *y, dr = *r;
    dx.base = d->staging[0]; dy.base = d->staging[1]; dr.base = d->staging[2]; dr.offset = 0;
    if ((rc = matmul_device(*d, device, &dx, &dy, &dr))) return rc;
    MAGB200_CUDA_TRY(cudaMemcpyAsync(view_data(r), d->staging[2], r_bytes, cudaMemcpyDeviceToHost, d->stream));
    MAGB200_CUDA_TRY(cudaStreamSynchronize(d->stream));
    return check_status_word(*d);
}

int magb200_cast_host(int device, const magb200_view_t *src, size_t src_bytes, const magb200_view_t *dst) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if ((rc = check_view(src, "cast source")) || (rc = check_view(dst, "cast result"))) return rc;
    const size_t dst_bytes = (size_t)view_numel(dst) * dtype_size(dst->dtype);
    if ((rc = check_view_fits(src, src_bytes, "cast source"))) return rc;
    if (!view_is_contiguous(dst)) { set_error("cast: result must be contiguous"); return MAGB200_ERR_INVALID_ARG; }
    if ((rc = ensure_staging(*d, 0, src_bytes)) || (rc = ensure_staging(*d, 2, dst_bytes))) return rc;
    MAGB200_CUDA_TRY(cudaMemcpyAsync(d->staging[0], src->base, src_bytes, cudaMemcpyHostToDevice, d->stream));
    magb200_view_t ds = *src, dd = *dst;
    ds.base = d->staging[0]; dd.base = d->staging[2]; dd.offset = 0;
    if ((rc = cast_device(*d, &ds, &dd, false))) return rc;
    MAGB200_CUDA_TRY(cudaMemcpyAsync(view_data(dst), d->staging[2], dst_bytes, cudaMemcpyDeviceToHost, d->stream));
    MAGB200_CUDA_TRY(cudaStreamSynchronize(d->stream));
    return MAGB200_OK;
}

int magb200_graph_begin_capture(int device) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if (d->capturing) { set_error("graph capture is already active on device %d", device); return MAGB200_ERR_INVALID_ARG; }
    MAGB200_CUDA_TRY(cudaStreamBeginCapture(d->stream, cudaStreamCaptureModeThreadLocal));
    d->capturing = true;
    return MAGB200_OK;
}
int magb200_graph_end_capture(int device, void **out_graph) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if (!d->capturing || !out_graph) { set_error("graph_end_capture without a capture in progress"); return MAGB200_ERR_INVALID_ARG; }
    d->capturing = false;
    cudaGraph_t graph = nullptr;
    MAGB200_CUDA_TRY(cudaStreamEndCapture(d->stream, &graph));
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGraphInstantiate", __FILE__, __LINE__);
    *out_graph = (void *)exec;
    return MAGB200_OK;
}
int magb200_graph_launch(int device, void *graph) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    if (!graph) { set_error("graph_launch: null graph"); return MAGB200_ERR_INVALID_ARG; }
    MAGB200_CUDA_TRY(cudaGraphLaunch((cudaGraphExec_t)graph, d->stream));
    return MAGB200_OK;
}
int magb200_graph_destroy(void *graph) {
    if (graph) MAGB200_CUDA_TRY(cudaGraphExecDestroy((cudaGraphExec_t)graph));
    return MAGB200_OK;
}

int magb200_event_create(void **out) {
    if (!out) { set_error("event_create: null out pointer"); return MAGB200_ERR_INVALID_ARG; }
    cudaEvent_t e;
    MAGB200_CUDA_TRY(cudaEventCreate(&e));
    *out = (void *)e;
    return MAGB200_OK;
}
int magb200_event_destroy(void *event) {
    if (event) MAGB200_CUDA_TRY(cudaEventDestroy((cudaEvent_t)event));
    return MAGB200_OK;
}
int magb200_event_record(int device, void *event) {
    DeviceState *d;
    int rc = ensure_device(device, &d);
    if (rc) return rc;
    MAGB200_CUDA_TRY(cudaEventRecord((cudaEvent_t)event, d->stream));
    return MAGB200_OK;
}
int magb200_event_elapsed_ms(void *start, void *stop, float *out_ms) {
    MAGB200_CUDA_TRY(cudaEventSynchronize((cudaEvent_t)stop));
    MAGB200_CUDA_TRY(cudaEventElapsedTime(out_ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return MAGB200_OK;
}

}  // extern "C"
