// Decode-shaped matmul for callers that must not allocate device memory.
//
// Who needs this: code that runs where cudaMalloc is off limits -- a plug-in called from inside another
// framework's stream-ordered region or memory pool, a real-time serving loop that is forbidden to touch
// the allocator once it is warm, a host thread that is not allowed to take the driver's allocation lock.
// The regular magb200_matmul may create its per-device stream and workspace on first use and may grow
// the split-K workspace; this entry point never does. Its split-K partial sums live in a fixed array that
// is part of the library image, so every GPU that loads the library carries these 4 MiB until exit.
//
// Limits and rules of use:
//   * the problem must be one the skinny kernels take (M <= 8, 16-byte aligned unit-stride weights) and
//     its partial sums, splits x batch x M x N floats, must fit kNoAllocScratchFloats; larger problems
//     are refused with MAGB200_ERR_TOO_LARGE and a message that names both numbers;
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
//     device current). That first call should be made before any stream capture begins;
//   * all calls share the one array and it keeps whatever the previous call left. Nothing in it has to start
//     at zero: each call's first kernel writes every partial sum that its second kernel reads. Two calls
//     whose kernels overlap on the GPU (different streams, or different host threads) race on the array;
//     keep calls on one stream or order them yourself;
//   * the call makes `device` the calling thread's current CUDA device and leaves it so; a NULL stream means the legacy
//     default stream here (the library's own per-device stream is used only by the entry points that own one).
#include "common.cuh"

#include <atomic>
#include <mutex>

namespace magb200 {

int canonicalize_skinny_problem(const magb200_view_t *x, const magb200_view_t *y, const magb200_view_t *r, GemmProblem *out);  // cabi.cu
size_t skinny_scratch_bytes(const GemmProblem &p);                                                                         // gemv.cu

namespace {

constexpr size_t kNoAllocScratchFloats = 1u << 20;  // 4 MiB of fp32 partial sums

// In host code this name is only a handle for the runtime, not a device address: it is never passed to a
// kernel. The address comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocScratchFloats];

constexpr int kMaxDev = 16;
std::atomic<float *> g_scratch_ptr[kMaxDev];
std::mutex g_setup_mu;

// Makes `device` current (the launch below needs that anyway) and returns the array's address there. Only the first call on
// a device takes the lock and asks the runtime; later calls read the cached address.
int scratch_address(int device, float **out) {
    if (device < 0 || device >= kMaxDev) { set_error("device %d out of range", device); return MAGB200_ERR_INVALID_ARG; }
    if (cudaSetDevice(device) != cudaSuccess) {
        (void)cudaGetLastError();
        set_error("no CUDA device %d: this library has no CPU fallback", device);
        return MAGB200_ERR_NO_DEVICE;
    }
    float *ptr = g_scratch_ptr[device].load(std::memory_order_acquire);
    if (!ptr) {
        std::lock_guard<std::mutex> lock(g_setup_mu);
        ptr = g_scratch_ptr[device].load(std::memory_order_relaxed);
        if (!ptr) {
            cudaDeviceProp prop;
            MAGB200_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
            if (prop.major != 10) { set_error("device %d (%s) is sm_%d%d; the kernels are built for sm_100a only", device, prop.name, prop.major, prop.minor); return MAGB200_ERR_NO_DEVICE; }
            // the symbol has one instance per device; with `device` current this is that device's
            MAGB200_CUDA_TRY(cudaGetSymbolAddress((void **)&ptr, g_noalloc_scratch));
            if (!ptr) { set_error("cudaGetSymbolAddress returned a null address for the built-in scratch array"); return MAGB200_ERR_CUDA; }
            g_scratch_ptr[device].store(ptr, std::memory_order_release);
        }
    }
    *out = ptr;
    return MAGB200_OK;
}

}  // namespace
}  // namespace magb200

using namespace magb200;

extern "C" __attribute__((visibility("default")))
int magb200_matmul_skinny_noalloc(int device, void *cuda_stream, const magb200_view_t *x, const magb200_view_t *y,
                                  const magb200_view_t *r) {
    GemmProblem g;
    int rc = canonicalize_skinny_problem(x, y, r, &g);
    if (rc) return rc;
    if (g.M > 8 || !skinny_supported(g)) {
        set_error("matmul_skinny_noalloc: only decode-shaped products run here (M <= 8 after folding, unit-stride 16-byte aligned "
                  "weights); got M=%lld N=%lld K=%lld", (long long)g.M, (long long)g.N, (long long)g.K);
        return MAGB200_ERR_INVALID_ARG;
    }
    const size_t need = skinny_scratch_bytes(g);
    if (need > kNoAllocScratchFloats * sizeof(float)) {
        set_error("matmul_skinny_noalloc: the split-K partial sums of this problem need %zu bytes, the built-in scratch array holds %zu; "
                  "use magb200_matmul, which may allocate", need, kNoAllocScratchFloats * sizeof(float));
        return MAGB200_ERR_TOO_LARGE;
    }
    float *scratch = nullptr;
    if ((rc = scratch_address(device, &scratch))) return rc;
    // the caller's stream is not tracked by this library: whether an earlier kernel on it still writes y is unknown, so the
    // kernels read the weights only after they have waited for their predecessors
    return launch_skinny(g, (cudaStream_t)cuda_stream, scratch, kNoAllocScratchFloats * sizeof(float), nullptr, /*weights_settled=*/false);
}
