/*
 * magnetron backend module for NVIDIA B200: takes the "cuda" slot of magnetron's backend registry.
 *
 * Built as libmagnetron_cuda.so and dropped next to libmagnetron_core.so, it is found by
 * mag_backend_registry_init (magnetron/core/mag_backend.c:205-251) and selected with
 * mag_ctx_create("cuda:N"). It implements the module ABI of magnetron/core/mag_backend.h:
 *
 *   mag_backend_module_hook_abi_cookie / _init / _shutdown      mag_backend.h:117-140
 *   mag_backend_t  {init, shutdown, versions, id, num_devices, best_device_id, get_device}  :101-113
 *   mag_device_t   {submit, alloc_storage, manual_seed}          :90-99
 *
 * following the reference CPU module as the model of the boundary (magnetron/cpu/mag_cpu.c:70-238):
 * storage headers come from the context's slab, are reference counted, and keep
 * telemetry.num_alive_storages balanced. Only the matmul / cast path runs here: MATMUL, CAST, CLONE and
 * FILL on {float32, float16, bfloat16} go to the sm_100a kernels through the C ABI of
 * include/magnetron_b200.h; the header-only view opcodes are accepted as no-ops; every other opcode
 * returns MAG_STATUS_ERR_OPERATOR_IMPOSSIBLE with a log line instead of aborting the process.
 *
 * This file is C host code compiled against the magnetron headers where they lie (-I to the magnetron
 * source tree); nothing of magnetron is copied into this repository. It must be compiled with the same
 * NDEBUG setting as the core, because MAG_DEBUG changes the layout of the reference-counted headers
 * (magnetron/core/mag_rc.h:22-28).
 *
 * The module ABI has no transfer entry (mag_backend.h:90-99) and the core's host-access calls refuse
 * non-CPU storage (mag_copy_raw_, magnetron/core/mag_op_stubs.c:1365-1374), so this module additionally
 * exports mag_b200_upload / mag_b200_download (and their _async forms on the copy streams) / mag_b200_synchronize for
 * callers that hold device tensors.
 */
#include <core/mag_backend.h>
#include <core/mag_context.h>
#include <core/mag_tensor.h>
#include <core/mag_alloc.h>

#include "magnetron_b200.h"

#include <stdio.h>
#include <string.h>

#define MAG_B200_BACKEND_VERSION mag_ver_encode(0, 1, 0)
#define MAG_B200_MAX_DEVICES 16
#define MAG_B200_MAX_CAT 64

typedef struct mag_b200_device_t {
    mag_device_t iface;     /* handed to the core; must outlive the context's tensors */
    int ordinal;
} mag_b200_device_t;

typedef struct mag_b200_backend_t {
    mag_context_t *ctx;
    uint32_t num_devices;
    mag_b200_device_t devices[MAG_B200_MAX_DEVICES];
} mag_b200_backend_t;

/* ---- status mapping --------------------------------------------------------------------------
 * Every C-ABI code has one magnetron status of its own, so a caller can tell the causes apart:
 *   out of device memory -> ERR_MEMORY_ALLOCATION_FAILED     shapes that form no matmul / cast -> ERR_OPERATOR_IMPOSSIBLE
 *   bad argument         -> ERR_INVALID_PARAM                beyond a fixed capacity            -> ERR_DIM_OVERFLOW
 *   a bounded device-side wait ran out (results of that launch are invalid, the device stays usable) -> ERR_INVALID_STATE
 *   no such device       -> ERR_INVALID_INDEX                any other CUDA runtime failure     -> ERR_UNKNOWN
 * Exported so that the mapping can be checked without a device. */
MAG_EXPORT mag_status_t mag_b200_status_of(int rc) {
    switch (rc) {
        case MAGB200_OK:              return MAG_STATUS_OK;
        case MAGB200_ERR_OOM:         return MAG_STATUS_ERR_MEMORY_ALLOCATION_FAILED;
        case MAGB200_ERR_SHAPE:       return MAG_STATUS_ERR_OPERATOR_IMPOSSIBLE;
        case MAGB200_ERR_INVALID_ARG: return MAG_STATUS_ERR_INVALID_PARAM;
        case MAGB200_ERR_TOO_LARGE:   return MAG_STATUS_ERR_DIM_OVERFLOW;
        case MAGB200_ERR_TIMEOUT:     return MAG_STATUS_ERR_INVALID_STATE;
        case MAGB200_ERR_NO_DEVICE:   return MAG_STATUS_ERR_INVALID_INDEX;
        default:                      return MAG_STATUS_ERR_UNKNOWN;
    }
}

static mag_status_t mag_b200_map_status(int rc, const char *what) {
    if (rc == MAGB200_OK) return MAG_STATUS_OK;
    mag_log_error("b200 backend: %s failed (%d): %s", what, rc, magb200_last_error());
    return mag_b200_status_of(rc);
}

/* ---- tensor header -> view ------------------------------------------------------------------- */
static bool mag_b200_dtype_ok(mag_dtype_t t) {
    return t == MAG_DTYPE_FLOAT32 || t == MAG_DTYPE_FLOAT16 || t == MAG_DTYPE_BFLOAT16;
}

static void mag_b200_view_of(const mag_tensor_t *t, magb200_view_t *v) {
    memset(v, 0, sizeof(*v));
    v->base = (void *)t->storage->base;
    v->offset = t->storage_offset;
    v->dtype = (int32_t)t->dtype;       /* MAGB200_F32/F16/BF16 share mag_dtype_t's values */
    v->rank = (int32_t)t->coords.rank;
    for (int64_t i = 0; i < t->coords.rank; ++i) {
        v->shape[i] = t->coords.shape[i];
        v->strides[i] = t->coords.strides[i];
    }
}

/* ---- submit ---------------------------------------------------------------------------------- */
static mag_status_t mag_b200_unsupported(const mag_command_t *cmd, const char *why) {
    mag_log_error("b200 backend: opcode %d %s; this module implements MATMUL, CAST, CLONE, CAT, FILL and the view opcodes", (int)cmd->op, why);
    return MAG_STATUS_ERR_OPERATOR_IMPOSSIBLE;
}

static mag_status_t mag_b200_submit(mag_device_t *dvc, const mag_command_t *cmd) {
    const int dev = ((mag_b200_device_t *)dvc->impl)->ordinal;
    magb200_view_t x, y, r;
    switch (cmd->op) {
        case MAG_OP_NOP:
        case MAG_OP_VIEW:
        case MAG_OP_TRANSPOSE:
        case MAG_OP_PERMUTE:
            return MAG_STATUS_OK;   /* header-only: the core already built the new tensor header */
        case MAG_OP_MATMUL:
            if (cmd->num_in != 2 || cmd->num_out != 1) return MAG_STATUS_ERR_INVALID_PARAM;
            if (!mag_b200_dtype_ok(cmd->in[0]->dtype)) return mag_b200_unsupported(cmd, "has a non floating point dtype");
            mag_b200_view_of(cmd->in[0], &x);
            mag_b200_view_of(cmd->in[1], &y);
            mag_b200_view_of(cmd->out[0], &r);
            return mag_b200_map_status(magb200_matmul(dev, &x, &y, &r), "matmul");
        case MAG_OP_CAST:
        case MAG_OP_CLONE:
            if (cmd->num_in != 1 || cmd->num_out != 1) return MAG_STATUS_ERR_INVALID_PARAM;
            if (!mag_b200_dtype_ok(cmd->in[0]->dtype) || !mag_b200_dtype_ok(cmd->out[0]->dtype))
                return mag_b200_unsupported(cmd, "has a dtype outside {float32, float16, bfloat16}");
            mag_b200_view_of(cmd->in[0], &x);
            mag_b200_view_of(cmd->out[0], &r);
            return mag_b200_map_status(cmd->op == MAG_OP_CAST ? magb200_cast(dev, &x, &r) : magb200_clone(dev, &x, &r),
                                       cmd->op == MAG_OP_CAST ? "cast" : "clone");
        case MAG_OP_CAT: {
            /* mag_cat (magnetron/core/mag_op_stubs.c:996-1030): contiguous inputs of one dtype, attrs[0] = the dim; the
             * KV-cache append of the Qwen3 example (examples/qwen3/model.py:126-127) arrives here */
            if (cmd->num_in < 1 || cmd->num_in > MAG_B200_MAX_CAT || cmd->num_out != 1) return mag_b200_unsupported(cmd, "has too many inputs for the device concat");
            if (!mag_b200_dtype_ok(cmd->out[0]->dtype)) return mag_b200_unsupported(cmd, "has a dtype outside {float32, float16, bfloat16}");
            if (cmd->attrs[0].tag != MAG_OP_ATTR_TYPE_I64) return MAG_STATUS_ERR_INVALID_PARAM;
            magb200_view_t parts[MAG_B200_MAX_CAT];
            const magb200_view_t *ptrs[MAG_B200_MAX_CAT];
            for (uint32_t i = 0; i < cmd->num_in; ++i) { mag_b200_view_of(cmd->in[i], &parts[i]); ptrs[i] = &parts[i]; }
            mag_b200_view_of(cmd->out[0], &r);
            return mag_b200_map_status(magb200_cat(dev, ptrs, (int)cmd->num_in, (int)mag_op_attr_unwrap_int64(cmd->attrs[0]), &r), "cat");
        }
        case MAG_OP_FILL:
            if (cmd->num_out != 1) return MAG_STATUS_ERR_INVALID_PARAM;
            if (!mag_b200_dtype_ok(cmd->out[0]->dtype)) return mag_b200_unsupported(cmd, "has a non floating point dtype");
            if (cmd->attrs[0].tag != MAG_OP_ATTR_TYPE_FLOAT64) return MAG_STATUS_ERR_INVALID_PARAM;
            mag_b200_view_of(cmd->out[0], &r);
            return mag_b200_map_status(magb200_fill(dev, &r, cmd->attrs[0].value.float64), "fill");
        default:
            return mag_b200_unsupported(cmd, "is outside the matmul / cast path");
    }
}

/* ---- storage --------------------------------------------------------------------------------- */
static mag_status_t mag_b200_storage_dtor(void *self) {
    mag_storage_buffer_t *buf = self;
    mag_context_t *ctx = buf->ctx;
    const int dev = ((mag_b200_device_t *)buf->device->impl)->ordinal;
    mag_status_t st = MAG_STATUS_OK;
    if (ctx->telemetry.num_alive_storages > 0) --ctx->telemetry.num_alive_storages;
    if (magb200_free(dev, (void *)buf->base) != MAGB200_OK) {
        mag_log_error("b200 backend: freeing device storage failed: %s", magb200_last_error());
        st = MAG_STATUS_ERR_MEMORY_DEALLOCATION_FAILED;
    }
    mag_slab_free(&ctx->storage_slab, buf);
    return st;
}

static mag_status_t mag_b200_alloc_storage(mag_device_t *dvc, mag_storage_buffer_t **out, size_t size, mag_dtype_t dtype) {
    (void)dtype;
    mag_context_t *ctx = dvc->ctx;
    const int dev = ((mag_b200_device_t *)dvc->impl)->ordinal;
    void *base = NULL;
    int rc = magb200_malloc(dev, &base, size);
    if (rc != MAGB200_OK) return mag_b200_map_status(rc, "device allocation");
    mag_storage_buffer_t *buf = mag_slab_alloc(&ctx->storage_slab);
    memset(buf, 0, sizeof(*buf));
    buf->ctx = ctx;
    buf->flags = MAG_STORAGE_FLAG_ACCESS_W;
    buf->alignment = 256;
    buf->base = (uintptr_t)base;
    buf->size = size;
    buf->device = dvc;
    mag_rc_init_object(buf, &mag_b200_storage_dtor);
    ++ctx->telemetry.num_alive_storages;
    ctx->telemetry.storage_bytes_allocated += size;
    *out = buf;
    return MAG_STATUS_OK;
}

static void mag_b200_manual_seed(mag_device_t *dvc, uint64_t seed) {
    (void)dvc; (void)seed;   /* no random fills on this path: operands are uploaded */
}

/* ---- backend vtable -------------------------------------------------------------------------- */
static bool mag_b200_init(mag_backend_t *self, mag_context_t *ctx) {
    mag_b200_backend_t *b = self->impl;
    b->ctx = ctx;
    int n = magb200_device_count();
    if (n > MAG_B200_MAX_DEVICES) n = MAG_B200_MAX_DEVICES;
    if (n <= 0) {
        mag_log_info("b200 backend: no sm_100 device visible; the cuda backend stays unavailable");
        return false;
    }
    b->num_devices = 0;
    for (int i = 0; i < n; ++i) {
        if (magb200_device_init(i) != MAGB200_OK) {
            mag_log_error("b200 backend: device %d failed to initialise: %s", i, magb200_last_error());
            break;
        }
        mag_b200_device_t *d = &b->devices[i];
        memset(d, 0, sizeof(*d));
        d->ordinal = i;
        d->iface.impl = d;
        d->iface.ctx = ctx;
        d->iface.id.type = MAG_BACKEND_TYPE_CUDA;
        d->iface.id.device_ordinal = (uint32_t)i;
        d->iface.is_async = true;   /* launches are stream ordered; download / synchronize wait */
        d->iface.submit = &mag_b200_submit;
        d->iface.alloc_storage = &mag_b200_alloc_storage;
        d->iface.manual_seed = &mag_b200_manual_seed;
        magb200_device_name(i, d->iface.physical_device_name, sizeof(d->iface.physical_device_name));
        ++b->num_devices;
    }
    return b->num_devices > 0;
}

static bool mag_b200_shutdown(mag_backend_t *self) {
    mag_b200_backend_t *b = self->impl;
    for (uint32_t i = 0; i < b->num_devices; ++i) magb200_synchronize((int)i);
    /* the per-device streams and workspaces are process-wide and shared by every context: they stay */
    return true;
}

static uint32_t mag_b200_backend_version(mag_backend_t *bck) { (void)bck; return MAG_B200_BACKEND_VERSION; }
static uint32_t mag_b200_runtime_version(mag_backend_t *bck) { (void)bck; return MAG_VERSION; }
static const char *mag_b200_id(mag_backend_t *bck) { (void)bck; return "cuda"; }
static uint32_t mag_b200_num_devices(mag_backend_t *bck) { return ((mag_b200_backend_t *)bck->impl)->num_devices; }
static uint32_t mag_b200_best_device(mag_backend_t *bck) { (void)bck; return 0; }
static mag_device_t *mag_b200_get_device(mag_backend_t *bck, uint32_t idx) {
    mag_b200_backend_t *b = bck->impl;
    return idx < b->num_devices ? &b->devices[idx].iface : NULL;
}

/* ---- module hooks ---------------------------------------------------------------------------- */
MAG_EXPORT uint32_t MAG_BACKEND_SYM_ABI_COOKIE(void) {
    return mag_pack_abi_cookie('M', 'A', 'G', MAG_BACKEND_MODULE_ABI_VER);
}

MAG_EXPORT mag_backend_t *MAG_BACKEND_SYM_INIT(mag_context_t *ctx) {
    (void)ctx;
    mag_backend_t *backend = (*mag_alloc)(NULL, sizeof(*backend) + sizeof(mag_b200_backend_t), 0);
    memset(backend, 0, sizeof(*backend) + sizeof(mag_b200_backend_t));
    backend->impl = backend + 1;
    backend->init = &mag_b200_init;
    backend->shutdown = &mag_b200_shutdown;
    backend->backend_version = &mag_b200_backend_version;
    backend->runtime_version = &mag_b200_runtime_version;
    backend->id = &mag_b200_id;
    backend->num_devices = &mag_b200_num_devices;
    backend->best_device_id = &mag_b200_best_device;
    backend->get_device = &mag_b200_get_device;
    return backend;
}

MAG_EXPORT void MAG_BACKEND_SYM_SHUTDOWN(mag_backend_t *backend) {
    (*mag_alloc)(backend, 0, 0);
}

/* ---- additive exports: data movement for device tensors --------------------------------------
 * Counterparts of mag_copy_raw_ (magnetron/core/mag_op_stubs.c:1365-1374) and mag_tensor_copy_data
 * (magnetron/core/mag_tensor.c:232-250) for tensors whose storage lives on this backend. The tensor must
 * be contiguous; `size_bytes` must equal numel * sizeof(dtype). */
static int mag_b200_check_transfer(const mag_tensor_t *t, size_t size_bytes, const char *what) {
    if (!t || !t->storage || t->storage->device->id.type != MAG_BACKEND_TYPE_CUDA) {
        mag_log_error("%s: tensor storage is not on the cuda backend", what);
        return 0;
    }
    if (!mag_tensor_is_contiguous(t)) { mag_log_error("%s: tensor must be contiguous", what); return 0; }
    const size_t want = (size_t)t->numel * mag_type_trait(t->dtype)->size;
    if (want != size_bytes) { mag_log_error("%s: %zu bytes given, tensor holds %zu", what, size_bytes, want); return 0; }
    return 1;
}

MAG_EXPORT mag_status_t mag_b200_upload(mag_tensor_t *tensor, const void *host_data, size_t size_bytes) {
    if (!host_data || !mag_b200_check_transfer(tensor, size_bytes, "mag_b200_upload")) return MAG_STATUS_ERR_INVALID_PARAM;
    const int dev = ((mag_b200_device_t *)tensor->storage->device->impl)->ordinal;
    char *dst = (char *)tensor->storage->base + tensor->storage_offset * (int64_t)mag_type_trait(tensor->dtype)->size;
    return mag_b200_map_status(magb200_upload(dev, dst, host_data, size_bytes), "upload");
}

MAG_EXPORT mag_status_t mag_b200_download(const mag_tensor_t *tensor, void *host_data, size_t size_bytes) {
    if (!host_data || !mag_b200_check_transfer(tensor, size_bytes, "mag_b200_download")) return MAG_STATUS_ERR_INVALID_PARAM;
    const int dev = ((mag_b200_device_t *)tensor->storage->device->impl)->ordinal;
    const char *src = (const char *)tensor->storage->base + tensor->storage_offset * (int64_t)mag_type_trait(tensor->dtype)->size;
    return mag_b200_map_status(magb200_download(dev, host_data, src, size_bytes), "download");
}

/* The same transfers without waiting: they run on the module's copy streams beside the kernels of other operators and
 * beside each other (the link is full duplex). The upload is ordered after the operators submitted so far and before the
 * ones submitted later; the download is ordered after the operators submitted so far. `host_data` must be page-locked
 * (mag_b200_host_alloc) and stay untouched until mag_b200_synchronize returns; the tensor may be released right after the
 * call -- its storage is not handed to a later writer before the copy has read it. */
MAG_EXPORT mag_status_t mag_b200_upload_async(mag_tensor_t *tensor, const void *host_data, size_t size_bytes) {
    if (!host_data || !mag_b200_check_transfer(tensor, size_bytes, "mag_b200_upload_async")) return MAG_STATUS_ERR_INVALID_PARAM;
    const int dev = ((mag_b200_device_t *)tensor->storage->device->impl)->ordinal;
    char *dst = (char *)tensor->storage->base + tensor->storage_offset * (int64_t)mag_type_trait(tensor->dtype)->size;
    return mag_b200_map_status(magb200_upload_overlapped(dev, dst, host_data, size_bytes), "upload");
}

MAG_EXPORT mag_status_t mag_b200_download_async(const mag_tensor_t *tensor, void *host_data, size_t size_bytes) {
    if (!host_data || !mag_b200_check_transfer(tensor, size_bytes, "mag_b200_download_async")) return MAG_STATUS_ERR_INVALID_PARAM;
    const int dev = ((mag_b200_device_t *)tensor->storage->device->impl)->ordinal;
    const char *src = (const char *)tensor->storage->base + tensor->storage_offset * (int64_t)mag_type_trait(tensor->dtype)->size;
    return mag_b200_map_status(magb200_download_overlapped(dev, host_data, src, size_bytes), "download");
}

/* Additive export: the gated MLP out = silu(x @ w_gate) * (x @ w_up) as one call, for callers that would otherwise issue
 * mag_matmul, mag_matmul, mag_silu, mag_mul (examples/qwen3/model.py:48-49); same result as that sequence. `out` is a
 * contiguous tensor of the product's shape on this backend (mag_empty). */
MAG_EXPORT mag_status_t mag_b200_matmul_swiglu(mag_tensor_t *x, mag_tensor_t *w_gate, mag_tensor_t *w_up, mag_tensor_t *out) {
    mag_tensor_t *all[4] = {x, w_gate, w_up, out};
    for (int i = 0; i < 4; ++i)
        if (!all[i] || !all[i]->storage || all[i]->storage->device->id.type != MAG_BACKEND_TYPE_CUDA) {
            mag_log_error("mag_b200_matmul_swiglu: every tensor must live on the cuda backend");
            return MAG_STATUS_ERR_INVALID_PARAM;
        }
    magb200_view_t vx, vg, vu, vr;
    mag_b200_view_of(x, &vx);
    mag_b200_view_of(w_gate, &vg);
    mag_b200_view_of(w_up, &vu);
    mag_b200_view_of(out, &vr);
    const int dev = ((mag_b200_device_t *)out->storage->device->impl)->ordinal;
    return mag_b200_map_status(magb200_matmul_swiglu(dev, &vx, &vg, &vu, &vr), "matmul_swiglu");
}

/* Additive export: a tensor that lives on the CPU backend -- typically one handed out by mag_snapshot_deserialize, which
 * maps the .mag file and works on a CPU context only (magnetron/core/mag_snapshot.c:566-640) -- becomes a tensor of the cuda
 * context `ctx`, whole (shard_dim < 0) or as one rank's equal share of dimension `shard_dim` (rank `shard` of `shards`: the
 * row block of a column-sharded nn.Linear weight [N, K] is shard_dim 0, the K slice of a row-sharded one shard_dim 1). The
 * bytes go straight from the mapped file to device memory; a slice of an inner dim is a pitched copy. `src` must be
 * contiguous. */
MAG_EXPORT mag_status_t mag_b200_tensor_to_device(mag_context_t *ctx, const mag_tensor_t *src, int64_t shard_dim, int64_t shard, int64_t shards,
                                                  mag_tensor_t **out) {
    if (!ctx || !ctx->active_device || ctx->active_device->id.type != MAG_BACKEND_TYPE_CUDA || !src || !out || !src->storage ||
        src->storage->device->id.type != MAG_BACKEND_TYPE_CPU || !mag_tensor_is_contiguous(src)) {
        mag_log_error("mag_b200_tensor_to_device: needs a cuda context and a contiguous tensor of the CPU backend");
        return MAG_STATUS_ERR_INVALID_PARAM;
    }
    const int64_t rank = src->coords.rank;
    int64_t shape[MAG_MAX_DIMS];
    for (int64_t i = 0; i < rank; ++i) shape[i] = src->coords.shape[i];
    int64_t outer = 1, inner = 1, len = 1, first = 0;
    if (shard_dim >= 0) {
        if (shard_dim >= rank || shards < 1 || shard < 0 || shard >= shards || shape[shard_dim] % shards) {
            mag_log_error("mag_b200_tensor_to_device: dimension %lld of extent %lld cannot be cut into %lld equal shards",
                          (long long)shard_dim, (long long)(shard_dim < rank ? shape[shard_dim] : -1), (long long)shards);
            return MAG_STATUS_ERR_INVALID_PARAM;
        }
        len = shape[shard_dim];
        for (int64_t i = 0; i < shard_dim; ++i) outer *= shape[i];
        for (int64_t i = shard_dim + 1; i < rank; ++i) inner *= shape[i];
        shape[shard_dim] = len / shards;
        first = shard * shape[shard_dim];
    }
    mag_error_t err;
    mag_status_t st = mag_empty(&err, out, ctx, src->dtype, rank, shape);
    if (st != MAG_STATUS_OK) return st;
    mag_tensor_t *dst = *out;
    const size_t es = mag_type_trait(src->dtype)->size;
    const int dev = ((mag_b200_device_t *)dst->storage->device->impl)->ordinal;
    char *d = (char *)dst->storage->base + dst->storage_offset * (int64_t)es;
    const char *s = (const char *)src->storage->base + src->storage_offset * (int64_t)es;
    int rc;
    if (shard_dim < 0) {
        rc = magb200_upload(dev, d, s, (size_t)src->numel * es);
    } else {
        const size_t width = (size_t)(shape[shard_dim] * inner) * es, pitch = (size_t)(len * inner) * es;
        rc = magb200_upload_2d(dev, d, width, s + (size_t)(first * inner) * es, pitch, width, (size_t)outer);
    }
    if (rc != MAGB200_OK) { mag_tensor_decref(dst); *out = NULL; }
    return mag_b200_map_status(rc, "tensor_to_device");
}

MAG_EXPORT mag_status_t mag_b200_host_alloc(void **out, size_t size_bytes) {
    return mag_b200_map_status(magb200_host_alloc_pinned(out, size_bytes), "page-locked host allocation");
}
MAG_EXPORT mag_status_t mag_b200_host_free(void *ptr) {
    return mag_b200_map_status(magb200_host_free_pinned(ptr), "page-locked host release");
}

MAG_EXPORT mag_status_t mag_b200_synchronize(mag_context_t *ctx) {
    if (!ctx || !ctx->active_device || ctx->active_device->id.type != MAG_BACKEND_TYPE_CUDA) return MAG_STATUS_ERR_INVALID_PARAM;
    return mag_b200_map_status(magb200_synchronize(((mag_b200_device_t *)ctx->active_device->impl)->ordinal), "synchronize");
}
