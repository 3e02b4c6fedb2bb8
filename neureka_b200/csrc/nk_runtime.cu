// Context lifecycle, device memory, transfers, error reporting, view validation, timers and IPC.
// This is the part of the library that stands in for OpenCLDevice's memory handling
// (src/main/java/neureka/devices/opencl/OpenCLDevice.java:316-334, 355-405, 553-594, 616-632, 676-690).

#include "nk_internal.h"

#include <new>

static thread_local std::string g_thread_error;

size_t nk_dtype_size(int dtype) {
    switch (dtype) {
        case NK_F32: return 4;
        case NK_F64: return 8;
        case NK_I8: return 1;
        case NK_I16: return 2;
        case NK_I32: return 4;
        case NK_I64: return 8;
    }
    return 0;
}

int nk_fail(nk_ctx* ctx, int status, const char* fmt, ...) {
    char msg[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof(msg), fmt, ap);
    va_end(ap);
    g_thread_error = msg;
    if (ctx != nullptr && ctx->magic == 0x4e4b4358) {
        std::lock_guard<std::mutex> lock(ctx->mu);
        ctx->last_error = msg;
    }
    return status;
}

int nk_cuda_fail(nk_ctx* ctx, cudaError_t e, const char* what) {
    int status = (e == cudaErrorMemoryAllocation) ? NK_ERR_OOM : NK_ERR_CUDA;
    // cudaGetLastError clears a non-sticky error so that later calls on this thread start clean.
    cudaGetLastError();
    return nk_fail(ctx, status, "CUDA error %d (%s) in %s", int(e), cudaGetErrorString(e), what);
}

int nk_after_launch(nk_ctx* ctx, const char* kernel_name) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return nk_cuda_fail(ctx, e, kernel_name);
    ctx->launches++;
    ctx->last_kernel = kernel_name;
    return NK_OK;
}

// The context's scratch block grows on demand. Both the release of the old block and the new allocation are ordered on
// the context's stream (the device's memory pool), so work already queued keeps its block and nothing waits for the
// device: a backward pass that needs a larger block in its middle does not stall the other streams.
int nk_scratch(nk_ctx* ctx, size_t bytes, void** out) {
    if (bytes > ctx->scratch_bytes) {
        if (ctx->scratch) {
            NK_CUDA(ctx, cudaFreeAsync(ctx->scratch, ctx->stream));
            ctx->scratch = nullptr;
            ctx->scratch_bytes = 0;
        }
        size_t want = bytes < (size_t(1) << 20) ? (size_t(1) << 20) : bytes;
        NK_CUDA(ctx, cudaMallocAsync(&ctx->scratch, want, ctx->stream));
        ctx->scratch_bytes = want;
    }
    *out = ctx->scratch;
    return NK_OK;
}

int nk_check_device_status(nk_ctx* ctx) {
    if (ctx->tma_status_host && *ctx->tma_status_host != 0) {
        *ctx->tma_status_host = 0;
        return nk_fail(ctx, NK_ERR_TIMEOUT, "a kernel gave up waiting for a tensor copy (bounded mbarrier wait expired); its results are incomplete");
    }
    return NK_OK;
}

// ------------------------------------------------------------------------------------------------
// views
// ------------------------------------------------------------------------------------------------
int nk_view_parse(nk_ctx* ctx, const char* who, const nk_buf* buf, const int32_t* cfg, int rank, int dtype, NkView* v) {
    if (buf == nullptr || buf->magic != 0x4e4b4246) return nk_fail(ctx, NK_ERR_BAD_ARG, "%s: invalid buffer handle", who);
    if (cfg == nullptr) return nk_fail(ctx, NK_ERR_BAD_ARG, "%s: view descriptor is null", who);
    if (rank < 1) return nk_fail(ctx, NK_ERR_BAD_ARG, "%s: rank %d < 1", who, rank);
    if (rank > NK_MAX_RANK) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "%s: rank %d exceeds the supported maximum %d", who, rank, NK_MAX_RANK);
    if (buf->dtype != dtype)
        return nk_fail(ctx, NK_ERR_BAD_ARG, "%s: buffer dtype %d does not match the call's dtype %d", who, buf->dtype, dtype);
    if (buf->device != ctx->device)
        return nk_fail(ctx, NK_ERR_BAD_ARG, "%s: buffer lives on device %d, context on device %d", who, buf->device, ctx->device);
    const int32_t *shape = cfg, *strides = cfg + rank, *imap = cfg + 2 * rank, *offset = cfg + 3 * rank, *spread = cfg + 4 * rank;
    v->rank = rank;
    v->base = 0;
    v->size = 1;
    // A virtual tensor's configuration is all zeros except the shape (every index maps to element 0,
    // ndim/config/types/views/virtual/VirtualNDConfiguration.java:33-64): decode it row-major.
    bool virtual_cfg = true;
    for (int k = 0; k < rank; k++) virtual_cfg = virtual_cfg && imap[k] == 0 && strides[k] == 0;
    int64_t vmap[NK_MAX_RANK];
    {
        int64_t m = 1;
        for (int k = rank - 1; k >= 0; k--) { vmap[k] = m; m *= (shape[k] > 0 ? shape[k] : 1); }
    }
    int64_t lo = 0, hi = 0;  // extreme element offsets reachable relative to base
    for (int k = 0; k < rank; k++) {
        if (shape[k] < 1) return nk_fail(ctx, NK_ERR_BAD_ARG, "%s: shape[%d] = %d, must be > 0", who, k, shape[k]);
        if (!virtual_cfg && imap[k] < 1) return nk_fail(ctx, NK_ERR_BAD_ARG, "%s: indicesMap[%d] = %d, must be > 0", who, k, imap[k]);
        v->shape[k] = shape[k];
        v->imap[k] = virtual_cfg ? vmap[k] : imap[k];
        v->estride[k] = int64_t(spread[k]) * strides[k];
        v->base += int64_t(offset[k]) * strides[k];
        // checked before the multiplication: eight extents of 2^16 would wrap int64 to 0 and pass every later test
        if (v->size > (int64_t(1) << 40) / shape[k])
            return nk_fail(ctx, NK_ERR_UNSUPPORTED, "%s: view of more than 2^40 elements is too large", who);
        v->size *= shape[k];
        int64_t reach = v->estride[k] * (shape[k] - 1);   // |spread * strides| < 2^62, extent < 2^31: no wrap
        if (reach > 0) hi += reach; else lo += reach;
        if (hi > (int64_t(1) << 62) || lo < -(int64_t(1) << 62))
            return nk_fail(ctx, NK_ERR_BOUNDS, "%s: view reaches beyond any buffer", who);
    }
    if (v->base + lo < 0 || v->base + hi >= buf->n_elems)
        return nk_fail(ctx, NK_ERR_BOUNDS, "%s: view reaches elements [%lld, %lld] of a buffer holding %lld",
                       who, (long long)(v->base + lo), (long long)(v->base + hi), (long long)buf->n_elems);
    int64_t rm = 1;
    v->imap_row_major = true;
    v->dense_row_major = true;
    for (int k = rank - 1; k >= 0; k--) {
        if (v->imap[k] != rm) v->imap_row_major = false;
        if (v->estride[k] != rm && v->shape[k] != 1) v->dense_row_major = false;
        rm *= v->shape[k];
    }
    return NK_OK;
}

// ------------------------------------------------------------------------------------------------
// lifecycle
// ------------------------------------------------------------------------------------------------
extern "C" const char* nk_version(void) { return "neureka_cuda 0.1 (sm_100a)"; }

extern "C" const char* nk_last_error(nk_ctx* ctx) {
    static thread_local std::string copy;
    if (ctx != nullptr && ctx->magic == 0x4e4b4358) {
        std::lock_guard<std::mutex> lock(ctx->mu);
        copy = ctx->last_error;
    } else {
        copy = g_thread_error;
    }
    return copy.c_str();
}

extern "C" int nk_device_count(int32_t* out_count) {
    if (!out_count) return nk_fail(nullptr, NK_ERR_BAD_ARG, "nk_device_count: out pointer is null");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) { *out_count = 0; return nk_cuda_fail(nullptr, e, "cudaGetDeviceCount"); }
    *out_count = n;
    return NK_OK;
}

extern "C" int nk_device_open(int32_t ordinal, nk_ctx** out_ctx) {
    if (!out_ctx) return nk_fail(nullptr, NK_ERR_BAD_ARG, "nk_device_open: out pointer is null");
    *out_ctx = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) return nk_cuda_fail(nullptr, e, "cudaGetDeviceCount (is a CUDA device present?)");
    if (ordinal < 0 || ordinal >= n) return nk_fail(nullptr, NK_ERR_BAD_ARG, "nk_device_open: ordinal %d outside [0, %d)", ordinal, n);
    nk_ctx* ctx = new (std::nothrow) nk_ctx();
    if (!ctx) return nk_fail(nullptr, NK_ERR_OOM, "nk_device_open: host allocation failed");
    ctx->device = ordinal;
    e = cudaSetDevice(ordinal);
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&ctx->prop, ordinal);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev0);
    if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev1);
    if (e == cudaSuccess) {
        // nk_alloc / nk_free go through the device's stream-ordered memory pool: freed blocks stay in the pool (no
        // release back to the driver at synchronisation points) and are handed out again without a device-wide wait
        cudaMemPool_t pool = nullptr;
        e = cudaDeviceGetDefaultMemPool(&pool, ordinal);
        uint64_t keep = UINT64_MAX;
        if (e == cudaSuccess) e = cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
    }
    if (e == cudaSuccess) e = cudaHostAlloc((void**)&ctx->tma_status_host, sizeof(int), cudaHostAllocMapped);
    if (e == cudaSuccess) { *ctx->tma_status_host = 0; e = cudaHostGetDevicePointer((void**)&ctx->tma_status_dev, ctx->tma_status_host, 0); }
    if (e != cudaSuccess) {
        int st = nk_cuda_fail(nullptr, e, "nk_device_open");
        delete ctx;
        return st;
    }
    if (ctx->prop.major < 10) {
        int st = nk_fail(nullptr, NK_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only",
                         ordinal, ctx->prop.major, ctx->prop.minor);
        cudaStreamDestroy(ctx->stream);
        cudaEventDestroy(ctx->ev0);
        cudaEventDestroy(ctx->ev1);
        delete ctx;
        return st;
    }
    *out_ctx = ctx;
    return NK_OK;
}

extern "C" int nk_device_close(nk_ctx* ctx) {
    if (ctx == nullptr) return NK_OK;
    NK_CHECK_CTX(ctx);
    if (ctx->scratch) cudaFreeAsync(ctx->scratch, ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->tma_status_host) cudaFreeHost(ctx->tma_status_host);
    cudaEventDestroy(ctx->ev0);
    cudaEventDestroy(ctx->ev1);
    cudaStreamDestroy(ctx->stream);
    ctx->magic = 0;
    delete ctx;
    return NK_OK;
}

extern "C" int nk_device_props(nk_ctx* ctx, nk_props* out) {
    NK_CHECK_CTX(ctx);
    if (!out) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_device_props: out pointer is null");
    memset(out, 0, sizeof(*out));
    strncpy(out->name, ctx->prop.name, sizeof(out->name) - 1);
    out->total_mem_bytes = ctx->prop.totalGlobalMem;
    out->sm_count = ctx->prop.multiProcessorCount;
    out->cc_major = ctx->prop.major;
    out->cc_minor = ctx->prop.minor;
    out->l2_bytes = ctx->prop.l2CacheSize;
    out->max_smem_per_block = int32_t(ctx->prop.sharedMemPerBlockOptin);
    int khz = 0;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, ctx->device);
    out->clock_khz = khz;
    return NK_OK;
}

extern "C" int nk_sync(nk_ctx* ctx) {
    NK_CHECK_CTX(ctx);
    NK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return nk_check_device_status(ctx);
}

extern "C" void* nk_stream(nk_ctx* ctx) {
    if (ctx == nullptr || ctx->magic != 0x4e4b4358) return nullptr;
    return (void*)ctx->stream;
}

// ------------------------------------------------------------------------------------------------
// memory
// ------------------------------------------------------------------------------------------------
// Largest element count a handle may claim: keeps n_elems * sizeof(element) far from wrapping size_t.
static const int64_t NK_MAX_ELEMS = int64_t(1) << 44;

static int nk_alloc_impl(nk_ctx* ctx, int32_t dtype, int64_t n_elems, bool pooled, nk_buf** out, const char* who) {
    NK_CHECK_CTX(ctx);
    if (!out) return nk_fail(ctx, NK_ERR_BAD_ARG, "%s: out pointer is null", who);
    *out = nullptr;
    size_t es = nk_dtype_size(dtype);
    if (es == 0) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "%s: unknown dtype %d", who, dtype);
    if (n_elems < 1) return nk_fail(ctx, NK_ERR_BAD_ARG, "%s: n_elems = %lld, must be > 0", who, (long long)n_elems);
    if (n_elems > NK_MAX_ELEMS) return nk_fail(ctx, NK_ERR_OOM, "%s: %lld elements exceed the supported maximum of 2^44 (more memory than any device holds)", who, (long long)n_elems);
    nk_buf* b = new (std::nothrow) nk_buf();
    if (!b) return nk_fail(ctx, NK_ERR_OOM, "%s: host allocation failed", who);
    cudaError_t e = pooled ? cudaMallocAsync(&b->ptr, size_t(n_elems) * es, ctx->stream) : cudaMalloc(&b->ptr, size_t(n_elems) * es);
    if (e != cudaSuccess) { delete b; return nk_cuda_fail(ctx, e, pooled ? "cudaMallocAsync" : "cudaMalloc"); }
    b->n_elems = n_elems;
    b->dtype = dtype;
    b->device = ctx->device;
    b->owned = true;
    b->pooled = pooled;
    *out = b;
    return NK_OK;
}

extern "C" int nk_alloc(nk_ctx* ctx, int32_t dtype, int64_t n_elems, nk_buf** out) {
    return nk_alloc_impl(ctx, dtype, n_elems, true, out, "nk_alloc");
}

extern "C" int nk_alloc_shared(nk_ctx* ctx, int32_t dtype, int64_t n_elems, nk_buf** out) {
    return nk_alloc_impl(ctx, dtype, n_elems, false, out, "nk_alloc_shared");
}

extern "C" int nk_wrap(nk_ctx* ctx, int32_t dtype, void* device_ptr, int64_t n_elems, nk_buf** out) {
    NK_CHECK_CTX(ctx);
    if (!out) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_wrap: out pointer is null");
    *out = nullptr;
    if (nk_dtype_size(dtype) == 0) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_wrap: unknown dtype %d", dtype);
    if (device_ptr == nullptr || n_elems < 1) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_wrap: null pointer or empty range");
    if (n_elems > NK_MAX_ELEMS) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_wrap: %lld elements exceed the supported maximum of 2^44", (long long)n_elems);
    nk_buf* b = new (std::nothrow) nk_buf();
    if (!b) return nk_fail(ctx, NK_ERR_OOM, "nk_wrap: host allocation failed");
    b->ptr = device_ptr;
    b->n_elems = n_elems;
    b->dtype = dtype;
    b->device = ctx->device;
    b->owned = false;
    *out = b;
    return NK_OK;
}

extern "C" int nk_free(nk_ctx* ctx, nk_buf* buf) {
    if (buf == nullptr) return NK_OK;
    NK_CHECK_CTX(ctx);
    if (buf->magic != 0x4e4b4246) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_free: invalid (or already freed) buffer handle");
    // Kernels already queued may still touch the allocation. A pooled block goes back to the pool in stream order
    // (after everything this context queued so far; nothing waits); cudaFree synchronises the device; an IPC close
    // does not, so wait for the stream first.
    cudaError_t e = cudaSuccess;
    if (buf->ipc) {
        cudaStreamSynchronize(ctx->stream);
        e = cudaIpcCloseMemHandle(buf->ptr);
    } else if (buf->owned) {
        e = buf->pooled ? cudaFreeAsync(buf->ptr, ctx->stream) : cudaFree(buf->ptr);
    }
    buf->magic = 0;
    delete buf;
    if (e != cudaSuccess) return nk_cuda_fail(ctx, e, "nk_free");
    return NK_OK;
}

extern "C" int nk_buf_info(nk_buf* buf, void** device_ptr, int64_t* n_elems, int32_t* dtype) {
    if (buf == nullptr || buf->magic != 0x4e4b4246) return nk_fail(nullptr, NK_ERR_BAD_ARG, "nk_buf_info: invalid buffer handle");
    if (device_ptr) *device_ptr = buf->ptr;
    if (n_elems) *n_elems = buf->n_elems;
    if (dtype) *dtype = buf->dtype;
    return NK_OK;
}

static int check_range(nk_ctx* ctx, const char* who, const nk_buf* buf, int64_t start, int64_t n) {
    if (buf == nullptr || buf->magic != 0x4e4b4246) return nk_fail(ctx, NK_ERR_BAD_ARG, "%s: invalid buffer handle", who);
    if (n < 0 || start < 0 || start + n > buf->n_elems)
        return nk_fail(ctx, NK_ERR_BOUNDS, "%s: range [%lld, %lld) outside a buffer of %lld elements", who,
                       (long long)start, (long long)(start + n), (long long)buf->n_elems);
    return NK_OK;
}

template <class T>
__global__ void nk_fill_kernel(T* __restrict__ p, T value, int64_t n) {
    int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = value;
}

extern "C" int nk_fill(nk_ctx* ctx, nk_buf* buf, double value, int64_t start, int64_t n) {
    NK_CHECK_CTX(ctx);
    int st = check_range(ctx, "nk_fill", buf, start, n);
    if (st) return st;
    if (n == 0) return NK_OK;
    int block = 256, grid = nk_grid_for(ctx, (n + 3) / 4, block, 8);
    switch (buf->dtype) {
        case NK_F32: nk_fill_kernel<float><<<grid, block, 0, ctx->stream>>>((float*)buf->ptr + start, float(value), n); break;
        case NK_F64: nk_fill_kernel<double><<<grid, block, 0, ctx->stream>>>((double*)buf->ptr + start, value, n); break;
        case NK_I8: nk_fill_kernel<int8_t><<<grid, block, 0, ctx->stream>>>((int8_t*)buf->ptr + start, int8_t(value), n); break;
        case NK_I16: nk_fill_kernel<int16_t><<<grid, block, 0, ctx->stream>>>((int16_t*)buf->ptr + start, int16_t(value), n); break;
        case NK_I32: nk_fill_kernel<int32_t><<<grid, block, 0, ctx->stream>>>((int32_t*)buf->ptr + start, int32_t(value), n); break;
        case NK_I64: nk_fill_kernel<int64_t><<<grid, block, 0, ctx->stream>>>((int64_t*)buf->ptr + start, int64_t(value), n); break;
        default: return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_fill: unknown dtype %d", buf->dtype);
    }
    return nk_after_launch(ctx, "nk_fill_kernel");
}

extern "C" int nk_write(nk_ctx* ctx, nk_buf* buf, const void* host, int64_t host_off, int64_t dev_start, int64_t n) {
    NK_CHECK_CTX(ctx);
    int st = check_range(ctx, "nk_write", buf, dev_start, n);
    if (st) return st;
    if (host == nullptr || host_off < 0) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_write: null host pointer or negative offset");
    if (n == 0) return NK_OK;
    size_t es = nk_dtype_size(buf->dtype);
    NK_CUDA(ctx, cudaMemcpyAsync((char*)buf->ptr + dev_start * es, (const char*)host + host_off * es, size_t(n) * es,
                                 cudaMemcpyHostToDevice, ctx->stream));
    NK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));  // the host array may be released right after the call
    return NK_OK;
}

extern "C" int nk_read(nk_ctx* ctx, nk_buf* buf, void* host, int64_t dev_start, int64_t n) {
    NK_CHECK_CTX(ctx);
    int st = check_range(ctx, "nk_read", buf, dev_start, n);
    if (st) return st;
    if (host == nullptr) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_read: null host pointer");
    if (n == 0) return NK_OK;
    size_t es = nk_dtype_size(buf->dtype);
    NK_CUDA(ctx, cudaMemcpyAsync(host, (const char*)buf->ptr + dev_start * es, size_t(n) * es, cudaMemcpyDeviceToHost, ctx->stream));
    NK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return nk_check_device_status(ctx);
}

extern "C" int nk_write_async(nk_ctx* ctx, nk_buf* buf, const void* host, int64_t host_off, int64_t dev_start, int64_t n) {
    NK_CHECK_CTX(ctx);
    int st = check_range(ctx, "nk_write_async", buf, dev_start, n);
    if (st) return st;
    if (host == nullptr || host_off < 0) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_write_async: null host pointer or negative offset");
    if (n == 0) return NK_OK;
    size_t es = nk_dtype_size(buf->dtype);
    NK_CUDA(ctx, cudaMemcpyAsync((char*)buf->ptr + dev_start * es, (const char*)host + host_off * es, size_t(n) * es,
                                 cudaMemcpyHostToDevice, ctx->stream));
    return NK_OK;
}

extern "C" int nk_read_async(nk_ctx* ctx, nk_buf* buf, void* host, int64_t dev_start, int64_t n) {
    NK_CHECK_CTX(ctx);
    int st = check_range(ctx, "nk_read_async", buf, dev_start, n);
    if (st) return st;
    if (host == nullptr) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_read_async: null host pointer");
    if (n == 0) return NK_OK;
    size_t es = nk_dtype_size(buf->dtype);
    NK_CUDA(ctx, cudaMemcpyAsync(host, (const char*)buf->ptr + dev_start * es, size_t(n) * es, cudaMemcpyDeviceToHost, ctx->stream));
    return NK_OK;
}

extern "C" int nk_copy(nk_ctx* ctx, nk_buf* dst, int64_t dst_start, nk_buf* src, int64_t src_start, int64_t n) {
    NK_CHECK_CTX(ctx);
    int st = check_range(ctx, "nk_copy(dst)", dst, dst_start, n);
    if (st) return st;
    st = check_range(ctx, "nk_copy(src)", src, src_start, n);
    if (st) return st;
    if (dst->dtype != src->dtype) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_copy: dtype mismatch (%d vs %d)", dst->dtype, src->dtype);
    if (n == 0) return NK_OK;
    size_t es = nk_dtype_size(dst->dtype);
    NK_CUDA(ctx, cudaMemcpyAsync((char*)dst->ptr + dst_start * es, (const char*)src->ptr + src_start * es, size_t(n) * es,
                                 cudaMemcpyDeviceToDevice, ctx->stream));
    return NK_OK;
}

extern "C" int nk_host_alloc(size_t bytes, void** out_host) {
    if (!out_host || bytes == 0) return nk_fail(nullptr, NK_ERR_BAD_ARG, "nk_host_alloc: null out pointer or zero size");
    cudaError_t e = cudaHostAlloc(out_host, bytes, cudaHostAllocPortable);
    if (e != cudaSuccess) { *out_host = nullptr; return nk_cuda_fail(nullptr, e, "cudaHostAlloc"); }
    return NK_OK;
}

extern "C" int nk_host_free(void* host) {
    if (!host) return NK_OK;
    cudaError_t e = cudaFreeHost(host);
    if (e != cudaSuccess) return nk_cuda_fail(nullptr, e, "cudaFreeHost");
    return NK_OK;
}

// ------------------------------------------------------------------------------------------------
// knobs, counters, timers
// ------------------------------------------------------------------------------------------------
extern "C" int nk_set_conv_path(nk_ctx* ctx, int32_t path) {
    NK_CHECK_CTX(ctx);
    if (path < NK_CONV_AUTO || path > NK_CONV_TC) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_set_conv_path: unknown path %d", path);
    ctx->conv_path = path;
    return NK_OK;
}

extern "C" int nk_last_conv_path(nk_ctx* ctx, int32_t* out_path) {
    NK_CHECK_CTX(ctx);
    if (!out_path) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_last_conv_path: out pointer is null");
    *out_path = ctx->last_conv_path;
    return NK_OK;
}

extern "C" const char* nk_last_kernel(nk_ctx* ctx) {
    if (ctx == nullptr || ctx->magic != 0x4e4b4358) return "";
    return ctx->last_kernel;
}

extern "C" int nk_launch_count(nk_ctx* ctx, uint64_t* out) {
    NK_CHECK_CTX(ctx);
    if (!out) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_launch_count: out pointer is null");
    *out = ctx->launches;
    return NK_OK;
}

extern "C" int nk_timer_begin(nk_ctx* ctx) {
    NK_CHECK_CTX(ctx);
    NK_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
    return NK_OK;
}

extern "C" int nk_timer_end(nk_ctx* ctx, float* out_ms) {
    NK_CHECK_CTX(ctx);
    if (!out_ms) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_timer_end: out pointer is null");
    NK_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
    NK_CUDA(ctx, cudaEventSynchronize(ctx->ev1));
    NK_CUDA(ctx, cudaEventElapsedTime(out_ms, ctx->ev0, ctx->ev1));
    return nk_check_device_status(ctx);
}

// ------------------------------------------------------------------------------------------------
// events: ordering between the streams of two contexts on one device
// ------------------------------------------------------------------------------------------------
struct nk_event {
    cudaEvent_t ev = nullptr;
    int device = 0;
    uint32_t magic = 0x4e4b4556;  // 'NKEV'
};

extern "C" int nk_event_create(nk_ctx* ctx, nk_event** out) {
    NK_CHECK_CTX(ctx);
    if (!out) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_event_create: out pointer is null");
    *out = nullptr;
    nk_event* e = new (std::nothrow) nk_event();
    if (!e) return nk_fail(ctx, NK_ERR_OOM, "nk_event_create: out of host memory");
    cudaError_t err = cudaEventCreateWithFlags(&e->ev, cudaEventDisableTiming);
    if (err != cudaSuccess) { delete e; return nk_cuda_fail(ctx, err, "cudaEventCreateWithFlags"); }
    e->device = ctx->device;
    *out = e;
    return NK_OK;
}

extern "C" int nk_event_record(nk_ctx* ctx, nk_event* ev) {
    NK_CHECK_CTX(ctx);
    if (!ev || ev->magic != 0x4e4b4556) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_event_record: not an event");
    if (ev->device != ctx->device) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_event_record: event of device %d on a context of device %d", ev->device, ctx->device);
    NK_CUDA(ctx, cudaEventRecord(ev->ev, ctx->stream));
    return NK_OK;
}

extern "C" int nk_stream_wait_event(nk_ctx* ctx, nk_event* ev) {
    NK_CHECK_CTX(ctx);
    if (!ev || ev->magic != 0x4e4b4556) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_stream_wait_event: not an event");
    NK_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ev->ev, 0));
    return NK_OK;
}

extern "C" int nk_event_free(nk_event* ev) {
    if (!ev || ev->magic != 0x4e4b4556) return NK_ERR_BAD_ARG;
    cudaSetDevice(ev->device);
    cudaEventDestroy(ev->ev);
    ev->magic = 0;
    delete ev;
    return NK_OK;
}

// ------------------------------------------------------------------------------------------------
// IPC: share one rank's buffer with the other single-GPU processes of the box
// ------------------------------------------------------------------------------------------------
static_assert(sizeof(cudaIpcMemHandle_t) <= NK_IPC_HANDLE_BYTES, "IPC handle does not fit");

extern "C" int nk_ipc_export(nk_ctx* ctx, nk_buf* buf, uint8_t handle[NK_IPC_HANDLE_BYTES]) {
    NK_CHECK_CTX(ctx);
    if (buf == nullptr || buf->magic != 0x4e4b4246 || handle == nullptr) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_ipc_export: invalid argument");
    if (!buf->owned || buf->pooled)
        return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_ipc_export: only buffers allocated by nk_alloc_shared can be exported (pooled memory has no IPC handle)");
    cudaIpcMemHandle_t h;
    NK_CUDA(ctx, cudaIpcGetMemHandle(&h, buf->ptr));
    memset(handle, 0, NK_IPC_HANDLE_BYTES);
    memcpy(handle, &h, sizeof(h));
    return NK_OK;
}

extern "C" int nk_ipc_open(nk_ctx* ctx, const uint8_t handle[NK_IPC_HANDLE_BYTES], int32_t dtype, int64_t n_elems, nk_buf** out) {
    NK_CHECK_CTX(ctx);
    if (!out || !handle) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_ipc_open: null argument");
    *out = nullptr;
    if (nk_dtype_size(dtype) == 0 || n_elems < 1 || n_elems > NK_MAX_ELEMS) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_ipc_open: bad dtype or size");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    NK_CUDA(ctx, cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    nk_buf* b = new (std::nothrow) nk_buf();
    if (!b) { cudaIpcCloseMemHandle(p); return nk_fail(ctx, NK_ERR_OOM, "nk_ipc_open: host allocation failed"); }
    b->ptr = p;
    b->n_elems = n_elems;
    b->dtype = dtype;
    b->device = ctx->device;  // addressable from this context's device
    b->owned = false;
    b->ipc = true;
    *out = b;
    return NK_OK;
}
