// Internal declarations shared by the translation units of libneureka_cuda.
#pragma once

#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "../../include/neureka_cuda.h"

#define NK_MAX_RANK 8

struct nk_buf {
    void* ptr = nullptr;
    int64_t n_elems = 0;
    int32_t dtype = NK_F32;
    int32_t device = 0;
    bool owned = true;    // released on nk_free
    bool pooled = false;  // from the device's stream-ordered pool (cudaFreeAsync), else cudaFree
    bool ipc = false;     // cudaIpcCloseMemHandle on nk_free
    uint32_t magic = 0x4e4b4246;  // 'NKBF'
};

struct nk_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    cudaDeviceProp prop{};
    std::mutex mu;
    std::string last_error;
    uint64_t launches = 0;
    const char* last_kernel = "";
    int conv_path = NK_CONV_AUTO;
    int last_conv_path = NK_CONV_AUTO;
    // scratch for two-pass (split) reductions; grows on demand, owned by the ctx
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    // one host-mapped word kernels set when a bounded device-side wait runs out (read after a synchronise)
    int* tma_status_host = nullptr;
    int* tma_status_dev = nullptr;
    uint32_t magic = 0x4e4b4358;  // 'NKCX'
};

size_t nk_dtype_size(int dtype);
int nk_fail(nk_ctx* ctx, int status, const char* fmt, ...);
int nk_cuda_fail(nk_ctx* ctx, cudaError_t e, const char* what);
int nk_scratch(nk_ctx* ctx, size_t bytes, void** out);
int nk_check_device_status(nk_ctx* ctx);   // NK_ERR_TIMEOUT if a kernel reported an expired wait since the last check

#define NK_CUDA(ctx, call)                                                     \
    do {                                                                       \
        cudaError_t _e = (call);                                               \
        if (_e != cudaSuccess) return nk_cuda_fail((ctx), _e, #call);          \
    } while (0)

#define NK_CHECK_CTX(ctx)                                                      \
    do {                                                                       \
        if ((ctx) == nullptr || (ctx)->magic != 0x4e4b4358)                    \
            return nk_fail(nullptr, NK_ERR_BAD_ARG, "invalid context handle"); \
        cudaError_t _e = cudaSetDevice((ctx)->device);                         \
        if (_e != cudaSuccess) return nk_cuda_fail((ctx), _e, "cudaSetDevice");\
    } while (0)

// Records the launch (name + counter) and converts a launch error into a status.
int nk_after_launch(nk_ctx* ctx, const char* kernel_name);

// ------------------------------------------------------------------------------------------------
// Views: an NDConfiguration inline array resolved against a buffer.
//   element(idx) = base + sum_k idx_k * estride_k        (estride = spread*strides, base = sum offset*strides)
//   flat i -> idx: idx_k = i / imap_k ; i %= imap_k       (NDConfiguration.indicesOfIndex)
// ------------------------------------------------------------------------------------------------
struct NkView {
    int rank = 0;
    int64_t shape[NK_MAX_RANK];
    int64_t estride[NK_MAX_RANK];
    int64_t imap[NK_MAX_RANK];
    int64_t base = 0;
    int64_t size = 1;
    bool imap_row_major = true;  // indicesMap equals the row-major strides of shape
    bool dense_row_major = true; // estride equals row-major strides of shape (base may be non-zero)
};

// Parses + validates cfg against buf. Returns a status; on error the message is stored in ctx.
int nk_view_parse(nk_ctx* ctx, const char* who, const nk_buf* buf, const int32_t* cfg, int rank, int dtype, NkView* out);

inline int nk_grid_for(const nk_ctx* ctx, int64_t work_items, int block, int ctas_per_sm) {
    int64_t need = (work_items + block - 1) / block;
    int64_t cap = int64_t(ctx->prop.multiProcessorCount) * ctas_per_sm;
    if (need < 1) need = 1;
    return int(need < cap ? need : cap);
}
