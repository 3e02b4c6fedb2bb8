// nk_sum_static: the tile-wise sum of nk_sum with its intermediate levels kept in a fixed, library-owned device
// array instead of the context's grow-on-demand scratch block, so that the call itself never allocates.
//
// Who needs this: a host that has handed the whole of the GPU's memory to its own tensor pool at start-up (the
// JVM-side device does exactly that when it pre-reserves HBM for tensors) cannot let the library grow a hidden
// block behind its back -- the cudaMalloc inside nk_sum may fail there although the host's accounting says
// everything fits, and when it succeeds it synchronises the whole device in the middle of a backward pass.
// Such a caller passes its own input and output buffers as usual and uses this entry point for the reduction.
//
// The price is a hard size limit (NK_SUM_STATIC_SCRATCH_BYTES of partial sums, i.e. views of up to about
// 16.6 million F64 or 33.2 million F32 elements) and shared state: every call on a device uses the same array, which
// keeps whatever the previous call left in it. Nothing has to be cleared -- each level is written completely
// before the next level reads it -- but two calls that overlap on the GPU (different streams or contexts of the
// same device) race on the array; callers must order them.

#include <mutex>

#include "nk_internal.h"

// One instance per device that loads this library; it occupies NK_SUM_STATIC_SCRATCH_BYTES there until exit.
static __device__ __align__(256) unsigned char nk_sum_static_scratch[NK_SUM_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_addr[kMaxDevices] = {};   // device address of the array, per device ordinal

// In host code the array's name is only a handle for the runtime; the address a kernel can use has to be asked
// for, per device, with that device current.
int scratch_address(nk_ctx* ctx, void** out) {
    if (ctx->device < 0 || ctx->device >= kMaxDevices)
        return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_sum_static: device ordinal %d beyond the supported %d", ctx->device, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_addr[ctx->device] == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, nk_sum_static_scratch);   // NK_CHECK_CTX made ctx->device current
        if (e != cudaSuccess) return nk_cuda_fail(ctx, e, "cudaGetSymbolAddress(nk_sum_static_scratch)");
        if (p == nullptr) return nk_fail(ctx, NK_ERR_CUDA, "nk_sum_static: the runtime returned a null scratch address");
        g_scratch_addr[ctx->device] = p;
    }
    *out = g_scratch_addr[ctx->device];
    return NK_OK;
}

struct SumView {
    int nd;
    int64_t div[NK_MAX_RANK], stride[NK_MAX_RANK];
    int64_t base;
};

// Same tiling and the same order of additions as nk_sum: 128 consecutive elements per tile, added in index
// order by one lane after the warp staged them; levels shrink by 128 until one value is left.
template <class T>
__global__ void __launch_bounds__(128) nk_sum_static_tiles_kernel(const T* __restrict__ in, SumView v, bool through_view, int64_t n,
                                                                  T* __restrict__ out, int64_t n_tiles) {
    __shared__ T tile[4][128 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int64_t t = int64_t(blockIdx.x) * 4 + warp; t < n_tiles; t += int64_t(gridDim.x) * 4) {
        const int64_t off = t * 128;
        const int64_t lim = (off + 128 < n) ? 128 : (n - off);
        for (int k = lane; k < lim; k += 32) {
            int64_t i = off + k, src = i;
            if (through_view) {
                int64_t rem = i;
                src = v.base;
                for (int j = 0; j < v.nd; j++) { int64_t idx = rem / v.div[j]; rem -= idx * v.div[j]; src += idx * v.stride[j]; }
            }
            tile[warp][k] = in[src];
        }
        __syncwarp();
        if (lane == 0) {
            T value = 0;
            for (int k = 0; k < lim; k++) value += tile[warp][k];
            out[t] = value;
        }
        __syncwarp();
    }
}

template <class T>
int sum_static(nk_ctx* ctx, const T* in, const SumView& v, int64_t n, T* out_elem, void* scratch) {
    const int64_t n1 = (n + 127) / 128, n2 = (n1 + 127) / 128;
    T* bufA = reinterpret_cast<T*>(scratch);
    T* bufB = bufA + n1 + 1;
    (void)n2;
    const T* src = in;
    int64_t cur = n;
    bool through_view = true;
    T* dst = bufA;
    while (true) {
        const int64_t tiles = (cur + 127) / 128;
        T* target = (tiles == 1) ? out_elem : dst;
        const int64_t want = (tiles + 3) / 4, cap = int64_t(ctx->prop.multiProcessorCount) * 16;
        nk_sum_static_tiles_kernel<T><<<int(want < cap ? want : cap), 128, 0, ctx->stream>>>(src, v, through_view, cur, target, tiles);
        int st = nk_after_launch(ctx, "nk_sum_static_tiles_kernel");
        if (st) return st;
        if (tiles == 1) break;
        src = target;
        through_view = false;
        cur = tiles;
        dst = (dst == bufA) ? bufB : bufA;
    }
    return NK_OK;
}

}  // namespace

extern "C" int nk_sum_static(nk_ctx* ctx, int32_t dtype, int32_t rank, nk_buf* src, const int32_t* cfg, nk_buf* out, int64_t out_index) {
    NK_CHECK_CTX(ctx);
    if (dtype != NK_F32 && dtype != NK_F64) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_sum_static: dtype %d not supported (F32/F64 only)", dtype);
    NkView view;
    int st;
    if ((st = nk_view_parse(ctx, "nk_sum_static(src)", src, cfg, rank, dtype, &view))) return st;
    if (out == nullptr || out->magic != 0x4e4b4246 || out->dtype != dtype) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_sum_static: invalid output buffer");
    if (out->device != ctx->device)
        return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_sum_static: output buffer lives on device %d, context on device %d", out->device, ctx->device);
    if (out_index < 0 || out_index >= out->n_elems) return nk_fail(ctx, NK_ERR_BOUNDS, "nk_sum_static: output index %lld outside the buffer", (long long)out_index);
    const size_t es = nk_dtype_size(dtype);
    const int64_t n = view.size, n1 = (n + 127) / 128, n2 = (n1 + 127) / 128;
    const size_t need = size_t(n1 + n2 + 2) * es;
    if (need > size_t(NK_SUM_STATIC_SCRATCH_BYTES))
        return nk_fail(ctx, NK_ERR_UNSUPPORTED,
                       "nk_sum_static: a view of %lld elements needs %zu bytes of partial sums, the fixed scratch array holds %d "
                       "(limit: about %lld elements of this type); use nk_sum for larger views",
                       (long long)n, need, int(NK_SUM_STATIC_SCRATCH_BYTES), (long long)(int64_t(NK_SUM_STATIC_SCRATCH_BYTES / es) * 127));
    void* scratch = nullptr;
    if ((st = scratch_address(ctx, &scratch))) return st;
    SumView v;
    v.nd = rank;
    v.base = view.base;
    for (int k = 0; k < rank; k++) { v.div[k] = view.imap[k]; v.stride[k] = view.estride[k]; }
    if (dtype == NK_F32) return sum_static<float>(ctx, (const float*)src->ptr, v, n, (float*)out->ptr + out_index, scratch);
    return sum_static<double>(ctx, (const double*)src->ptr, v, n, (double*)out->ptr + out_index, scratch);
}
