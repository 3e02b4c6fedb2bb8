// Min / Max of a tensor as the index of the extreme element: replaces CLReduce
// (src/main/java/neureka/backend/main/operations/linear/internal/opencl/CLReduce.java:34-147) with the semantics of the CPU
// implementation, CPUReduce (src/main/java/neureka/backend/main/operations/other/internal/CPUReduce.java:72-140): the result is
// ONE int, the flat index of the smallest / largest element, found with a strict comparison (`current < value` /
// `current > value`), so among equal extremes the lowest index wins. The operations Min / Max read the item at that index,
// and the index is what their backward pass needs.
//
// Two launches on the context's stream: every CTA scans a contiguous block of the flat index space (a thread walks its
// elements in rising order; lanes and warps are combined with "better value, or equal value and lower index"), writes
// its (value, index) pair to scratch, and one CTA combines the pairs. NaN: the reference's answer for data that
// contains NaNs depends on where its 64-element tiles start (a NaN that opens a tile survives it, any other NaN is
// skipped); here a NaN is never selected unless every element is NaN (then index 0).
#include "nk_internal.h"

namespace {

struct ArgView {
    int nd;
    int64_t n;
    int64_t base;
    int64_t div[NK_MAX_RANK], stride[NK_MAX_RANK];
    int dense;   // flat index == element offset - base
};

template <class T>
struct Best {
    T v;
    long long i;   // -1: nothing seen yet
};

template <class T, bool MAX>
__device__ __forceinline__ bool better(T cand, long long ci, T cur, long long ki) {
    if (ci < 0) return false;
    if (ki < 0) return true;
    if (cand != cand) return false;                 // NaN never wins
    if (cur != cur) return true;                    // ... and always loses
    if (MAX ? cand > cur : cand < cur) return true;
    return cand == cur && ci < ki;
}

template <class T, bool MAX>
__device__ __forceinline__ Best<T> cta_reduce(Best<T> b) {
    __shared__ T sv[8];
    __shared__ long long si[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const T ov = __shfl_down_sync(0xffffffffu, b.v, o);
        const long long oi = __shfl_down_sync(0xffffffffu, b.i, o);
        if (better<T, MAX>(ov, oi, b.v, b.i)) { b.v = ov; b.i = oi; }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) { sv[warp] = b.v; si[warp] = b.i; }
    __syncthreads();
    if (warp == 0) {
        b.v = lane < 8 ? sv[lane] : T(0);
        b.i = lane < 8 ? si[lane] : -1;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
            const T ov = __shfl_down_sync(0xffffffffu, b.v, o);
            const long long oi = __shfl_down_sync(0xffffffffu, b.i, o);
            if (better<T, MAX>(ov, oi, b.v, b.i)) { b.v = ov; b.i = oi; }
        }
    }
    return b;   // valid in thread 0
}

template <class T, bool MAX>
__global__ void __launch_bounds__(256) nk_arg_reduce_kernel(const T* __restrict__ src, ArgView a, T* __restrict__ pv, long long* __restrict__ pi) {
    const int64_t per = (a.n + gridDim.x - 1) / gridDim.x;
    const int64_t lo = int64_t(blockIdx.x) * per;
    const int64_t hi = lo + per < a.n ? lo + per : a.n;
    Best<T> b{T(0), -1};
    for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        int64_t off = a.base;
        if (a.dense) off += i;
        else {
            int64_t rem = i;
            for (int k = 0; k < a.nd; k++) { const int64_t idx = rem / a.div[k]; rem -= idx * a.div[k]; off += idx * a.stride[k]; }
        }
        const T v = src[off];
        if (better<T, MAX>(v, i, b.v, b.i)) { b.v = v; b.i = i; }
    }
    b = cta_reduce<T, MAX>(b);
    if (threadIdx.x == 0) { pv[blockIdx.x] = b.v; pi[blockIdx.x] = b.i; }
}

template <class T, bool MAX>
__global__ void __launch_bounds__(256) nk_arg_reduce_finish_kernel(const T* __restrict__ pv, const long long* __restrict__ pi, int parts, int32_t* __restrict__ out) {
    Best<T> b{T(0), -1};
    for (int p = threadIdx.x; p < parts; p += blockDim.x)
        if (better<T, MAX>(pv[p], pi[p], b.v, b.i)) { b.v = pv[p]; b.i = pi[p]; }
    b = cta_reduce<T, MAX>(b);
    if (threadIdx.x == 0) *out = b.i < 0 ? 0 : int32_t(b.i);   // all NaN (or nothing comparable): index 0
}

template <class T>
int launch(nk_ctx* ctx, bool want_max, const T* src, const ArgView& a, int32_t* out) {
    const int parts = nk_grid_for(ctx, a.n, 256 * 8, 4);
    void* scratch = nullptr;
    int st = nk_scratch(ctx, size_t(parts) * (sizeof(long long) + sizeof(T)) + 16, &scratch);
    if (st) return st;
    long long* pi = reinterpret_cast<long long*>(scratch);
    T* pv = reinterpret_cast<T*>(pi + parts);
    if (want_max) nk_arg_reduce_kernel<T, true><<<parts, 256, 0, ctx->stream>>>(src, a, pv, pi);
    else nk_arg_reduce_kernel<T, false><<<parts, 256, 0, ctx->stream>>>(src, a, pv, pi);
    if ((st = nk_after_launch(ctx, "nk_arg_reduce_kernel"))) return st;
    if (want_max) nk_arg_reduce_finish_kernel<T, true><<<1, 256, 0, ctx->stream>>>(pv, pi, parts, out);
    else nk_arg_reduce_finish_kernel<T, false><<<1, 256, 0, ctx->stream>>>(pv, pi, parts, out);
    return nk_after_launch(ctx, "nk_arg_reduce_finish_kernel");
}

}  // namespace

extern "C" int nk_arg_reduce(nk_ctx* ctx, int32_t want_max, int32_t dtype, int32_t rank, nk_buf* src, const int32_t* cfg, nk_buf* out_i32,
                             int64_t out_index) {
    NK_CHECK_CTX(ctx);
    if (dtype != NK_F32 && dtype != NK_F64) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_arg_reduce: dtype %d not supported (F32/F64 only)", dtype);
    NkView v;
    int st;
    if ((st = nk_view_parse(ctx, "nk_arg_reduce(src)", src, cfg, rank, dtype, &v))) return st;
    if (out_i32 == nullptr || out_i32->magic != 0x4e4b4246 || out_i32->dtype != NK_I32)
        return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_arg_reduce: the result buffer must hold I32 elements (the reference returns a Tensor<Integer>)");
    if (out_i32->device != ctx->device)
        return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_arg_reduce: result buffer lives on device %d, context on device %d", out_i32->device, ctx->device);
    if (out_index < 0 || out_index >= out_i32->n_elems) return nk_fail(ctx, NK_ERR_BOUNDS, "nk_arg_reduce: output index %lld outside the buffer", (long long)out_index);
    if (v.size >= (int64_t(1) << 31)) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_arg_reduce: the index of a tensor of 2^31 or more elements does not fit the I32 result");
    ArgView a;
    a.nd = rank;
    a.n = v.size;
    a.base = v.base;
    a.dense = v.dense_row_major && v.imap_row_major ? 1 : 0;
    for (int k = 0; k < rank; k++) { a.div[k] = v.imap[k]; a.stride[k] = v.estride[k]; }
    int32_t* out = static_cast<int32_t*>(out_i32->ptr) + out_index;
    if (dtype == NK_F32) return launch<float>(ctx, want_max != 0, static_cast<const float*>(src->ptr), a, out);
    return launch<double>(ctx, want_max != 0, static_cast<const double*>(src->ptr), a, out);
}
