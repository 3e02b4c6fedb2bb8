// nk_conv: entry point and the generic gather kernels (any rank <= 8, any view, F32/F64, forward and
// deconvolution). The generic family is the correctness anchor and the route for odd views; dense
// stencil-shaped calls are routed to the tiled family in nk_conv_tiled.cu.

#include "nk_conv_plan.h"

int nk_conv_gemm_try(nk_ctx* ctx, int dtype, nk_buf* drn, const NkView& v0, nk_buf* s1, const NkView& v1, nk_buf* s2, const NkView& v2,
                     int d, bool* handled);
int nk_conv_tiled_try(nk_ctx* ctx, int dtype, nk_buf* drn, const NkView& v0, nk_buf* s1, const NkView& v1,
                      nk_buf* s2, const NkView& v2, int d, bool force, bool* handled);

namespace {

// ---- generic A: one thread per drain element ---------------------------------------------------------
template <class T>
__global__ void __launch_bounds__(256) nk_conv_gather_kernel(T* __restrict__ out, const T* __restrict__ A, const T* __restrict__ B, ConvPlan c) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < c.total; i += stride) {
        int64_t rem = i, o0 = c.b0, oa = c.bA, ob = c.bB;
        int64_t lo[NK_MAX_RANK], cnt[NK_MAX_RANK], qa[NK_MAX_RANK], qb[NK_MAX_RANK];
        int nact = 0;
        bool empty = false;
        for (int k = 0; k < c.rank; k++) {
            int64_t p = rem / c.odiv[k];
            rem -= p * c.odiv[k];
            o0 += p * c.s0[k]; oa += p * c.pa[k]; ob += p * c.pb[k];
            int64_t l, h;
            nk_box_range(c, k, p, &l, &h);
            if (h < l) empty = true;
            oa += l * c.qa[k]; ob += l * c.qb[k];
            if (h > l) { lo[nact] = l; cnt[nact] = h - l + 1; qa[nact] = c.qa[k]; qb[nact] = c.qb[k]; nact++; }
        }
        T value = 0;
        if (!empty) {
            if (nact == 0) {
                value = A[oa] * B[ob];
            } else {
                // innermost active dim as a plain loop, the others as an odometer (last dim fastest)
                const int in = nact - 1;
                const int64_t n_in = cnt[in], sa = qa[in], sb = qb[in];
                int64_t q[NK_MAX_RANK];
                for (int k = 0; k < in; k++) q[k] = 0;
                while (true) {
                    for (int64_t j = 0; j < n_in; j++) value += A[oa + j * sa] * B[ob + j * sb];
                    int k = in - 1;
                    for (; k >= 0; k--) {
                        q[k]++; oa += qa[k]; ob += qb[k];
                        if (q[k] < cnt[k]) break;
                        oa -= q[k] * qa[k]; ob -= q[k] * qb[k]; q[k] = 0;
                    }
                    if (k < 0) break;
                }
            }
        }
        out[o0] = value;
    }
}

// ---- generic B: few drain elements, long reductions -> a group of CTAs per drain element --------------
// blockIdx.x = drain element, blockIdx.y = split. Partial sums go to scratch[element*splits + split]
// (or straight to the drain when splits == 1); nk_conv_finish_kernel adds them in split order, so the
// result does not depend on scheduling.
template <class T>
__global__ void __launch_bounds__(256) nk_conv_reduce_kernel(T* __restrict__ out, T* __restrict__ partial, const T* __restrict__ A,
                                                             const T* __restrict__ B, ConvPlan c, int splits) {
    __shared__ T warp_sums[8];
    const int64_t i = blockIdx.x;
    const int split = blockIdx.y;
    int64_t rem = i, o0 = c.b0, oa = c.bA, ob = c.bB;
    uint32_t cnt[NK_MAX_RANK];
    int64_t qa[NK_MAX_RANK], qb[NK_MAX_RANK];
    int nact = 0;
    uint64_t terms = 1;
    for (int k = 0; k < c.rank; k++) {
        int64_t p = rem / c.odiv[k];
        rem -= p * c.odiv[k];
        o0 += p * c.s0[k]; oa += p * c.pa[k]; ob += p * c.pb[k];
        int64_t l, h;
        nk_box_range(c, k, p, &l, &h);
        if (h < l) { terms = 0; h = l; }
        oa += l * c.qa[k]; ob += l * c.qb[k];
        if (h > l) { cnt[nact] = uint32_t(h - l + 1); qa[nact] = c.qa[k]; qb[nact] = c.qb[k]; terms *= cnt[nact]; nact++; }
    }
    const uint64_t chunk = (terms + splits - 1) / splits;
    const uint64_t t0 = chunk * split;
    uint64_t t1 = t0 + chunk;
    if (t1 > terms) t1 = terms;
    T value = 0;
    for (uint64_t t = t0 + threadIdx.x; t < t1; t += blockDim.x) {
        uint64_t r = t;
        int64_t a = oa, b = ob;
        for (int k = nact - 1; k >= 0; k--) {
            uint64_t qk = r % cnt[k];
            r /= cnt[k];
            a += int64_t(qk) * qa[k]; b += int64_t(qk) * qb[k];
        }
        value += A[a] * B[b];
    }
    // fixed-shape tree: shuffle inside the warp, then warp 0 adds the warp sums in order
    for (int off = 16; off > 0; off >>= 1) value += __shfl_down_sync(0xffffffffu, value, off);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = value;
    __syncthreads();
    if (threadIdx.x == 0) {
        T total = 0;
        for (int w = 0; w < int(blockDim.x >> 5); w++) total += warp_sums[w];
        if (splits == 1) out[o0] = total;
        else partial[i * splits + split] = total;
    }
}

template <class T>
__global__ void nk_conv_finish_kernel(T* __restrict__ out, const T* __restrict__ partial, ConvPlan c, int splits) {
    const int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= c.total) return;
    int64_t rem = i, o0 = c.b0;
    for (int k = 0; k < c.rank; k++) {
        int64_t p = rem / c.odiv[k];
        rem -= p * c.odiv[k];
        o0 += p * c.s0[k];
    }
    T total = 0;
    for (int s = 0; s < splits; s++) total += partial[i * splits + s];
    out[o0] = total;
}

template <class T>
int run_generic(nk_ctx* ctx, T* out, const T* A, const T* B, const ConvPlan& c) {
    const int sms = ctx->prop.multiProcessorCount;
    const bool few_outputs = c.total < int64_t(sms) * 64 && c.max_terms >= 1024;
    if (!few_outputs) {
        int block = 256, grid = nk_grid_for(ctx, c.total, block, 8);
        nk_conv_gather_kernel<T><<<grid, block, 0, ctx->stream>>>(out, A, B, c);
        return nk_after_launch(ctx, "nk_conv_gather_kernel");
    }
    if (c.total > 65535 * int64_t(1024)) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_conv: reduction grid too large");
    int64_t want = (int64_t(sms) * 8 + c.total - 1) / c.total;
    int64_t by_len = (c.max_terms + 8191) / 8192;
    int64_t splits = want < by_len ? want : by_len;
    if (splits < 1) splits = 1;
    if (splits > 1024) splits = 1024;
    T* partial = nullptr;
    if (splits > 1) {
        void* scratch = nullptr;
        int st = nk_scratch(ctx, size_t(c.total) * size_t(splits) * sizeof(T), &scratch);
        if (st) return st;
        partial = reinterpret_cast<T*>(scratch);
    }
    dim3 grid((unsigned)c.total, (unsigned)splits);
    nk_conv_reduce_kernel<T><<<grid, 256, 0, ctx->stream>>>(out, partial, A, B, c, int(splits));
    int st = nk_after_launch(ctx, "nk_conv_reduce_kernel");
    if (st || splits == 1) return st;
    nk_conv_finish_kernel<T><<<unsigned((c.total + 127) / 128), 128, 0, ctx->stream>>>(out, partial, c, int(splits));
    return nk_after_launch(ctx, "nk_conv_finish_kernel");
}

}  // namespace

extern "C" int nk_conv(nk_ctx* ctx, int32_t dtype, int32_t rank,
                       nk_buf* drn, const int32_t* cfg0, nk_buf* src1, const int32_t* cfg1, nk_buf* src2, const int32_t* cfg2,
                       int32_t d) {
    NK_CHECK_CTX(ctx);
    // AbstractCPUConvolution.java:49-65: Float and Double only, anything else is an IllegalArgumentException
    if (dtype != NK_F32 && dtype != NK_F64) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_conv: dtype %d not supported (F32/F64 only)", dtype);
    NkView v0, v1, v2;
    int st;
    if ((st = nk_view_parse(ctx, "nk_conv(drain)", drn, cfg0, rank, dtype, &v0))) return st;
    if ((st = nk_view_parse(ctx, "nk_conv(src1)", src1, cfg1, rank, dtype, &v1))) return st;
    if ((st = nk_view_parse(ctx, "nk_conv(src2)", src2, cfg2, rank, dtype, &v2))) return st;

    const int path = ctx->conv_path;
    if (path == NK_CONV_AUTO || path == NK_CONV_GEMM || path == NK_CONV_TC) {
        bool handled = false;
        st = nk_conv_gemm_try(ctx, dtype, drn, v0, src1, v1, src2, v2, d, &handled);   // sets last_conv_path (GEMM or TC)
        if (st) return st;
        if (handled) return NK_OK;
        if (path != NK_CONV_AUTO) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_conv: the forced kernel family %d does not apply to these views", path);
    }
    if (path != NK_CONV_GENERIC) {
        bool handled = false;
        st = nk_conv_tiled_try(ctx, dtype, drn, v0, src1, v1, src2, v2, d, path != NK_CONV_AUTO, &handled);
        if (st) return st;
        if (handled) return NK_OK;
        if (path != NK_CONV_AUTO) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_conv: the forced kernel family %d does not apply to these views", path);
    }
    ConvPlan c;
    if ((st = nk_conv_make_plan(ctx, v0, v1, v2, d, &c))) return st;
    ctx->last_conv_path = NK_CONV_GENERIC;
    if (dtype == NK_F32) return run_generic<float>(ctx, (float*)drn->ptr, (const float*)src1->ptr, (const float*)src2->ptr, c);
    return run_generic<double>(ctx, (double*)drn->ptr, (const double*)src1->ptr, (const double*)src2->ptr, c);
}
